"""CPU tests: graph tracing / fusion / memory plan / artifacts, the pointwise code generator (render + NVRTC
compile for sm_100a, no GPU needed), the tuning service and its cache, collective tuning votes, doctor + CLI."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from incin_b200 import graph as G
from incin_b200.codegen.pointwise import Arg, Binary, Const, Layout, Scalar, Ternary, Unary, count_args, kernel_key, render_cuda
from incin_b200.tuning import (Candidate, Identity, PersistentCache, TuningPolicy, TuningRecord, TuningService,
                               candidates, prune)
from incin_b200.tuning import collective as C


def _fn(x, w, b):
    h = torch.relu(x @ w + b)
    h = torch.tanh(h * 2.0)
    return h.sum()


def test_trace_records_ops_and_io():
    x, w, b = torch.randn(8, 16), torch.randn(16, 32), torch.randn(8, 32)
    g = G.trace(_fn, x, w, b)
    ops = [n.op for n in g.nodes]
    assert ops[:3] == ["input"] * 3 and "mm" in ops and ops[-1] == "sum"
    assert len(g.inputs) == 3 and g.outputs == [g.nodes[-1].id]
    assert G.tracing_graph_snapshot() is g
    assert g.digest() == G.trace(_fn, x, w, b).digest()
    assert g.digest() != G.trace(_fn, x[:4], w, b[:4]).digest()


def test_fusion_groups_pointwise_chain_and_lowers_to_one_kernel():
    x, w, b = torch.randn(8, 16), torch.randn(16, 32), torch.randn(8, 32)
    g = G.trace(_fn, x, w, b)
    groups = G.fusion_pass(g)
    assert len(groups) == 1 and [g.nodes[i].op for i in groups[0].nodes] == ["add", "relu", "mul", "tanh"]
    expr, ext = G.lower_group(g, groups[0])
    assert len(ext) == 2 and count_args(expr) == (2, 0)
    src, key = render_cuda(expr, "f32")
    assert "tanhf" in src and "fmaxf" in src and key.entry in src


def test_fusion_stops_at_fanout():
    def f(x):
        a = torch.relu(x)
        return a * 2.0 + torch.exp(a)   # relu has two consumers: it ends its group
    g = G.trace(f, torch.randn(4, 4))
    for grp in G.fusion_pass(g):
        assert all(g.nodes[i].op != "relu" or i == grp.nodes[-1] for i in grp.nodes)


def test_memory_plan_reuses_dead_buffers_without_overlap():
    x, w, b = torch.randn(64, 64), torch.randn(64, 64), torch.randn(64, 64)
    g = G.trace(_fn, x, w, b)
    mp = G.plan_memory(g)
    assert mp.peak_bytes < mp.naive_bytes
    live = G.liveness(g)
    ids = list(mp.offsets)
    size = {n.id: max(256, (torch.Size(n.shape).numel() * 4 + 255) // 256 * 256) for n in g.nodes}
    for i in ids:
        for j in ids:
            if i < j and not (live[i][1] < live[j][0] or live[j][1] < live[i][0]):
                a0, b0 = mp.offsets[i], mp.offsets[j]
                assert a0 + size[i] <= b0 or b0 + size[j] <= a0, (i, j)


def test_compiled_plan_guard_and_artifact_roundtrip(tmp_path):
    x, w, b = torch.randn(8, 16), torch.randn(16, 32), torch.randn(8, 32)
    plan = G.CompiledPlan.build(_fn, x, w, b)
    assert plan.guard.admits(x, w, b) and not plan.guard.admits(x[:4], w, b[:4])
    assert not plan.guard.admits(x.double(), w, b)
    p = tmp_path / "plan.bin"
    G.write_artifact(p, plan)
    back = G.read_artifact(p)
    assert back["plan"]["graph_digest"] == plan.graph_digest and back["manifest"]["arch"] == "sm_100a"
    raw = bytearray(p.read_bytes())
    raw[-3] ^= 0x40
    p.write_bytes(bytes(raw))
    with pytest.raises(ValueError, match="checksum"):
        G.read_artifact(p)
    p.write_bytes(b"garbage!" + bytes(raw[8:]))
    with pytest.raises(ValueError, match="not a compiled"):
        G.read_artifact(p)


def test_shape_buckets():
    assert [G.shape_bucket(n) for n in (1, 64, 65, 128, 1000)] == [64, 64, 128, 128, 1024]


# ------------------------------------------------------------------------------------------------ codegen
def test_wgsl_and_msl_text_emitters_cover_every_op():
    """Substring checks, as the reference tests its shader emitters (crates/incin-backends/src/codegen/pointwise.rs:342-499)."""
    from incin_b200.codegen import pointwise as PW
    from incin_b200.codegen.shading import _BINARY, _TERNARY, _UNARY, render_msl, render_wgsl
    assert set(_UNARY) == set(PW.UNARY) and set(_BINARY) == set(PW.BINARY) and set(_TERNARY) == set(PW.TERNARY)
    e = Ternary("fma", Unary("gelu_tanh", Arg(0)), Scalar(0), Binary("max", Arg(1), Const(0.5)))
    w = render_wgsl(e, "f32", workgroup_size=64)
    assert "@group(0) @binding(0) var<storage, read> in0: array<f32>;" in w
    assert "@group(0) @binding(2) var<storage, read_write> out_data: array<f32>;" in w
    assert "@compute @workgroup_size(64, 1, 1)" in w and "if (idx >= arrayLength(&out_data)) { return; }" in w
    assert "fma((0.5 * val0 * (1.0 + tanh(0.79788456 * (val0 + 0.044715 * val0 * val0 * val0)))), scalars.s0, max(val1, 0.5))" in w
    assert "var<uniform> scalars: Scalars;" in w
    m = render_msl(e, "bf16", name="fused0")
    assert "kernel void fused0(" in m and "device const half* in1 [[buffer(1)]]," in m and "device half* out_data [[buffer(2)]]," in m
    assert "uint idx [[thread_position_in_grid]]" in m and "fmax(val1, 0.5f)" in m and "static_cast<half>(" in m
    assert "enable f16;" in render_wgsl(Unary("rsqrt", Arg(0)), "f16") and "inverseSqrt(val0)" in render_wgsl(Unary("rsqrt", Arg(0)))
    assert "let val1 = f32(in1[0]);" in render_wgsl(Binary("add", Arg(0), Arg(1)), scalar_broadcast=1)
    for op in PW.UNARY:
        assert "val0" in render_wgsl(Unary(op, Arg(0))) and "val0" in render_msl(Unary(op, Arg(0)))
    with pytest.raises(ValueError):
        render_wgsl(Const(float("inf")) + Arg(0))


def test_render_every_op_and_reject_bad_trees():
    e = Ternary("fma", Unary("gelu_tanh", Arg(0)), Scalar(0), Binary("max", Arg(1), Const(0.5)))
    assert count_args(e) == (2, 1)
    for dt in ("f32", "bf16", "f16"):
        for lay in (Layout.CONTIGUOUS, Layout.STRIDED):
            src, key = render_cuda(e, dt, lay)
            assert key.entry in src and "fmaf" in src
    assert kernel_key(e, "bf16", Layout.CONTIGUOUS) == kernel_key(e, "bf16", Layout.CONTIGUOUS)
    assert kernel_key(e, "bf16", Layout.CONTIGUOUS) != kernel_key(e, "f16", Layout.CONTIGUOUS)
    with pytest.raises(ValueError):
        Unary("nope", Arg(0))
    assert count_args(Binary("add", Arg(0), Arg(2))) == (3, 0)   # an unused input still takes a slot


def test_nvrtc_compiles_generated_kernel_for_sm100a():
    rt = pytest.importorskip("incin_b200.codegen.runtime")
    e = Binary("mul", Unary("swish", Arg(0)), Arg(1))
    for dt in ("bf16", "f32"):
        for lay in (Layout.CONTIGUOUS, Layout.STRIDED):
            src, key = render_cuda(e, dt, lay)
            cubin = rt.nvrtc_compile(src, key.entry + ".cu")
            assert cubin[:4] == b"\x7fELF" and len(cubin) > 1000
    with pytest.raises(rt.CompileError):
        rt.nvrtc_compile("__global__ void k() { this is not C++; }")


# ------------------------------------------------------------------------------------------------ tuning
def test_candidates_and_pruning():
    cs = candidates(block=[128, 256], vec=[1, 4])
    assert len(cs) == 4 and cs[0].as_dict() == {"block": 128, "vec": 1}
    kept = prune(cs, {"n": 130}, [lambda c, s: s["n"] % c["vec"] == 0 or c["vec"] == 1])
    assert [c.as_dict()["vec"] for c in kept] == [1, 1]


def test_service_policies_measure_cache_and_persist(tmp_path):
    ident = Identity("B200", "sm_100a", "12.9", "0.1.0")
    cache = PersistentCache(tmp_path / "tune.json")
    cs = candidates(tile=[64, 128, 256])
    calls = []

    def measure(p):
        calls.append(p["tile"])
        return {64: 3.0, 128: 1.0, 256: 2.0}[p["tile"]]
    heur = lambda: {"tile": 64}
    assert TuningService(TuningPolicy.DISABLED, cache, ident).choose("k", cs, heur, measure) == {"tile": 64}
    assert TuningService(TuningPolicy.HEURISTIC, cache, ident).choose("k", cs, heur, measure) == {"tile": 64}
    assert calls == []
    svc = TuningService(TuningPolicy.PROFILE_GUIDED, cache, ident)
    assert svc.choose("k", cs, heur, measure) == {"tile": 128} and calls == [64, 128, 256]
    assert svc.choose("k", cs, heur, measure) == {"tile": 128} and len(calls) == 3      # LRU hit
    assert "tile=128" in svc.explain() or "128" in svc.explain()
    # a new process with the same identity reads the record from disk; another identity ignores it
    assert TuningService(TuningPolicy.HEURISTIC, PersistentCache(tmp_path / "tune.json"), ident).choose("k", cs, heur) == {"tile": 128}
    other = Identity("H100", "sm_90a", "12.9", "0.1.0")
    assert TuningService(TuningPolicy.HEURISTIC, PersistentCache(tmp_path / "tune.json"), other).choose("k", cs, heur) == {"tile": 64}
    # warm-up policy measures only until end_warmup()
    w = TuningService(TuningPolicy.COORDINATED_WARMUP, None, ident)
    w.end_warmup()
    assert w.choose("k2", cs, heur, measure) == {"tile": 64}


def test_corrupt_cache_file_is_ignored(tmp_path):
    p = tmp_path / "tune.json"
    ident = Identity("B200", "sm_100a", "12.9", "0.1.0")
    c = PersistentCache(p)
    c.store(TuningRecord("k", ident.token(), {"tile": 128}, 1.0))
    assert [r.key for r in PersistentCache(p).load().values()] == ["k"]
    p.write_text(p.read_text().replace("128", "256", 1))
    assert PersistentCache(p).load() == {}


def test_failing_candidate_is_skipped():
    svc = TuningService(TuningPolicy.PROFILE_GUIDED, None, Identity("B200", "sm_100a", "12.9", "0.1.0"))

    def measure(p):
        if p["tile"] == 128:
            raise RuntimeError("cannot launch")
        return float(p["tile"])
    assert svc.choose("k", candidates(tile=[128, 64, 256]), lambda: {"tile": 1}, measure) == {"tile": 64}


def test_collective_tuning_commit_needs_agreement():
    reports = [C.SampleReport(r, c, s) for r in range(2) for c, s in (("a", (10, 12, 11)), ("b", (7 + 10 * r, 8, 9)))]
    sc = C.score(reports)
    assert sc["a"] == 11 and sc["b"] == 9    # max over ranks per sample, then median
    votes = [C.local_vote(r, reports) for r in range(2)]
    out = C.commit(2, reports, votes)
    assert out.candidate == "b" and out.world == 2
    with pytest.raises(C.TuningDisagreement):
        C.commit(2, reports, [C.CommitVote(0, "a"), C.CommitVote(1, "b")])
    with pytest.raises(C.TuningDisagreement):
        C.commit(3, reports, votes)
    with pytest.raises(C.TuningDisagreement):
        C.commit(2, reports, [C.CommitVote(0, "zz"), C.CommitVote(1, "zz")])


# ------------------------------------------------------------------------------------------------ doctor / CLI
class _FakeHost:
    def __init__(self, devices, tools=None, libs=None):
        self._d, self._t, self._l = devices, tools or {"nvcc": "/usr/local/cuda/bin/nvcc"}, libs or {}

    def python(self): return "3.12.3"
    def torch_version(self): return "2.11.0"
    def cuda_devices(self): return self._d
    def tools(self): return self._t
    def libraries(self): return self._l


def _dev(i, arch="sm_100", peers=()):
    return {"index": i, "name": "NVIDIA B200" if arch == "sm_100" else "NVIDIA H100", "arch": arch, "sms": 148,
            "memory_gib": 178.4, "peers": list(peers)}


def test_doctor_reports_against_fake_hosts():
    from incin_b200.doctor import doctor
    libs = {"libincin_sm100.so": True, "libincin_host.so": True}
    good = doctor(_FakeHost([_dev(0, peers=[1]), _dev(1, peers=[0])], libs=libs))
    assert good.healthy and "B200" in good.to_text() and good.findings[0].code == "all-good"
    none = doctor(_FakeHost([], libs=libs))
    assert none.healthy and "no CUDA device" in none.to_text() and json.loads(none.to_json())["healthy"]
    old = doctor(_FakeHost([_dev(0, "sm_90")], libs=libs))
    assert not old.healthy and old.findings[0].code == "arch-unsupported"
    unbuilt = doctor(_FakeHost([_dev(0)], libs={}))
    assert {f.code for f in unbuilt.findings} >= {"native-missing", "host-missing"}
    lonely = doctor(_FakeHost([_dev(0), _dev(1, peers=[0])], tools={"nvcc": None}, libs=libs))
    assert {f.code for f in lonely.findings} == {"peer-access", "nvcc-missing"} and lonely.healthy


def test_cli_subcommands_run():
    def run(*a):
        r = subprocess.run([sys.executable, "-m", "incin_b200", *a], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-800:]
        return r.stdout
    assert "sm_100a" in run("capabilities") or "tcgen05" in run("capabilities")
    out = run("plan", "--world", "8")
    assert "chosen" in out and "dp=8" in out
    assert run("doctor", "--json").lstrip().startswith("{")


# ------------------------------------------------------------------------------------------------ ffi / budgets / misc
def test_rust_bindings_match_the_c_headers():
    from pathlib import Path
    from incin_b200 import ffi
    structs, funcs = ffi.parse_headers()
    assert {s.name for s in structs} >= {"incin_gemm_desc", "incin_attn_desc", "incin_dp_desc", "incin_conv_geom"}
    names = {f.name for f in funcs}
    assert {"incin_gemm_bf16", "incin_flash_attn_fwd", "incin_dp_reduce_adamw", "incin_peer_barrier", "incin_coll_reduce",
            "incin_layernorm_bwd_noalloc", "incin_rdv_connect", "incin_cpu_mlp_train"} <= names
    committed = (Path(ffi.__file__).resolve().parent.parent / "rust" / "incin-b200-sys" / "src" / "lib.rs").read_text()
    assert committed == ffi.render_rust(), "run `python -m incin_b200 ffi --write` after changing a header"
    gemm = next(s for s in structs if s.name == "incin_gemm_desc")
    from incin_b200._native import GemmDesc
    assert [f[0] for f in gemm.fields] == [n for n, _ in GemmDesc._fields_]      # ctypes mirror has the same layout


def test_budget_check(tmp_path):
    from incin_b200.budgets import check_bench, feature_table, load_budgets
    floor = load_budgets()["entries"]["gpt2-small/n1"]["value"]        # a result at the recorded floor passes
    good = tmp_path / "b.json"
    good.write_text('noise\n{"value": %.1f, "unit": "tokens/s", "n_gpus": 1, "higher_is_better": true, "config": {"model": "gpt2-small"}}\n' % floor)
    assert check_bench(good)[0]
    bad = tmp_path / "c.json"
    bad.write_text('{"value": 300000.0, "unit": "tokens/s", "n_gpus": 1, "higher_is_better": true, "config": {"model": "gpt2-small"}}')
    ok, rep = check_bench(bad)
    assert not ok and "REGRESSION" in rep
    assert check_bench(tmp_path / "b.json", None)[1].startswith("gpt2-small/n1")
    assert "| matmul |" in feature_table()


def test_backends_dispatch_dummy_and_conformance():
    from incin_b200.backends import BackendUnavailable, CpuBackend, DispatchBackend, DummyBackend, run_conformance
    res = run_conformance(CpuBackend())
    assert res and all(r.status == "passed" for r in res), [r for r in res if r.status != "passed"]
    d = DummyBackend()
    assert d.run("matmul", torch.empty(4, 8), torch.empty(8, 16)).shape == (4, 16)
    assert d.run("matmul", torch.empty(4, 8), torch.empty(8, 16)).device.type == "meta"
    disp = DispatchBackend()
    assert float(disp.run("sum", torch.ones(3, 3))) == 9.0
    with pytest.raises(BackendUnavailable):
        disp.backend_for(torch.empty(2, device="meta"))

    class Claimless(CpuBackend):       # a subject that claims nothing is skipped everywhere, not failed
        def supports(self, op, dtype):
            from incin_b200.core.spec import SupportLevel
            return SupportLevel.UNSUPPORTED
    assert all(r.status == "skipped" for r in run_conformance(Claimless()))
    # an external library behind the same contract: what it claims must pass, what it does not claim is skipped
    from incin_b200.backends import NumpyBackend
    ext = run_conformance(NumpyBackend())
    by = {s: [r for r in ext if r.status == s] for s in ("passed", "failed", "skipped")}
    assert not by["failed"], by["failed"]
    assert len(by["passed"]) >= 20 and all(r.dtype == "f32" for r in by["passed"])
    assert {r.op for r in by["skipped"]} >= {"conv2d", "max_pool2d"} and any(r.dtype == "bf16" for r in by["skipped"])
    assert len({r.op for r in res}) >= 25                                      # case families of the suite


def test_iteration_plans_collapse_broadcast_and_bounds():
    from incin_b200.core.iteration import IterationError, check_bounds, plan, unary_plan
    from incin_b200.core.spec import LayoutClass, TensorMeta
    a, b, o = torch.empty(4, 1, 8), torch.empty(3, 8), torch.empty(4, 3, 8)
    p = plan([TensorMeta.of(a), TensorMeta.of(b)], TensorMeta.of(o))
    assert p.shape == (4, 3, 8) and p.operands[0].strides == (8, 0, 1) and p.operands[1].strides == (0, 8, 1)
    assert p.layout is LayoutClass.BROADCAST
    x = torch.empty(6, 10, 7)
    assert unary_plan(TensorMeta.of(x), TensorMeta.of(torch.empty(6, 10, 7))).shape == (420,)     # fully collapsed
    pt = plan([TensorMeta.of(x.transpose(0, 1))], TensorMeta.of(torch.empty(10, 6, 7)))
    assert pt.layout is LayoutClass.STRIDED and pt.operands[0].strides == (7, 70, 1)
    check_bounds(pt, [420, 420])
    with pytest.raises(IterationError):
        check_bounds(pt, [400, 420])
    with pytest.raises(IterationError):
        plan([TensorMeta.of(torch.empty(5, 8))], TensorMeta.of(torch.empty(4, 8)))
    s = plan([TensorMeta.of(torch.empty(1)), TensorMeta.of(x)], TensorMeta.of(torch.empty(6, 10, 7)))
    assert s.layout is LayoutClass.SCALAR


def test_onnx_roundtrip_and_diagnostics(tmp_path):
    from torch import nn
    from incin_b200.diagnostics import explain, humanize
    from incin_b200.io import onnx as O
    m = nn.Sequential(nn.Flatten(), nn.Linear(784, 64), nn.ReLU(), nn.Dropout(0.1), nn.LayerNorm(64), nn.Linear(64, 10, bias=False),
                      nn.Softmax(-1)).eval()
    p = tmp_path / "m.onnx"
    g = O.export_module(m, (4, 1, 28, 28), p)
    assert [n.op_type for n in g.nodes] == ["Flatten", "Gemm", "Relu", "Identity", "LayerNormalization", "Gemm", "Softmax"]
    back = O.import_model(p)
    x = torch.randn(4, 1, 28, 28)
    torch.testing.assert_close(back.run(x)[0], m(x))
    torch.testing.assert_close(back.to_module().eval()(x), m(x))
    assert back.inputs == [("input", (4, 1, 28, 28))] and back.outputs[0][1] == (4, 10)
    p.write_bytes(p.read_bytes()[:1000])
    with pytest.raises(ValueError):
        O.import_model(p)
    with pytest.raises(RuntimeError, match="looks transposed"):
        with humanize():
            torch.randn(3, 4) @ torch.randn(5, 4)
    assert "not divisible" in str(explain("shape '[3, -1, 5]' is invalid for input of size 32"))
    assert explain("something else entirely") is None


def test_tensor_creation_is_seeded_and_graph_passes():
    from incin_b200 import graph as G
    from incin_b200 import tensor as Tn
    Tn.manual_seed(7)
    a = Tn.randn(4, 5)
    Tn.manual_seed(7)
    assert torch.equal(a, Tn.randn(4, 5)) and not torch.equal(a, Tn.randn(4, 5))
    assert abs(float(Tn.rand(4000).mean()) - 0.5) < 0.03 and Tn.to_vec1(Tn.arange(4)) == [0, 1, 2, 3]
    x = torch.randn(2, 8, 4, 4)
    torch.testing.assert_close(Tn.group_norm(x, 4), torch.nn.functional.group_norm(x, 4), rtol=1e-4, atol=1e-5)
    g = G.trace(lambda x, w: x @ w + (w * 2.0).sum(), torch.randn(3, 4), torch.randn(4, 5))
    assert [g.nodes[i].op for i in G.constant_fold(g, {1})] == ["mul", "sum"]
    assert list(G.weight_prepack_plan(g, {1})) == [1]


def test_translate_command_and_shape_error_parsers(capsys):
    """`translate` explains a pasted error: every parser is fed the message PyTorch really raises for its case."""
    import torch.nn.functional as TF
    from incin_b200.__main__ import main
    from incin_b200.diagnostics import RULES, explain, translate
    cases = {
        "axis": lambda: torch.zeros(2, 3).transpose(0, 3),
        "slice": lambda: torch.zeros(12).narrow(0, 5, 10),
        "pool2d": lambda: TF.max_pool2d(torch.zeros(1, 3, 2, 2), 3),
        "conv2d": lambda: TF.conv2d(torch.zeros(1, 1, 2, 2), torch.zeros(1, 1, 3, 3)),
        "stack": lambda: torch.stack([torch.zeros(2, 3), torch.zeros(2, 4)]),
        "matmul": lambda: torch.zeros(4, 8) @ torch.zeros(16, 8),
        "concat": lambda: torch.cat([torch.zeros(2, 3), torch.zeros(3, 4)], 1),
    }
    for op, fn in cases.items():
        with pytest.raises(Exception) as ei:
            fn()
        d = explain(str(ei.value))
        assert d is not None and d.op == op and op in RULES, (op, str(ei.value))
    assert "[5, 15)" in translate("start (5) + length (10) exceeds dimension size (12).")
    assert translate("nothing to see here") == "nothing to see here"
    msg = "mat1 and mat2 shapes cannot be multiplied (4x8 and 16x8)"
    assert main(["translate", "--explain", msg]) == 0
    out = capsys.readouterr().out
    assert "looks transposed" in out and "rule:" in out
    assert main(["translate", "--raw", msg]) == 0
    assert capsys.readouterr().out.strip() == msg


def test_cli_run_passthrough_explains_shape_errors(tmp_path, capsys):
    from incin_b200.__main__ import main
    bad = tmp_path / "bad.py"
    bad.write_text("import sys, torch\nprint('args', sys.argv[1:])\ntorch.zeros(4, 8) @ torch.zeros(16, 8)\n")
    assert main(["run", str(bad), "--flag", "1"]) == 1
    cap = capsys.readouterr()
    assert "args ['--flag', '1']" in cap.out and "[matmul]" in cap.err and "looks transposed" in cap.err
    good = tmp_path / "good.py"
    good.write_text("print('fine')\n")
    assert main(["run", str(good)]) == 0


def test_capability_document_matches_the_registries():
    """docs/capabilities.md is generated: a change of the registries without regenerating it fails here."""
    from pathlib import Path
    from incin_b200.__main__ import CAPABILITIES_HEADER
    from incin_b200.doctor import capability_report
    doc = Path(__file__).resolve().parent.parent / "docs" / "capabilities.md"
    assert doc.read_text() == CAPABILITIES_HEADER + capability_report(), \
        "run `python -m incin_b200 capabilities --write` after changing incin_b200/core/spec.py"


def test_trace_summary_and_hook_install(tmp_path):
    """The launch hook is installed only while tracing is on; summaries group rows by launch name and the JSONL record
    carries the totals."""
    import json
    from incin_b200 import _native
    from incin_b200.telemetry import trace
    assert _native.LAUNCH_HOOK is None
    trace.enable(nvtx=False, events=True)
    assert _native.LAUNCH_HOOK is trace.on_launch
    trace.enable(events=False)
    assert _native.LAUNCH_HOOK is None and not trace.active()
    rows = [("gemm", 0.5), ("norm", 0.1), ("gemm", 0.25), ("adamw", 0.15)]
    top = trace.summary(rows)
    assert [r["name"] for r in top] == ["gemm", "adamw", "norm"]
    assert top[0] == {"name": "gemm", "calls": 2, "ms": 0.75, "share": 0.75}
    trace.to_jsonl(tmp_path / "t.jsonl", rows, step=3)
    rec = json.loads((tmp_path / "t.jsonl").read_text())
    assert rec["step"] == 3 and rec["launches"] == 4 and abs(rec["total_ms"] - 1.0) < 1e-9
    with trace.op_range("anything"):   # off: a plain no-op, also without a GPU
        pass


def _viz_run(tmp_path):
    from incin_b200 import telemetry as T
    p = tmp_path / "run.jsonl"
    evs = [T.Event("hyperparam", "lr", None, None, {"value": 3e-4}, ts=100.0)]
    for i in range(40):
        evs.append(T.Event("scalar", "loss", 4.0 / (i + 1), i + 1, ts=100.0 + i))
        evs.append(T.Event("scalar", "tokens_per_s", 7e5 + i, i + 1, ts=100.0 + i))
        evs.append(T.Event("gradient_norm", "wte", 2.0 - i * 0.01, i + 1, ts=100.0 + i))
        evs.append(T.Event("weight_norm", "wte", 30.0, i + 1, ts=100.0 + i))
    evs.append(T.Event("gradient_norm", "lm_head", float("inf"), 41, ts=141.0))
    evs.append(T.Event("memory", "memory", None, 40, {"rss_bytes": 512 * 2**20, "cuda_allocated": 3 * 2**30}, ts=141.0))
    evs.append(T.Event("graph_snapshot", "graph", None, 40, {"nodes": [
        {"id": 0, "op": "input", "inputs": [], "shape": [4, 8], "dtype": "bf16"},
        {"id": 1, "op": "matmul", "inputs": [0, 0], "shape": [4, 4], "dtype": "bf16"},
        {"id": 2, "op": "relu", "inputs": [1], "shape": [4, 4], "dtype": "bf16"}]}, ts=141.0))
    evs.append(T.Event("epoch", "epoch", 1.0, None, {"steps": 40}, ts=142.0))
    p.write_text("".join(e.to_json() + "\n" for e in evs))
    return p, evs


def test_viz_panels_render_every_event_kind(tmp_path):
    from incin_b200.telemetry import viz
    p, evs = _viz_run(tmp_path)
    frame = viz.render(p, 140, 48)
    assert "step 40" in frame and "best 0.1" in frame                      # loss panel
    assert "tokens_per_s" in frame                                          # scalars
    assert "NON-FINITE" in frame and "wte" in frame                         # norms: the inf gradient is flagged
    assert "3072.0 MiB" in frame and "epochs 1" in frame and "0.0003" in frame   # system
    assert "3 nodes @ step 40" in frame and "matmul" in frame and "%0,%0" in frame  # graph
    assert all(len(line) <= 140 for line in frame.splitlines()) and len(frame.splitlines()) <= 48
    # the same panels fit a small terminal and a stacked layout without raising
    app = viz.App()
    app.feed(evs)
    app.on_key("t")
    small = app.render(60, 16).to_text()
    assert not app.failed and "loss" in small
    assert "\033[1m" in app.render(80, 24).to_ansi()


def test_viz_focus_keymap_plugin_and_failure_isolation(tmp_path):
    from incin_b200.telemetry import viz
    p, evs = _viz_run(tmp_path)

    class Counter(viz.Panel):
        id, title = "counter", "event counter"
        def __init__(self):
            self.n, self.keys, self.explode = 0, [], False
        def update(self, e):
            self.n += 1
        def render(self, canvas, area):
            if self.explode:
                raise RuntimeError("boom")
            canvas.text(area, 0, 0, f"seen {self.n} events " + "x" * 500)       # clipped to the tile
        def handle_key(self, key):
            self.keys.append(key)
            return True
        def reset(self):
            self.n, self.explode = 0, False

    class Bundle(viz.Plugin):
        def panels(self):
            return [Counter()]

    app = viz.App(plugins=[Bundle()])
    assert [q.id for q in app.panels] == ["loss", "scalars", "norms", "system", "graph", "counter"]
    with pytest.raises(ValueError):
        viz.App(plugins=[Bundle(), Bundle()])                                # duplicate ids are refused
    app.feed(evs)
    counter = app.panels[-1]
    assert counter.n == len(evs) and f"seen {len(evs)} events" in app.render(120, 40).to_text()
    # focus: grid of two columns
    assert app.focus == 0
    app.on_key("l"); assert app.focus == 1
    app.on_key("j"); assert app.focus == 3
    app.on_key("h"); assert app.focus == 2
    app.on_key("k"); assert app.focus == 0
    app.on_key("k"); assert app.focus == 0                                   # no wrap at the edge
    app.on_key("\x1b[Z"); assert app.focus == 5                              # Shift-Tab wraps
    assert app.on_key("z") is viz.Action.PANEL_LOCAL and counter.keys == ["z"]
    # a failing panel is fenced off, the others keep rendering, retry brings it back with the run replayed
    counter.explode = True
    frame = app.render(120, 40).to_text()
    assert "[failed]" in frame and "RuntimeError: boom" in frame and "step 40" in frame and "xxxx" not in frame
    app.feed(evs[:3])
    assert counter.n == len(evs)                                             # fenced off: no more updates
    app.on_key("r")
    assert "counter" not in app.failed and counter.n == len(evs) + 3
    assert f"seen {len(evs) + 3} events" in app.render(120, 40).to_text()
    # graph panel keys scroll the node list
    g = app.panels[4]
    app.focus = 4
    app.on_key("G"); assert g.scroll == 2
    app.on_key("0"); assert g.scroll == 0
    assert '"op": "matmul"' in g.hover_text(0, 3)
    # keymap file: rebinding drops the default key of that action; unknown actions are an error
    f = tmp_path / "incin-viz.toml"
    f.write_text('[keymap]\nquit = ["x", "esc"]\ntoggle_layout = "space"\n')
    km = viz.Keymap.from_toml(f)
    assert km.resolve("x") is viz.Action.QUIT and km.resolve("\x1b") is viz.Action.QUIT
    assert km.resolve("q") is viz.Action.PANEL_LOCAL and km.resolve(" ") is viz.Action.TOGGLE_LAYOUT
    f.write_text('[keymap]\nquitt = "x"\n')
    with pytest.raises(ValueError, match="unknown action"):
        viz.Keymap.from_toml(f)
    app2 = viz.App(keymap=km)
    app2.on_key("x")
    assert not app2.running


def test_viz_tail_follows_a_growing_file_and_a_restart(tmp_path, monkeypatch):
    import sys
    import types
    from incin_b200 import telemetry as T
    from incin_b200.telemetry import viz
    p = tmp_path / "live.jsonl"
    tail = viz.RunTail(p)
    assert tail.poll() == []                                                  # not there yet
    a = T.Event("scalar", "loss", 2.0, 1).to_json()
    b = T.Event("scalar", "loss", 1.0, 2).to_json()
    p.write_text(a + "\n" + b[:10])
    assert [e.value for e in tail.poll()] == [2.0]                            # the torn line waits
    with open(p, "a") as f:
        f.write(b[10:] + "\nnot json\n")
    assert [e.value for e in tail.poll()] == [1.0] and tail.poll() == []
    p.write_text(a + "\n")                                                    # a new run under the same name
    assert [e.value for e in tail.poll()] == [2.0] and tail.restarted
    # plug-ins named in the environment are loaded by the one-frame renderer
    mod = types.ModuleType("viz_test_plugin")

    class P(viz.Panel):
        id, title = "extra", "extra panel"
        def update(self, e): pass
        def render(self, canvas, area): canvas.text(area, 0, 0, "hello from a plug-in")

    class Pl(viz.Plugin):
        def panels(self): return [P()]
    mod.make = Pl
    monkeypatch.setitem(sys.modules, "viz_test_plugin", mod)
    monkeypatch.setenv("INCIN_VIZ_PLUGINS", "viz_test_plugin:make")
    assert "hello from a plug-in" in viz.render(p)
    viz.watch(p, interval=0.0, iterations=2)                                  # not a terminal: prints frames and returns


def test_xtask_ledger_is_sound_and_detects_drift(tmp_path):
    """The committed ledger passes; each kind of damage is reported."""
    import copy
    from incin_b200 import xtask
    assert xtask.check_ledger() == []
    assert xtask.docs(check=True) == []                                        # every generated document is current
    good = xtask.load_ledger()
    table = xtask.render_table(good)
    assert "| K1 | core | kernel | complete |" in table and len(good) >= 60

    def errors(mutate, tbl=None):
        t = copy.deepcopy(good)
        mutate(t)
        return xtask.check_ledger(tasks=t, table=xtask.render_table(t) if tbl is None else tbl)

    assert any("unknown component Z9" in e for e in errors(lambda t: t["K2"]["depends"].append("Z9")))
    assert any("does not exist" in e for e in errors(lambda t: t["K2"]["files"].append("csrc/nope.cu")))
    assert any("without evidence" in e for e in errors(lambda t: t["K5"].update(tests=[])))
    assert any("unknown tier" in e for e in errors(lambda t: t["C1"].update(tier="stable")))
    assert any("without a note" in e for e in errors(lambda t: t["B5"].pop("note")))
    # a core component must not lean on a preview one
    assert any("which is only preview" in e for e in errors(lambda t: t["C1"]["depends"].append("M4")))
    # cycles: K1 -> K2 -> K1
    cyc = errors(lambda t: t["K1"]["depends"].append("K2"))
    assert any(e.startswith("dependency cycle") and "K1" in e and "K2" in e for e in cyc)
    assert xtask.find_cycles({"a": {"depends": ["b"]}, "b": {"depends": ["c"]}, "c": {"depends": []}}) == []
    # the markdown rendering is part of the contract
    assert any("differs from the rendering" in e for e in errors(lambda t: None, tbl=table.replace("complete", "done", 1)))
    assert xtask.main(["ledger"]) == 0 and xtask.main([]) == 2


def test_lsp_proxy_frames_and_rewrites(tmp_path):
    import io
    import json
    import subprocess
    import sys
    from incin_b200 import lsp
    # framing: case-insensitive header, extra headers, back-to-back frames, truncated tail
    buf = io.BytesIO()
    lsp.write_frame(buf, b'{"a":1}')
    buf.write(b"content-length: 2\r\nContent-Type: application/vscode-jsonrpc; charset=utf-8\r\n\r\n{}")
    buf.write(b"Content-Length: 10\r\n\r\n{}")
    buf.seek(0)
    assert lsp.read_frame(buf) == b'{"a":1}' and lsp.read_frame(buf) == b"{}" and lsp.read_frame(buf) is None
    with pytest.raises(ValueError):
        lsp.read_frame(io.BytesIO(b"Content-Length: banana\r\n\r\n"))
    with pytest.raises(ValueError):
        lsp.read_frame(io.BytesIO(b"Content-Length: 99999999999\r\n\r\n"))
    # diagnostics: the recognised message gains the explanation, the other entry and other messages pass through
    err = "mat1 and mat2 shapes cannot be multiplied (4x8 and 16x2)"
    pend = lsp.PendingRequests()
    msg = {"jsonrpc": "2.0", "method": "textDocument/publishDiagnostics",
           "params": {"uri": "file:///x.py", "diagnostics": [{"message": err, "severity": 1}, {"message": "unused import"}]}}
    out = lsp.rewrite_from_server(msg, pend)
    d0, d1 = out["params"]["diagnostics"]
    assert d0["message"].startswith(err) and "hint:" in d0["message"] and "rule:" in d0["message"] and d0["severity"] == 1
    assert d1 == {"message": "unused import"} and msg["params"]["diagnostics"][0]["message"] == err    # input untouched
    assert lsp.rewrite_from_server(out, pend) is None                                # never explained twice
    assert lsp.rewrite_from_server({"jsonrpc": "2.0", "method": "window/logMessage", "params": {"message": err}}, pend) is None
    assert lsp.rewrite_from_server(msg, pend, hints=False) is None
    # hovers: only answers to hover requests that went through the proxy are touched
    answer = {"jsonrpc": "2.0", "id": 7, "result": {"contents": {"kind": "markdown", "value": err}}}
    assert lsp.rewrite_from_server(answer, pend) is None
    pend.observe_outgoing({"jsonrpc": "2.0", "id": 7, "method": "textDocument/hover", "params": {}})
    new = lsp.rewrite_from_server(answer, pend)
    assert "hint:" in new["result"]["contents"]["value"] and new["result"]["contents"]["kind"] == "markdown"
    assert lsp.rewrite_from_server(answer, pend) is None                             # the id was consumed
    # end to end through a child "server" that publishes one diagnostic per request and echoes the rest
    server = tmp_path / "server.py"
    server.write_text(
        "import sys, json\n"
        "sys.path.insert(0, %r)\n"
        "from incin_b200.lsp import read_frame, write_frame\n"
        "while (b := read_frame(sys.stdin.buffer)) is not None:\n"
        "    m = json.loads(b)\n"
        "    if m.get('method') == 'exit': break\n"
        "    write_frame(sys.stdout.buffer, json.dumps({'jsonrpc': '2.0', 'method': 'textDocument/publishDiagnostics',\n"
        "        'params': {'uri': 'u', 'diagnostics': [{'message': m['params']['text']}]}}).encode())\n"
        % str(Path(__file__).resolve().parent.parent))
    req = io.BytesIO()
    lsp.write_frame(req, json.dumps({"jsonrpc": "2.0", "method": "x", "params": {"text": err}}).encode())
    lsp.write_frame(req, json.dumps({"jsonrpc": "2.0", "method": "x", "params": {"text": "fine"}}).encode())
    lsp.write_frame(req, json.dumps({"jsonrpc": "2.0", "method": "exit"}).encode())
    p = subprocess.run([sys.executable, "-m", "incin_b200", "lsp", "--", sys.executable, str(server)], input=req.getvalue(),
                       capture_output=True, timeout=120, cwd=str(Path(__file__).resolve().parent.parent))
    assert p.returncode == 0, p.stderr.decode()[-2000:]
    got = io.BytesIO(p.stdout)
    first, second = json.loads(lsp.read_frame(got)), json.loads(lsp.read_frame(got))
    assert "hint:" in first["params"]["diagnostics"][0]["message"]
    assert second["params"]["diagnostics"][0]["message"] == "fine"


def test_row_chain_fuser_renders_and_compiles_without_a_gpu():
    """pointwise -> row normalisation -> pointwise as ONE kernel: the source carries the whole chain, compiles for
    sm_100a with NVRTC, and malformed chains are refused at render time."""
    from incin_b200.codegen import Col, Norm, reference_rows, render_row_cuda
    from incin_b200.codegen.runtime import nvrtc_compile
    chains = {
        "masked scaled softmax": ("softmax", Arg(0) * Scalar(0) + Col(0), None),
        "log-softmax of a sum": ("log_softmax", Arg(0) + Arg(1), None),
        "residual layer norm with gain and bias": ("layer_norm", Arg(0) + Arg(1), Norm() * Col(0) + Col(1)),
        "gelu of a gained rms norm": ("rms_norm", Arg(0), Unary("gelu", Norm() * Col(0))),
    }
    for name, (kind, pre, post) in chains.items():
        for dt in ("bf16", "f32"):
            src, key = render_row_cuda(kind, pre, post, dt)
            assert key.entry in src and src.count("__global__") == 1, name
            assert len(nvrtc_compile(src, key.entry + ".cu")) > 1000, name
    src, key = render_row_cuda("layer_norm", Arg(0) + Arg(1), Norm() * Col(0) + Col(1), "bf16")
    assert "in1 + base + c" in src and "col1 + c" in src and "rsqrtf" in src and (key.n_args, key.n_cols, key.n_scalars) == (2, 2, 0)
    assert render_row_cuda("softmax", Arg(0) * Scalar(0), None, "bf16")[1] != render_row_cuda("softmax", Arg(0) * Scalar(1), None, "bf16")[1]
    with pytest.raises(ValueError):
        render_row_cuda("softmax", Norm() + Arg(0))                    # the prologue has nothing normalised yet
    with pytest.raises(ValueError):
        render_row_cuda("median", Arg(0))
    with pytest.raises(ValueError):
        render_row_cuda("softmax", Col(0))                             # no row tensor
    # the fp32 oracle of a chain (also the CPU path) agrees with plain PyTorch
    x, r = torch.randn(5, 33), torch.randn(5, 33)
    g, b = torch.rand(33) + 0.5, torch.randn(33)
    got = reference_rows("layer_norm", Arg(0) + Arg(1), [x, r], post=Norm() * Col(0) + Col(1), cols=[g, b])
    assert torch.allclose(got, torch.nn.functional.layer_norm(x + r, (33,), g, b), atol=1e-5)
    got = reference_rows("softmax", Arg(0) * Scalar(0) + Col(0), [x], cols=[b], scalars=[0.25])
    assert torch.allclose(got, torch.softmax(x * 0.25 + b, -1), atol=1e-6)


def test_row_fusion_pass_finds_and_lowers_softmax_chains():
    from incin_b200.codegen import reference_rows

    def f(x, mask, y):
        return torch.softmax(x * 0.5 + mask, -1) * y

    x, mask, y = torch.randn(6, 40), torch.randn(40), torch.randn(6, 40)
    g = G.trace(f, x, mask, y)
    groups = G.row_fusion_pass(g)
    assert len(groups) == 1 and len(groups[0].pre) == 2 and len(groups[0].post) == 1
    kind, pre, post, rows_ext, cols_ext = G.lower_row_group(g, groups[0])
    assert kind == "softmax" and len(rows_ext) == 2 and len(cols_ext) == 1
    by_id = {nid: t for nid, t in zip(g.inputs, (x, mask, y))}
    got = reference_rows(kind, pre, [by_id[i] for i in rows_ext], post=post, cols=[by_id[i] for i in cols_ext])
    assert torch.allclose(got, f(x, mask, y), atol=1e-6)
    # a value that something outside the group also reads stays out of the prologue
    def h(x):
        t = x * 2.0
        return torch.log_softmax(t, -1), t
    g2 = G.trace(h, x)
    assert G.row_fusion_pass(g2) == []
    # a softmax over another axis is not a row op of this pass
    assert G.row_fusion_pass(G.trace(lambda a: torch.softmax(a + 1.0, 0), x)) == []


def test_saved_tensors_extend_liveness_and_bounded_plan_tuner():
    def f(x, w, m):
        h = torch.relu(x @ w)
        p = torch.softmax(h * 0.5 + m, -1)
        return (p * h).sum()

    x, w, m = torch.randn(16, 32), torch.randn(32, 64), torch.randn(64)
    g = G.trace(f, x, w, m)
    saved = G.saved_for_backward(g)
    ops = {n.id: n.op for n in g.nodes}
    relu_id = next(i for i, o in ops.items() if o == "relu")
    sm_id = next(i for i, o in ops.items() if o in ("_softmax", "softmax"))
    assert relu_id in saved and sm_id in saved and g.inputs[0] in saved          # relu / softmax outputs, matmul operands
    plain, kept = G.liveness(g), G.liveness(g, saved)
    assert kept[relu_id][1] == len(g.nodes) >= plain[relu_id][1]
    assert all(kept[i][1] >= plain[i][1] for i in plain)
    assert G.plan_memory(g, saved=saved).peak_bytes >= G.plan_memory(g).peak_bytes   # saved values cannot be reused
    rep = G.BoundedPlanTuner(max_iterations=8, min_speedup_target=1.05).tune_plan(g)
    assert rep.is_bounded and rep.iterations_evaluated <= 8 and rep.tuned_latency_us < rep.baseline_latency_us
    assert rep.best != "baseline" and rep.met_target and abs(rep.speedup_ratio - rep.baseline_latency_us / rep.tuned_latency_us) < 1e-9
    one = G.BoundedPlanTuner(max_iterations=1).tune_plan(g)                          # bound reached before any variant
    assert one.iterations_evaluated == 1 and one.best == "baseline" and one.speedup_ratio == 1.0
    with pytest.raises(ValueError):
        G.BoundedPlanTuner(max_iterations=0)


def test_cli_doc_clippy_and_fix(tmp_path):
    root = str(Path(__file__).resolve().parent.parent)
    run = lambda *a: subprocess.run([sys.executable, "-m", "incin_b200", *a], capture_output=True, text=True, cwd=root, timeout=300)
    d = run("doc", "tensor.from_raw")
    assert d.returncode == 0 and "from_raw" in d.stdout and "Nothing is copied" in d.stdout
    assert run("doc", "no.such.thing").returncode == 1
    clean = run("clippy")                                                  # the package itself is clean
    assert clean.returncode == 0 and "0 finding(s)" in clean.stdout
    bad = tmp_path / "bad.py"
    bad.write_text("def f(x=[]):\n    try:\n        pass\n    except:\n        pass\n")
    c = run("clippy", str(bad))
    assert c.returncode == 1 and "mutable default" in c.stdout and "bare `except:`" in c.stdout and "[fix:" not in c.stdout
    f = run("fix", str(bad))
    assert f.returncode == 1 and "[fix: `except Exception:`]" in f.stdout
    broken = tmp_path / "broken.py"
    broken.write_text("def f(:\n")
    assert "error" in run("clippy", str(broken)).stdout
