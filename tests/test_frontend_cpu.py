"""CPU tests of the front end: shapes, policies, descriptors, nn layers, optimisers and schedulers, checkpoints,
exporters, metrics, distributions, telemetry, data loader, Trainer and the native MLP benchmark."""
import json
import os

import pytest
import torch

from incin_b200 import core, distributions as D, io, metrics as MT, nn, telemetry as T
from incin_b200.core import policy as P, spec as S
from incin_b200.core.shapes import matmul_shape


def test_shapes_named_axes_and_errors():
    B, Sq = core.dim("Batch", "Seq")
    env = {}
    core.s(B, Sq, 768).check(torch.zeros(4, 16, 768), env)
    assert env == {"Batch": 4, "Seq": 16}
    with pytest.raises(core.ShapeError) as e:
        core.s(B, 10).check(torch.zeros(5, 10), env)
    assert e.value.op is core.OperationKind.BIND
    with pytest.raises(core.ShapeError):
        core.broadcast_shapes(core.s(B, 4), core.s(Sq, 4))      # distinct named axes never unify
    assert core.broadcast_shapes((8, 1, 6, 1), (7, 1, 5)).dims == core.s(8, 7, 6, 5).dims
    with pytest.raises(core.ShapeError):
        core.broadcast_shapes((3, 4), (5, 4))
    assert matmul_shape(core.s(B, 16, 32), core.s(32, 8)) == core.s(B, 16, 8)
    with pytest.raises(core.ShapeError):
        matmul_shape((4, 5), (6, 7))
    assert core.reshape_infer(24, (2, -1, 3)) == (2, 4, 3)
    with pytest.raises(core.ShapeError):
        core.reshape_infer(24, (5, -1))
    with pytest.raises(core.ShapeError):
        core.Shape(range(9))                                     # MAX_RANK


def test_broadcast_fuzz_against_torch():
    g = torch.Generator().manual_seed(0)
    for _ in range(200):
        ra, rb = int(torch.randint(0, 5, (1,), generator=g)), int(torch.randint(0, 5, (1,), generator=g))
        a = [int(torch.randint(1, 4, (1,), generator=g)) for _ in range(ra)]
        b = [int(torch.randint(1, 4, (1,), generator=g)) for _ in range(rb)]
        try:
            ref = tuple(torch.broadcast_shapes(tuple(a), tuple(b)))
        except RuntimeError:
            with pytest.raises(core.ShapeError):
                core.broadcast_shapes(a, b)
            continue
        assert tuple(d.size for d in core.broadcast_shapes(a, b).dims) == ref


def test_idx_slicing_is_bounds_checked():
    x = torch.arange(8 * 4 * 40).reshape(8, 4, 40)
    assert core.idx[0:5, ..., 15:30].apply(x).shape == (5, 4, 15)
    assert torch.equal(core.idx[2].apply(x), x[2])
    with pytest.raises(core.ShapeError):
        core.idx[0:9].apply(x)
    with pytest.raises(core.ShapeError):
        core.idx[..., ...]


def test_dtype_and_device():
    assert core.size_bytes(core.DTypeId.Q8_0, 32) == 34 and core.size_bytes(core.DTypeId.Q8_0, 33) == 68
    assert core.size_bytes(core.DTypeId.BF16, 10) == 20
    assert core.from_torch(torch.bfloat16) is core.DTypeId.BF16
    with pytest.raises(TypeError):
        core.to_torch(core.DTypeId.Q8_0)
    assert core.detect_device(core.DevicePreference.DEFAULT) == core.Cpu    # the default backend is always the CPU
    assert len(core.DeviceSet.cuda(range(4))) == 4
    with pytest.raises(ValueError):
        core.DeviceSet([core.Cpu, core.Cuda(0)])
    with pytest.raises(ValueError):
        core.DeviceSet([core.Cuda(1), core.Cuda(1)])


def test_policy_scopes_and_loss_scaling():
    assert P.current_policy().determinism is P.Determinism.PERMITTED
    with P.policy_scope(determinism=P.Determinism.REQUIRED) as outer:
        with P.policy_scope(math=P.MathMode.FAST):
            assert P.current_policy().determinism is P.Determinism.REQUIRED and P.current_policy().math is P.MathMode.FAST
        assert P.current_policy() == outer
    assert P.current_policy() == P.ExecutionPolicy()
    assert P.ExecutionPolicy().cache_key() != P.ExecutionPolicy(math=P.MathMode.FAST).cache_key()
    with P.no_grad():
        assert P.grad_mode() is P.GradMode.DISABLED
    ls = P.LossScaling.dynamic(1024.0, 2.0, 0.5, 3)
    ls.update(True)
    assert ls.scale() == 512.0
    for _ in range(3):
        ls.update(False)
    assert ls.scale() == 1024.0
    tiny = P.LossScaling.dynamic(1.5, 2.0, 0.5, 10)
    tiny.update(True)
    assert tiny.scale() == 1.0                                    # never below 1
    assert P.PrecisionPolicy.mixed_bf16().compute is core.DTypeId.BF16
    assert P.PrecisionPolicy.mixed_f16().loss_scaling.kind == "dynamic"


def test_descriptors_and_capabilities():
    a, b = S.TensorMeta.of(torch.zeros(4, 3, 5)), S.TensorMeta.of(torch.zeros(5, 7))
    v = S.validate(S.MatMulSpec(a, b))
    assert v.output_shape == (4, 3, 7)
    v.audit()
    with pytest.raises(core.ShapeError):
        S.validate(S.MatMulSpec(a, a))
    assert S.validate(S.ReductionSpec(a, S.ReduceOp.MEAN, (0, 2))).output_shape == (3,)
    with pytest.raises(core.ShapeError):
        S.validate(S.ReductionSpec(a, S.ReduceOp.SUM, (1, 1)))
    assert S.TensorMeta.of(torch.zeros(3, 4).t()).layout is S.LayoutClass.STRIDED
    assert S.TensorMeta.of(torch.zeros(3, 4).t()).max_physical_index() == 11
    cuda = S.REGISTRIES[core.DeviceKind.CUDA]
    assert cuda.query(S.CapabilityQuery("matmul", core.DTypeId.BF16, core.DeviceKind.CUDA)).level is S.SupportLevel.NATIVE
    assert not cuda.supports("topk", core.DTypeId.BF16)
    assert "gemm_tcgen05" in S.capability_table_markdown() or "matmul" in S.capability_table_markdown()
    assert S.ProofLevel.STATIC.meet(S.ProofLevel.RANKED) is S.ProofLevel.RANKED


def test_layers_match_torch_and_state_dict_layout():
    nn.manual_seed(0)
    m = nn.seq(nn.Flatten(), nn.Linear(12, 8), nn.GELU(), nn.LayerNorm(8), nn.Linear(8, 3))
    assert [n for n, _ in m.named_parameters()] == ["1.weight", "1.bias", "3.weight", "3.bias", "4.weight", "4.bias"]
    assert sorted(io.state_dict(m))[0] == "1.bias."               # trailing dot, as in incin checkpoints
    assert m[1].weight.shape == (8, 12) and m[1].weight.abs().max() <= 1 / 12 ** 0.5 + 1e-6
    x = torch.randn(5, 3, 4)
    ref = torch.nn.functional.linear(x.flatten(1), m[1].weight, m[1].bias)
    ref = torch.nn.functional.layer_norm(torch.nn.functional.gelu(ref), (8,), m[3].weight, m[3].bias)
    assert torch.allclose(m(x), torch.nn.functional.linear(ref, m[4].weight, m[4].bias), atol=1e-6)
    r = nn.RMSNorm(8)
    z = torch.randn(2, 8)
    assert torch.allclose(r(z), z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + 1e-5), atol=1e-6)
    d = nn.Dropout(0.5, seed=3).train()
    y = d(torch.ones(10000))
    assert abs(float((y == 0).float().mean()) - 0.5) < 0.03 and abs(float(y.mean()) - 1.0) < 0.05
    assert torch.equal(d.eval()(z), z)
    st = nn.ComputeStats.of(m)
    assert st.parameters == 12 * 8 + 8 + 16 + 8 * 3 + 3
    out, (h, c) = nn.LSTM(4, 6)(torch.randn(2, 5, 4))
    assert out.shape == (2, 5, 6) and torch.equal(out[:, -1], h)


def test_flat_optimizers_match_torch_and_schedulers():
    from incin_b200.optim import SGD, AdamW, CosineAnnealingLR, LinearLR, StepLR, make_store
    torch.manual_seed(0)
    m1 = torch.nn.Linear(6, 4)
    m2 = torch.nn.Linear(6, 4)
    m2.load_state_dict(m1.state_dict())
    ref = torch.optim.AdamW(m1.parameters(), lr=1e-2, weight_decay=0.1)
    store = make_store(m2, decay_filter=lambda n, p: True)
    opt = AdamW(store, lr=1e-2, weight_decay=0.1)
    x, y = torch.randn(16, 6), torch.randn(16, 4)
    for _ in range(5):
        ref.zero_grad()
        ((m1(x) - y) ** 2).mean().backward()
        ref.step()
        store.zero_grad()
        ((m2(x) - y) ** 2).mean().backward()
        store.collect_autograd_grads()
        opt.step()
    assert torch.allclose(m1.weight, m2.weight, atol=1e-6) and torch.allclose(m1.bias, m2.bias, atol=1e-6)
    sd = opt.state_dict()
    assert sd["step_count"] == 5 and "m.weight" in sd and "v.bias" in sd
    s2 = SGD(make_store(torch.nn.Linear(2, 2)), lr=0.1)
    lin = LinearLR(s2, 0.0, 1.0, 10)
    assert [round(lin.step(), 3) for _ in range(3)] == [0.01, 0.02, 0.03]
    cos = CosineAnnealingLR(s2, 100, base_lr=1.0)
    assert abs(cos.lr_at(50) - 0.5) < 1e-9 and cos.lr_at(100) == 0.0
    assert StepLR(s2, 10, 0.5, base_lr=1.0).lr_at(25) == 0.25
    st = lin.state_dict()
    lin2 = LinearLR(s2, 0.0, 1.0, 10)
    lin2.load_state_dict(st)
    assert lin2.last_step == 3


def test_checkpoint_roundtrip_resharding_and_limits(tmp_path):
    from incin_b200.optim import AdamW, make_store
    nn.manual_seed(1)
    m = nn.seq(nn.Linear(16, 8), nn.ReLU(), nn.Linear(8, 4))
    opt = AdamW(make_store(m), lr=1e-3)
    m(torch.randn(3, 16)).sum().backward()
    opt.store.collect_autograd_grads()
    opt.step()
    io.save_checkpoint(tmp_path, m, world_size=2, placements={"0.weight": "sharded:0", "2.weight": "sharded:1"},
                       optimizer=opt, trainer_state={"scheduler": {"last_step": 7}})
    man = json.loads((tmp_path / "manifest.json").read_text())
    assert man["world_size"] == 2 and man["tensors"]["0.weight."]["placement_kind"] == "sharded:0"
    m2 = nn.seq(nn.Linear(16, 8), nn.ReLU(), nn.Linear(8, 4))
    opt2 = AdamW(make_store(m2), lr=1e-3)
    extra = io.load_checkpoint(tmp_path, m2, opt2)
    assert torch.equal(m[0].weight, m2[0].weight) and torch.equal(opt.m, opt2.m) and opt2.step_count == 1
    assert extra["scheduler"]["last_step"] == 7
    m3 = nn.seq(nn.Linear(16, 8), nn.ReLU(), nn.Linear(8, 4))
    io.load_checkpoint(tmp_path, m3, threads=3)                     # native threaded readers give the same tensors
    assert torch.equal(m[2].weight, m3[2].weight)
    for world in (2, 4):
        parts = [io.load_resharded_checkpoint(tmp_path, r, world, threads=2 if world == 4 else 0) for r in range(world)]
        assert torch.equal(torch.cat([p["0.weight."] for p in parts], 0), m[0].weight.detach())
        assert torch.equal(torch.cat([p["2.weight."] for p in parts], 1), m[2].weight.detach())
        assert torch.equal(parts[1]["0.bias."], m[0].bias.detach())
    with pytest.raises(ValueError):
        io.slice_bytes_for_rank(b"\0" * 24, [2, 3], core.DTypeId.F32, 1, 0, 2)
    with pytest.raises(io.LimitError):
        io.load_safetensors(tmp_path / "model.safetensors", io.ResourceLimits(max_tensor_count=1))
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes((10 ** 12).to_bytes(8, "little") + b"{}")
    with pytest.raises(io.LimitError):
        io.load_safetensors(bad)


def test_checkpoint_resume_restores_fp32_master_of_flat_optimizer(tmp_path):
    """With a low-precision shadow the optimiser steps from fp32 master weights: a resumed run must get those
    back (not the rounded shadow, not its own fresh initialisation) and then take bit-identical steps."""
    from incin_b200.optim import AdamW, make_store

    def build(seed):
        nn.manual_seed(seed)
        m = nn.seq(nn.Linear(16, 8), nn.ReLU(), nn.Linear(8, 4))
        return m, AdamW(make_store(m, compute_dtype=torch.bfloat16), lr=1e-2)

    def one_step(m, opt, x):
        opt.zero_grad()
        m(x.to(torch.bfloat16)).float().sum().backward()
        opt.store.collect_autograd_grads()
        opt.step()

    x = torch.randn(3, 16)
    m, opt = build(1)
    one_step(m, opt, x)
    io.save_checkpoint(tmp_path, m, optimizer=opt)
    saved = io.load_safetensors(tmp_path / "model.safetensors")
    assert saved["0.weight."].dtype == torch.float32                       # the master, not the bf16 shadow
    m2, opt2 = build(2)                                                    # different initial weights
    io.load_checkpoint(tmp_path, m2, opt2)
    assert torch.equal(opt.store.master, opt2.store.master)
    assert torch.equal(opt.store.shadow, opt2.store.shadow) and torch.equal(m[0].weight, m2[0].weight)
    one_step(m, opt, x)
    one_step(m2, opt2, x)
    assert torch.equal(opt.store.master, opt2.store.master) and torch.equal(m[2].weight, m2[2].weight)


def test_flat_optimizer_hyper_ring_keeps_steps_apart():
    from incin_b200.optim import AdamW, make_store
    nn.manual_seed(0)
    m = nn.seq(nn.Linear(4, 4))
    opt = AdamW(make_store(m), lr=1.0)
    seen = []
    for step in range(1, 2 * opt.HYPER_RING + 2):
        opt.set_lr(1.0 / step)
        opt.prepare_step()
        seen.append(opt._hyper_host)
        assert float(opt.hyper[5]) == step and abs(float(opt.hyper[0]) - 1.0 / step) < 1e-7
    assert len({id(h) for h in seen[:opt.HYPER_RING]}) == opt.HYPER_RING   # consecutive steps never share a slot


def test_safetensors_malformed_headers_raise_limit_error(tmp_path):
    import struct

    def write(header: bytes, payload: bytes = b""):
        p = tmp_path / "m.safetensors"
        p.write_bytes(struct.pack("<Q", len(header)) + header + payload)
        return p

    cases = [
        b'{"a": 3}',                                                              # entry is not an object
        b'{"a": {"dtype": "F32", "shape": [2]}}',                                 # missing offsets
        b'{"a": {"dtype": "F32", "shape": [-1, -4], "data_offsets": [0, 16]}}',   # negative dims (numel 4 would match)
        b'{"a": {"dtype": "F32", "shape": [1.5], "data_offsets": [0, 4]}}',       # non-integer dim
        b'{"a": {"dtype": "F32", "shape": "x", "data_offsets": [0, 4]}}',
        b'{"a": {"dtype": 7, "shape": [1], "data_offsets": [0, 4]}}',
        b'{"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, "4"]}}',
        b'{"__metadata__": [1, 2]}',
        b'{not json',
    ]
    for h in cases:
        with pytest.raises(io.LimitError):
            io.load_safetensors(write(h, b"\0" * 16))


def test_exporters_and_quantisation(tmp_path):
    from incin_b200.ops.quant import dequantize_q8_0, quantize_q8_0, quantized_matmul
    w = torch.randn(8, 64)
    q = quantize_q8_0(w)
    assert q.numel() == 8 * 64 // 32 * 34
    assert (dequantize_q8_0(q, w.numel()).reshape(8, 64) - w).abs().max() <= w.abs().max() / 127 + 1e-6
    x = torch.randn(3, 64)
    assert torch.allclose(quantized_matmul(x, q, 8, 64), x @ w.t(), atol=0.6)
    io.export_gguf({"w": w, "b": torch.zeros(8)}, tmp_path / "m.gguf", quantize="q8_0")
    idx = io.read_gguf_index(tmp_path / "m.gguf")
    assert idx["tensors"]["w"] == {"shape": [8, 64], "type": 8, "offset": idx["tensors"]["w"]["offset"]}
    assert idx["tensors"]["b"]["type"] == 0
    rep = io.inspect_file(tmp_path / "m.gguf")
    assert rep.format == "gguf" and rep.parameters == 8 * 64 + 8
    io.export_mlx({"w": w}, tmp_path / "mlx", {"hidden": 64})
    assert io.inspect_file(tmp_path / "mlx" / "weights.safetensors").metadata == {"format": "mlx"}


def test_metrics_and_distributions():
    p, t = torch.tensor([0, 1, 2, 2, 1]), torch.tensor([0, 1, 1, 2, 1])
    acc, f1, cm = MT.Accuracy(), MT.F1Score(3), MT.ConfusionMatrix(3)
    for m in (acc, f1, cm):
        m.update(p, t)
    assert acc.compute() == 0.8 and cm.compute()[1].tolist() == [0, 2, 1]
    assert abs(f1.compute() - (1.0 + 0.8 + 2 / 3) / 3) < 1e-9
    assert MT.Precision(3, "micro").compute() == 0.0
    mse = MT.MSE()
    mse.update(torch.tensor([1.0, 3.0]), torch.tensor([0.0, 1.0]))
    assert mse.compute() == 2.5
    u = D.Uniform(-1, 1).sample((20000,), seed=0)
    assert -1 < float(u.min()) and float(u.max()) < 1 and abs(float(u.mean())) < 0.02
    n = D.Normal(2, 3).sample((100000,), seed=1, offset=5)
    assert abs(float(n.mean()) - 2) < 0.05 and abs(float(n.std()) - 3) < 0.05
    assert torch.equal(n, D.Normal(2, 3).sample((100000,), seed=1, offset=5))      # (seed, offset) names a stream
    assert not torch.equal(n, D.Normal(2, 3).sample((100000,), seed=1, offset=6))
    assert abs(float(D.Bernoulli(0.3).sample((20000,), 2).mean()) - 0.3) < 0.02
    assert abs(float(D.Exponential(2).sample((20000,), 3).mean()) - 0.5) < 0.02
    assert abs(float(D.Gumbel().sample((50000,), 4).mean()) - 0.5772) < 0.03


def test_telemetry_emitter_bounds_and_viewer(tmp_path):
    class Slow:
        def __init__(self):
            self.lines = []
        def send(self, line):
            import time
            time.sleep(0.0005)
            self.lines.append(line)
        def close(self):
            pass
    tr = Slow()
    e = T.Emitter(tr)
    e.emit(T.Event("epoch", "epoch", 1.0), priority=True)
    for i in range(T.BULK_CAP + 2000):
        e.emit(T.Event("scalar", "loss", float(i), i))
    e.close()
    assert e.dropped > 0 and len(tr.lines) + e.dropped == T.BULK_CAP + 2001
    assert any('"epoch"' in ln for ln in tr.lines)                 # priority events survive a bulk flood
    p = tmp_path / "run.jsonl"
    e2 = T.Emitter(T.FileTransport(p))
    T.set_emitter(e2)
    for i in range(20):
        T.emit_scalar("loss", 1.0 / (i + 1), i)
    T.emit_hyperparam("lr", 3e-4)
    e2.close()
    T.set_emitter(None)
    evs = T.read_run(p)
    assert len(evs) == 21 and evs[0].v == T.SCHEMA_VERSION
    fut = T.Event.from_json('{"kind":"new_kind","name":"x","future_field":3}')
    assert fut.kind == "new_kind" and fut.payload["future_field"] == 3
    from incin_b200.telemetry.viz import render
    frame = render(p)
    assert "loss" in frame and "0.0003" in frame and "events 21" in frame
    a, b = T.uuid7(), T.uuid7()
    assert a[14] == "7" and a[:8] <= b[:8]


def test_dataloader_order_workers_and_transforms():
    from incin_b200.data import CenterCrop, Compose, DataLoader, Normalize, Scale, SyntheticTokens, TensorDataset
    ds = TensorDataset(torch.arange(23).float().unsqueeze(1), torch.arange(23))
    a = [b[1].tolist() for b in DataLoader(ds, 5, shuffle=True, workers=3, seed=1)]
    b = [x[1].tolist() for x in DataLoader(ds, 5, shuffle=True, workers=0, seed=1)]
    assert a == b and sorted(sum(a, [])) == list(range(23)) and len(a) == 5
    assert len(list(DataLoader(ds, 5, drop_last=True))) == 4
    dl = DataLoader(ds, 5, shuffle=True, seed=1)
    e1 = [x[1].tolist() for x in dl]
    e2 = [x[1].tolist() for x in dl]
    assert e1 != e2                                                # reshuffled every epoch
    class Bad(TensorDataset):
        def __getitem__(self, i):
            raise RuntimeError("boom")
    with pytest.raises(RuntimeError, match="boom"):
        list(DataLoader(Bad(torch.zeros(4, 1)), 2, workers=2))
    x = Compose(Scale(2.0), Normalize([1.0], [2.0]), CenterCrop(2, 2))(torch.ones(1, 4, 4))
    assert x.shape == (1, 2, 2) and float(x[0, 0, 0]) == 0.5
    tok, tgt = SyntheticTokens(4, 16, 100)[0]
    assert tok.shape == (16,) and torch.equal(tok[1:], tgt[:-1])


def test_trainer_plan_explain_and_fit():
    from incin_b200.data import DataLoader, TensorDataset
    from incin_b200.optim import SGD, make_store
    from incin_b200.train import CollectivesUnavailable, DeviceUnavailable, NotCompiledIn, Trainer
    class NoGpu:
        def compiled_in(self, k): return k is not core.DeviceKind.WGPU
        def has_device(self, d): return d.kind is core.DeviceKind.CPU
        def collectives_available(self, n): return False
    plan = Trainer.plan().epochs(3).build_on(NoGpu())
    assert [d.code for d in plan.decisions] == ["devices-requested", "devices-resolved", "epochs"]
    assert json.loads(plan.explain_json())["devices"] == ["cpu"] and "[epochs] 3" in plan.explain()
    with pytest.raises(DeviceUnavailable):
        Trainer.plan().devices(core.DeviceSet.cuda(range(2))).build_on(NoGpu())
    with pytest.raises(NotCompiledIn):
        Trainer.plan().devices(core.DeviceSet([core.DeviceId(core.DeviceKind.WGPU)])).build_on(NoGpu())
    class TwoGpus(NoGpu):
        def has_device(self, d): return True
    p2 = Trainer.plan().devices(core.DeviceSet.cuda(range(2))).build_on(TwoGpus())
    assert "collectives-required" in [d.code for d in p2.decisions] and p2.is_multi_device
    nn.manual_seed(0)
    m = nn.seq(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 2))
    opt = SGD(make_store(m), lr=0.1)
    with pytest.raises(CollectivesUnavailable):
        Trainer(p2, TwoGpus()).fit(m, opt, [], None)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 8, generator=g)
    y = (x[:, 0] > 0).long()
    hist = Trainer(plan).fit(m, opt, DataLoader(TensorDataset(x, y), 16), lambda mod, a, b: nn.cross_entropy_loss(mod(a), b))
    assert len(hist) == 12 and hist[-1] < hist[0]


def test_native_mlp_benchmark_matches_pytorch_cpu():
    from incin_b200.models.mlp import train_native, train_torch
    a, _ = train_native(steps=100)
    b, _ = train_torch(steps=100)
    assert abs(a[0] - 2.3025) < 1e-3 and a[-1] < 0.7
    assert max(abs(x - y) for x, y in zip(a, b)) < 1e-5


def test_native_tape_linear_shapes_gradients_and_fork():
    """The tape's linear op against PyTorch fp32 on shapes that reach both transposition choices, the vector tiles,
    the scalar column tail and the row pool; an input without gradient gets none; a forked child (which has no
    pool threads) computes the same losses."""
    import ctypes as C
    import os
    from incin_b200 import _native as nat
    from incin_b200.models.mlp import train_native
    h = nat.host()
    for f in ("incin_tape_tensor", "incin_tape_linear", "incin_tape_cross_entropy"):
        getattr(h, f).restype = C.c_int64
    h.incin_tape_tensor.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int]
    h.incin_tape_linear.argtypes = [C.c_int64] * 3
    h.incin_tape_cross_entropy.argtypes = [C.c_int64, C.c_void_p]
    h.incin_tape_backward.argtypes = [C.c_int64]
    h.incin_tape_read.argtypes = h.incin_tape_grad.argtypes = [C.c_int64, C.c_void_p]
    g = torch.Generator().manual_seed(0)
    for m, n, k, x_grad in ((7, 13, 37, True), (64, 300, 200, False), (33, 520, 96, True), (128, 10, 64, True)):
        h.incin_tape_reset()
        x = torch.randn(m, k, generator=g)
        w = torch.randn(n, k, generator=g) / k ** 0.5
        b = torch.randn(n, generator=g)
        t = torch.randint(0, n, (m,), generator=g)
        hx = h.incin_tape_tensor(x.data_ptr(), m, k, int(x_grad))
        hw = h.incin_tape_tensor(w.data_ptr(), n, k, 1)
        hb = h.incin_tape_tensor(b.data_ptr(), 1, n, 1)
        hy = h.incin_tape_linear(hx, hw, hb)
        loss = h.incin_tape_cross_entropy(hy, t.data_ptr())
        assert hy and loss and h.incin_tape_backward(loss) == 0
        y = torch.empty(m, n)
        h.incin_tape_read(hy, y.data_ptr())
        xr, wr, br = (v.clone().requires_grad_() for v in (x, w, b))
        ref = xr @ wr.t() + br
        torch.nn.functional.cross_entropy(ref, t).backward()
        assert torch.allclose(y, ref.detach(), atol=2e-5, rtol=1e-5)
        for hnd, want in ((hw, wr.grad), (hb, br.grad.view(1, n)), (hx, xr.grad)):
            got = torch.zeros_like(want)
            rc = h.incin_tape_grad(hnd, got.data_ptr())
            if hnd == hx and not x_grad:
                assert rc == 2
            else:
                assert rc == 0 and torch.allclose(got, want, atol=2e-6, rtol=1e-4), (m, n, k)
    h.incin_tape_reset()
    a, _ = train_native(steps=3)
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", DeprecationWarning)   # the fork is the point of this check
        pid = os.fork()
    if pid == 0:
        try:
            os._exit(0 if train_native(steps=3)[0] == a else 3)
        finally:
            os._exit(4)
    import signal
    import time
    deadline = time.monotonic() + 60.0          # a child that never returns fails the test instead of hanging it
    while True:
        done, status = os.waitpid(pid, os.WNOHANG)
        if done:
            break
        if time.monotonic() > deadline:
            os.kill(pid, signal.SIGKILL)
            os.waitpid(pid, 0)
            pytest.fail("forked child did not finish")
        time.sleep(0.01)
    assert os.waitstatus_to_exitcode(status) == 0


def test_linear_cross_entropy_cpu_twin_and_model_loss():
    """Off the GPU the fused LM-head loss is linear followed by cross_entropy over the first `num_classes` columns, and
    the GPT-2 model routes its training loss through it."""
    from incin_b200.models.gpt2 import GPT2, GPT2Config
    from incin_b200.ops import functional as F
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 5, 16, generator=g, requires_grad=True)
    w = torch.randn(40, 16, generator=g, requires_grad=True)
    t = torch.randint(0, 33, (2, 5), generator=g)
    loss = F.linear_cross_entropy(x, w, t, 33)
    loss.backward()
    ref = torch.nn.functional.cross_entropy((x.detach().reshape(-1, 16) @ w.detach().T)[:, :33], t.reshape(-1))
    assert abs(loss.item() - ref.item()) < 1e-6
    assert w.grad[33:].abs().max().item() == 0.0          # padded vocabulary rows take no gradient
    cfg = GPT2Config(vocab_size=50, n_layer=1, n_head=2, d_model=16, d_mlp=32, max_seq=8)
    m = GPT2(cfg)
    tok = torch.randint(0, 50, (2, 8), generator=g)
    logits = m(tok)
    l2 = m(tok, tok)
    assert logits.shape[-1] == 50 and torch.isfinite(l2)
    assert abs(l2.item() - torch.nn.functional.cross_entropy(logits.reshape(-1, 50).float(), tok.reshape(-1)).item()) < 1e-4


def test_gradcheck_on_functional_ops_and_detects_a_wrong_backward():
    """Central differences against the analytic gradients of the CPU twins of the model ops, and against a deliberately
    wrong backward (which must be reported)."""
    from incin_b200.gradcheck import gradcheck
    from incin_b200.ops import functional as F
    g = torch.Generator().manual_seed(3)
    r = lambda *s: torch.randn(*s, generator=g, requires_grad=True)   # noqa: E731
    gradcheck(lambda x, w, b: F.linear(x, w, b, act="gelu"), [r(3, 8), r(5, 8), r(5)])
    gradcheck(lambda x, gm, bt: F.layer_norm(x, gm, bt, 1e-5), [r(4, 16), r(16), r(16)])
    gradcheck(lambda x, gm: F.rms_norm(x, gm, 1e-5), [r(4, 16), r(16)])
    tgt = torch.randint(0, 7, (6,), generator=g)
    gradcheck(lambda lg: F.cross_entropy(lg, tgt, 7), [r(6, 8)])
    gradcheck(lambda x, w: F.linear_cross_entropy(x, w, tgt, 7), [r(6, 4), r(8, 4)])
    gradcheck(lambda x, w1, b1, w2, b2: F.mlp(x, w1, b1, w2, b2, act="gelu", residual=x),
              [r(3, 6), r(12, 6), r(12), r(6, 12), r(6)])

    class Wrong(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x):
            ctx.save_for_backward(x)
            return x * x

        @staticmethod
        def backward(ctx, dy):
            (x,) = ctx.saved_tensors
            return dy * x          # should be 2 x dy

    found = gradcheck(Wrong.apply, [r(5)], raise_on_failure=False)
    assert found and "central difference" in str(found[0])
    with pytest.raises(AssertionError):
        gradcheck(Wrong.apply, [r(5)])


def test_shape_algebra_fuzz_against_torch():
    """Seeded fuzz of the shape algebra (spatial geometry, reshape inference, batched matmul shapes) against what
    PyTorch computes, including the rejected cases (the reference fuzzes its shape proofs against an
    integer oracle: crates/incin-core/tests/{spatial_geometry,rank_matrix,shape_buf}.rs)."""
    import random
    import torch.nn.functional as TF
    from incin_b200.core.shapes import ShapeError, conv2d_out, matmul_shape, reshape_infer
    rng = random.Random(1234)
    ok = bad = 0
    for _ in range(300):
        h, w = rng.randint(1, 20), rng.randint(1, 20)
        k = (rng.randint(1, 5), rng.randint(1, 5))
        st = (rng.randint(1, 3), rng.randint(1, 3))
        pd = (rng.randint(0, 2), rng.randint(0, 2))
        dl = (rng.randint(1, 2), rng.randint(1, 2))
        x = torch.zeros(1, 2, h, w)          # real tensors: the meta kernels do not reject an oversized window
        wt = torch.zeros(3, 2, *k)
        try:
            ref = tuple(TF.conv2d(x, wt, stride=st, padding=pd, dilation=dl).shape[-2:])
        except RuntimeError:
            ref = None
        try:
            got = conv2d_out(h, w, k, st, pd, dl)
        except ShapeError:
            got = None
        assert got == ref, (h, w, k, st, pd, dl, got, ref)
        ok += ref is not None
        bad += ref is None
    assert ok > 100 and bad > 10
    for _ in range(300):
        dims = [rng.randint(1, 6) for _ in range(rng.randint(1, 4))]
        n = 1
        for d in dims:
            n *= d
        target = [rng.randint(1, 6) for _ in range(rng.randint(1, 4))]
        if rng.random() < 0.6:
            target[rng.randrange(len(target))] = -1
        try:
            ref = tuple(torch.empty(dims, device="meta").reshape(target).shape)
        except RuntimeError:
            ref = None
        try:
            got = reshape_infer(n, target)
        except ShapeError:
            got = None
        assert got == ref, (dims, target, got, ref)
    for _ in range(300):
        batch_a = [rng.choice([1, 2, 3]) for _ in range(rng.randint(0, 2))]
        batch_b = [rng.choice([1, 2, 3]) for _ in range(rng.randint(0, 2))]
        m, k1, k2, n = rng.randint(1, 5), rng.randint(1, 4), rng.randint(1, 4), rng.randint(1, 5)
        a, b = batch_a + [m, k1], batch_b + [k2, n]
        try:
            ref = tuple((torch.empty(a, device="meta") @ torch.empty(b, device="meta")).shape)
        except RuntimeError:
            ref = None
        try:
            got = tuple(d.size for d in matmul_shape(a, b).dims)
        except ShapeError:
            got = None
        assert got == ref, (a, b, got, ref)


def test_tensor_api_names_of_the_reference_surface():
    """Creation, reductions and manipulation under the reference's names (crates/incin-core/src/tensor/base.rs,
    tensor/ops/{reduce,manipulation}.rs): thin front ends over the native ops and their PyTorch twins."""
    import ctypes
    import incin_b200.tensor as T
    x = torch.arange(24.0).reshape(2, 3, 4)
    assert T.flatten(x, 1).shape == (2, 12)
    assert torch.equal(T.slice(x, 2, 1, 4, 2), x[:, :, 1:4:2]) and torch.equal(T.slice(x, 0, 1, 2), x[1:2])
    assert T.to_dtype(x, "bf16").dtype == torch.bfloat16 and T.to_dtype(x, torch.float64).dtype == torch.float64
    assert torch.equal(T.where_cond(x > 5, x, -x), torch.where(x > 5, x, -x))
    idx = torch.tensor([[[0, 3], [1, 1], [2, 0]], [[3, 3], [0, 1], [2, 2]]])
    assert torch.equal(T.gather(x, -1, idx), torch.gather(x, -1, idx))
    assert torch.equal(T.gather(x, 1, idx[:, :, :1].expand(2, 3, 4) % 3), torch.gather(x, 1, idx[:, :, :1].expand(2, 3, 4) % 3))
    z = torch.zeros(2, 3, 4)
    assert torch.equal(T.scatter(z, -1, idx, torch.ones(2, 3, 2)), torch.scatter(z, -1, idx, torch.ones(2, 3, 2)))
    assert float(T.sum(x)) == 276 and float(T.mean(x)) == 11.5 and float(T.max(x)) == 23 and float(T.min(x)) == 0
    assert T.argmin(x.flatten()).item() == 0 and torch.equal(T.argmax(x, 2), x.argmax(2))
    assert torch.equal(T.sum(x, 1, keepdim=True), x.sum(1, keepdim=True))
    a = (ctypes.c_float * 6)(1, 2, 3, 4, 5, 6)
    t = T.from_raw(ctypes.addressof(a), (2, 3), "f32", owner=a)
    assert t.tolist() == [[1, 2, 3], [4, 5, 6]]
    a[0] = 9                                                  # a view of the caller's memory, not a copy
    assert t[0, 0].item() == 9


def test_descriptor_vocabulary_axis_mask_alignment_handles_and_index_objects():
    from incin_b200.core.iteration import UnaryIterationPlan, unary_plan
    from incin_b200.core.shapes import BroadcastShape, InferDim, ReshapeShape, ShapeError, Slice, idx, s
    from incin_b200.core.spec import Alignment, AxisMask, ExecutionContext, TensorHandle, TensorMeta
    m = AxisMask.from_axes([-1, 0], 3)
    assert m.axes() == (0, 2) and m.contains(2) and not m.contains(1) and len(m) == 2
    assert m.reduced_shape((4, 5, 6)) == (5,) and m.reduced_shape((4, 5, 6), keepdim=True) == (1, 5, 1)
    assert AxisMask.all(4).axes() == (0, 1, 2, 3)
    for bad in ([1, 1], [3], [-4]):
        with pytest.raises(ShapeError):
            AxisMask.from_axes(bad, 3)
    with pytest.raises(ShapeError):
        m.reduced_shape((4, 5))
    assert Alignment.of_address(256) is Alignment.LINE and Alignment.of_address(96) is Alignment.VEC32
    assert Alignment.of_address(48) is Alignment.VEC16 and Alignment.of_address(12) is Alignment.WORD
    assert Alignment.of_address(6) is Alignment.BYTE and Alignment.VEC32 > Alignment.VEC16
    t = torch.zeros(4, 8)
    h = TensorHandle.of(t)
    assert h.meta.shape == (4, 8) and h.address == t.data_ptr() and h.alignment >= Alignment.VEC16
    ctx = ExecutionContext.current()
    assert ctx.policy is not None and ctx.stream >= 0
    assert BroadcastShape((4, 1, 6), (5, 6)).result == s(4, 5, 6)
    with pytest.raises(ShapeError):
        BroadcastShape((4, 3), (5,)).result
    assert ReshapeShape((4, 6), (InferDim, 3)).result == (8, 3) and ReshapeShape((4, 6), (2, 12)).result == (2, 12)
    with pytest.raises(ShapeError):
        ReshapeShape((4, 6), (InferDim, 5)).result
    x = torch.arange(24).reshape(4, 6)
    assert torch.equal(idx[Slice(1, 3), ...].apply(x), x[1:3]) and torch.equal(idx[..., Slice(0, 6, 2)].apply(x), x[:, 0:6:2])
    with pytest.raises(ShapeError):
        idx[Slice(2, 9)].apply(x)
    p = unary_plan(TensorMeta.of(t), TensorMeta.of(t))
    assert isinstance(p, UnaryIterationPlan) and p.input is p.operands[0]


def test_collate_objects_and_hub_lookup(tmp_path):
    from incin_b200.data import Collate, DataLoader, TensorDataset, from_pretrained
    pad = Collate(pad_value=-1)
    b = pad([(torch.tensor([1, 2, 3]), torch.tensor(0)), (torch.tensor([4]), torch.tensor(1))])
    assert b[0].tolist() == [[1, 2, 3], [4, -1, -1]] and b[1].tolist() == [0, 1]
    assert Collate()([(torch.ones(2), 1), (torch.zeros(2), 0)])[0].shape == (2, 2)
    assert Collate(lambda s: len(s))([1, 2, 3]) == 3
    ds = TensorDataset(torch.arange(10.0).unsqueeze(1), torch.arange(10))
    assert [x[1].tolist() for x in DataLoader(ds, 4, collate=Collate())] == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9]]
    with pytest.raises(FileNotFoundError):                     # offline: only what is already in the cache resolves
        from_pretrained("nobody/nothing", cache_dir=tmp_path)
