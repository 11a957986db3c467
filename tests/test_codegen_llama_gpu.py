"""The NVRTC pointwise fuser on the device (every op, both layouts, runtime scalars, fusion groups lowered from a
traced graph) and the single-GPU Llama (RMSNorm, RoPE, GQA flash attention, SwiGLU) against PyTorch fp32 math."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

from _tol import check_close  # noqa: E402
DEV = "cuda"


def test_every_unary_binary_ternary_op_matches_torch():
    from incin_b200.codegen.pointwise import BINARY, TERNARY, UNARY, Arg, Binary, Ternary, Unary
    from incin_b200.codegen.runtime import fused
    torch.manual_seed(0)
    x = torch.randn(3000, device=DEV)
    pos = x.abs() + 0.1
    ref_unary = {
        "relu": torch.relu, "step": lambda t: (t > 0).float(), "sigmoid": torch.sigmoid, "tanh": torch.tanh,
        "swish": torch.nn.functional.silu, "softplus": torch.nn.functional.softplus, "elu": torch.nn.functional.elu,
        "gelu": torch.nn.functional.gelu, "gelu_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh"),
        "exp": torch.exp, "log": torch.log, "sqrt": torch.sqrt, "rsqrt": torch.rsqrt, "neg": torch.neg, "abs": torch.abs,
        "sign": torch.sign, "mish": torch.nn.functional.mish, "recip": torch.reciprocal, "square": torch.square,
        "sin": torch.sin, "cos": torch.cos, "floor": torch.floor, "ceil": torch.ceil,
    }
    assert set(ref_unary) == set(UNARY)
    for op, ref in ref_unary.items():
        inp = pos if op in ("log", "sqrt", "rsqrt", "recip") else x
        torch.testing.assert_close(fused(Unary(op, Arg(0)), inp), ref(inp), rtol=2e-3, atol=2e-3, msg=op)
    y = torch.randn(3000, device=DEV)
    ref_binary = {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div, "max": torch.maximum,
                  "min": torch.minimum, "pow": torch.pow}
    assert set(ref_binary) == set(BINARY)
    for op, ref in ref_binary.items():
        a = pos if op == "pow" else x
        torch.testing.assert_close(fused(Binary(op, Arg(0), Arg(1)), a, y), ref(a, y), rtol=2e-3, atol=2e-3, msg=op)
    z = torch.randn(3000, device=DEV)
    lo, hi = torch.minimum(y, z), torch.maximum(y, z)
    torch.testing.assert_close(fused(Ternary("clamp", Arg(0), Arg(1), Arg(2)), x, lo, hi), torch.clamp(x, lo, hi))
    torch.testing.assert_close(fused(Ternary("fma", Arg(0), Arg(1), Arg(2)), x, y, z), x * y + z, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(fused(Ternary("where", Arg(0), Arg(1), Arg(2)), (x > 0).float(), y, z), torch.where(x > 0, y, z))
    assert set(TERNARY) == {"clamp", "fma", "where"}


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_chain_with_scalars_and_broadcast_layouts(dtype):
    from incin_b200.codegen.pointwise import Arg, Scalar, Unary
    from incin_b200.codegen.runtime import fused
    torch.manual_seed(1)
    a = torch.randn(64, 1, 96, device=DEV).to(dtype)
    b = torch.randn(1, 33, 96, device=DEV).to(dtype)
    expr = Unary("gelu_tanh", Arg(0) * Scalar(0) + Arg(1)) * Scalar(1)
    for s in ((0.5, 2.0), (1.5, -1.0)):        # the same compiled kernel serves every scalar value
        got = fused(expr, a, b, scalars=s)
        ref = torch.nn.functional.gelu(a.float() * s[0] + b.float(), approximate="tanh") * s[1]
        tol = 1e-4 if dtype == torch.float32 else 3e-2
        torch.testing.assert_close(got.float(), ref, rtol=tol, atol=tol)
    x = torch.randn(1000003, device=DEV).to(dtype)       # odd length: vector body + scalar tail
    torch.testing.assert_close(fused(Unary("relu", Arg(0)) * 3.0, x).float(), torch.relu(x.float()) * 3.0, rtol=2e-2, atol=2e-2)
    t = torch.randn(128, 256, device=DEV).to(dtype)
    torch.testing.assert_close(fused(Arg(0) + Arg(1), t, t.t().contiguous().t()), t + t)     # strided operand


def test_fusion_group_from_traced_graph_runs_as_one_kernel():
    from incin_b200 import graph as G
    from incin_b200.codegen.runtime import fused

    def f(x, w, b):
        return torch.tanh(torch.relu(x @ w + b) * 2.0)
    x, w, b = torch.randn(64, 32), torch.randn(32, 48), torch.randn(64, 48)
    g = G.trace(f, x, w, b)
    (grp,) = G.fusion_pass(g)
    expr, ext = G.lower_group(g, grp)
    mm = (x @ w).to(DEV)
    feeds = {nid: t for nid, t in zip(ext, [None] * len(ext))}
    for nid in ext:
        feeds[nid] = mm if g.nodes[nid].op == "mm" else b.to(DEV)
    got = fused(expr, *[feeds[n] for n in ext])
    torch.testing.assert_close(got.cpu(), f(x, w, b), rtol=1e-4, atol=1e-4)


def test_llama_single_gpu_matches_fp32_reference_and_trains():
    from incin_b200.engine import TrainStep
    from incin_b200.models.llama import Llama, LlamaConfig
    from incin_b200.ops import gemm as G
    from incin_b200.optim import AdamW, ParamStore
    cfg = LlamaConfig.tiny()
    cpu = Llama(cfg, seed=3)
    gpu = copy.deepcopy(cpu).cuda()
    g = torch.Generator().manual_seed(1)
    tok = torch.randint(0, cfg.vocab_size, (2, 128), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (2, 128), generator=g)
    store = ParamStore(gpu.named_parameters())
    loss_c = cpu(tok, tgt)
    loss_c.backward()
    store.zero_grad()
    loss_g = gpu(tok.cuda(), tgt.cuda())
    loss_g.backward()
    assert abs(loss_g.item() - loss_c.item()) < 3e-2
    ref = dict(cpu.named_parameters())
    for name, p, o, k in store.entries:
        g_gpu, g_cpu = p.main_grad.float().cpu(), ref[name].grad
        denom = g_cpu.abs().max().item() + 1e-6
        assert (g_gpu - g_cpu).abs().max().item() <= 8e-2 * denom + 2e-4, name
        # a whole model in bf16 against fp32: the direction of every parameter gradient must still agree, and no
        # element may be off by more than a tenth of the gradient's RMS plus a tenth of its own size
        check_close(g_gpu, g_cpu, rtol=1e-1, atol_rms=1e-1, min_cos=0.995, what=f"grad {name}")
    del loss_g      # a live autograd graph from the default stream would keep capture from working (see TrainStep)
    opt = AdamW(store, lr=1e-3)
    step = TrainStep(gpu, opt, use_graph=True)
    tok, tgt = tok.cuda(), tgt.cuda()
    losses = [step(tok, tgt).item() for _ in range(12)]
    assert losses[-1] < losses[0] - 0.5, losses
    assert step.graph is not None, step.capture_error
    G.check_status()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_row_chain_fuser_matches_fp32_math(dtype):
    """softmax / log-softmax / layer norm / rms norm with pointwise prologues and epilogues, one kernel each, against
    the fp32 evaluation of the same chain; odd widths and more rows than warps in flight."""
    from _tol import check_close
    from incin_b200.codegen import Arg, Col, Norm, Scalar, Unary, fused_rows, reference_rows
    g = torch.Generator().manual_seed(5)
    for rows, C in ((37, 100), (4096, 768), (3, 2049)):
        x = torch.randn(rows, C, generator=g).to(dtype).cuda()
        r = torch.randn(rows, C, generator=g).to(dtype).cuda()
        gain = (torch.rand(C, generator=g) + 0.5).to(dtype).cuda()
        bias = torch.randn(C, generator=g).to(dtype).cuda()
        chains = [("softmax", Arg(0) * Scalar(0) + Col(0), None, [x], [bias], [0.125]),
                  ("log_softmax", Arg(0) + Arg(1), None, [x, r], [], []),
                  ("layer_norm", Arg(0) + Arg(1), Norm() * Col(0) + Col(1), [x, r], [gain, bias], []),
                  ("rms_norm", Arg(0), Unary("gelu", Norm() * Col(0)), [x], [gain], [])]
        for kind, pre, post, rin, cols, sc in chains:
            got = fused_rows(kind, pre, rin, post=post, cols=cols, scalars=sc)
            want = reference_rows(kind, pre, rin, post=post, cols=cols, scalars=sc)
            assert got.dtype == dtype and got.shape == x.shape
            tol = dict(rtol=2e-2, atol_rms=2e-2) if dtype == torch.bfloat16 else dict(rtol=2e-3, atol_rms=1e-3)
            check_close(got, want, what=f"{kind} {rows}x{C} {dtype}", **tol)
