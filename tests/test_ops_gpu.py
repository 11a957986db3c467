"""Every non-GEMM sm_100a kernel against a PyTorch fp32 reference of the same op."""
import math

import pytest
import torch
import torch.nn.functional as TF

pytestmark = pytest.mark.gpu


def rnd(shape, seed, dtype=torch.bfloat16, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).cuda()


def close(a, b, tol=2e-2):
    from _tol import check_close
    fp32_out = a.dtype == torch.float32
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    assert err <= tol * (b.abs().max().item() + 1e-6), f"err {err}"
    check_close(a, b, rtol=1e-2 if fp32_out else 1.6e-2, atol_rms=1e-2 if fp32_out else 1.5e-2, min_cos=0.9999, what="op")


@pytest.mark.parametrize("rows,C", [(64, 768), (333, 1024), (17, 100), (8, 4096), (5000, 768), (3, 264)])
def test_layernorm_fwd_bwd(rows, C):
    from incin_b200.ops import kernels as K
    x, g, b, dy, add = rnd((rows, C), 1), rnd((C,), 2), rnd((C,), 3), rnd((rows, C), 4), rnd((rows, C), 5)
    y, mean, rstd = K.layernorm_fwd(x, g, b, 1e-5)
    xf = x.float().requires_grad_()
    gf, bf = g.float().requires_grad_(), b.float().requires_grad_()
    yr = TF.layer_norm(xf, (C,), gf, bf, 1e-5)
    close(y, yr)
    yr.backward(dy.float())
    dg = torch.zeros(C, device="cuda")
    db = torch.zeros(C, device="cuda")
    dx = K.layernorm_bwd(dy, x, g, mean, rstd, add, dg, db)
    close(dx, xf.grad + add.float())
    close(dg, gf.grad)
    close(db, bf.grad)


@pytest.mark.parametrize("rows,C", [(64, 2048), (33, 96), (3000, 512)])
def test_rmsnorm_fwd_bwd(rows, C):
    from incin_b200.ops import kernels as K
    x, g, dy = rnd((rows, C), 1), rnd((C,), 2), rnd((rows, C), 4)
    y, rstd = K.rmsnorm_fwd(x, g, 1e-5)
    xf, gf = x.float().requires_grad_(), g.float().requires_grad_()
    yr = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * gf
    close(y, yr)
    yr.backward(dy.float())
    dg = torch.zeros(C, device="cuda")
    dx = K.rmsnorm_bwd(dy, x, g, rstd, None, dg)
    close(dx, xf.grad)
    close(dg, gf.grad)


def test_embedding():
    from incin_b200.ops import kernels as K
    V, T, C, B = 1000, 64, 256, 4
    wte, wpe = rnd((V, C), 1), rnd((T, C), 2)
    tok = torch.randint(0, V, (B, T), generator=torch.Generator().manual_seed(3)).cuda()
    out = K.embedding_fwd(tok, wte, wpe)
    close(out, wte.float()[tok] + wpe.float()[None])
    dout = rnd((B, T, C), 4)
    dwte, dwpe = torch.zeros(V, C, device="cuda"), torch.zeros(T, C, device="cuda")
    K.embedding_bwd(dout, tok, dwte, dwpe)
    ref = torch.zeros(V, C, device="cuda").index_add_(0, tok.view(-1), dout.float().view(-1, C))
    close(dwte, ref, 1e-3)
    close(dwpe, dout.float().sum(0), 1e-3)


@pytest.mark.parametrize("rows,V,ld", [(64, 50257, 50304), (10, 509, 512), (7, 33, 33)])
def test_cross_entropy(rows, V, ld):
    from incin_b200.ops import kernels as K
    full = rnd((rows, ld), 1, scale=3.0)
    tgt = torch.randint(0, V, (rows,), generator=torch.Generator().manual_seed(2)).cuda()
    lf = full.float()[:, :V].clone().requires_grad_()
    ref = TF.cross_entropy(lf, tgt, reduction="none")
    loss, lse = K.xent_fwd(full, tgt, V)
    close(loss, ref, 1e-3)
    ref.mean().backward()
    dl = torch.full((1,), 1.0, device="cuda")
    K.xent_bwd_(full, tgt, lse, dl, 1.0 / rows, V)
    close(full[:, :V], lf.grad, 2e-2)
    assert full[:, V:].abs().max().item() == 0 if ld > V else True
    close(K.mean_f32(loss), ref.mean(), 1e-4)


def test_causal_softmax():
    from incin_b200.ops import kernels as K
    Bt, T = 3, 128
    s = rnd((Bt, T, T), 1)
    mask = torch.ones(T, T, device="cuda").tril().bool()
    sf = s.float().requires_grad_()
    ref = torch.softmax((sf * 0.5).masked_fill(~mask, float("-inf")), -1)
    p = K.causal_softmax_fwd_(s.clone(), T, 0.5)
    close(p, ref)
    dp = rnd((Bt, T, T), 2)
    ref.backward(dp.float())
    ds = K.causal_softmax_bwd_(dp.clone(), p, T, 0.5)
    close(ds, sf.grad, 3e-2)


def test_colsum_and_gradcheck_kernels():
    from incin_b200.ops import kernels as K
    dy = rnd((1000, 300), 1)
    db = torch.ones(300, device="cuda")
    K.colsum_accum(dy, db)
    close(db, 1 + dy.float().sum(0), 1e-3)
    x = torch.randn(100000, device="cuda")
    out = torch.zeros(2, device="cuda")
    K.sumsq_nonfinite(x, out)
    assert abs(out[0].item() - (x * x).sum().item()) < 1e-2 * (x * x).sum().item()
    assert out[1].item() == 0
    x[777] = float("nan")
    out.zero_()
    K.sumsq_nonfinite(x, out)
    assert out[1].item() == 1


def test_adamw_and_sgd_flat():
    from incin_b200.ops import kernels as K
    n, nd = 10007, 6000
    w = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    shadow = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    wr, mr, vr = w.clone(), m.clone(), v.clone()
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.999, 1e-8, 0.1
    for t in (1, 2, 3):
        hyper = torch.tensor([lr, b1, b2, eps, wd, t, 1.0, 0], device="cuda")
        K.adamw_flat(w, m, v, g, shadow, nd, hyper)
        mr = b1 * mr + (1 - b1) * g
        vr = b2 * vr + (1 - b2) * g * g
        decay = torch.zeros(n, device="cuda")
        decay[:nd] = wd
        wr = wr - lr * decay * wr - lr * (mr / (1 - b1 ** t)) / ((vr / (1 - b2 ** t)).sqrt() + eps)
    close(w, wr, 1e-5)
    close(shadow, wr, 1e-2)
    w2 = torch.randn(n, device="cuda")
    ref = w2 - 0.01 * g
    K.sgd_flat(w2, None, g, None, 0, torch.tensor([0.01, 0, 0, 0, 0, 0, 1.0, 0], device="cuda"))
    close(w2, ref, 1e-6)


def test_swiglu_rope_act():
    from incin_b200 import _native as nat
    from incin_b200.ops import functional as F, kernels as K
    gu = rnd((50, 2 * 96), 1).requires_grad_()
    y = F.swiglu(gu)
    gf = gu.detach().float().requires_grad_()
    a, b = gf.chunk(2, -1)
    ref = TF.silu(a) * b
    close(y, ref)
    dy = rnd((50, 96), 2)
    y.backward(dy)
    ref.backward(dy.float())
    close(gu.grad, gf.grad)
    x = rnd((2, 16, 6, 64), 3)
    out = F.rope(x, 4, 64, 10000.0)
    close(out, F._rope_cpu(x.cpu(), 4, 64, 10000.0).cuda())
    h = rnd((1000,), 4)
    close(K.act_fwd(h, nat.ACT_GELU), TF.gelu(h.float()))
    close(K.act_fwd(h, nat.ACT_SILU), TF.silu(h.float()))


def test_philox_and_dropout():
    from incin_b200.ops import kernels as K
    u = K.philox_uniform((1 << 20,), 0, 0, "cuda")
    assert 0.0 < u.min().item() and u.max().item() < 1.0
    assert abs(u.mean().item() - 0.5) < 2e-3
    n1 = K.philox_normal((1 << 20,), 0, 1, "cuda", 0.0, 0.02)
    assert abs(n1.mean().item()) < 1e-3 and abs(n1.std().item() - 0.02) < 1e-3
    n2 = K.philox_normal((1 << 20,), 0, 1, "cuda", 0.0, 0.02)
    assert torch.equal(n1, n2)  # same (seed, offset) -> same stream
    x = torch.ones(1 << 20, dtype=torch.bfloat16, device="cuda")
    y = K.dropout(x, 0.25, 5, 9)
    keep = (y != 0).float().mean().item()
    assert abs(keep - 0.75) < 5e-3
    assert abs(y.float().mean().item() - 1.0) < 1e-2


def test_linear_cross_entropy_fused():
    """Loss and gradients of the fused LM-head + cross-entropy op against linear -> cross_entropy in fp32, with an
    upstream gradient other than one (it reaches the two products as a device scalar)."""
    from incin_b200.ops import functional as F
    rows, C, V, Vpad = 300, 256, 1000, 1024
    x = rnd((3, 100, C), 1).requires_grad_()
    w = rnd((Vpad, C), 2, scale=0.05).requires_grad_()
    tgt = torch.randint(0, V, (3, 100), generator=torch.Generator().manual_seed(3)).cuda()
    w.main_grad = torch.zeros(Vpad, C, device="cuda")
    loss = F.linear_cross_entropy(x, w, tgt, V)
    (loss * 3.0).backward()
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    ref = TF.cross_entropy((xf.reshape(-1, C) @ wf.T)[:, :V], tgt.reshape(-1))
    (ref * 3.0).backward()
    assert abs(loss.item() - ref.item()) < 2e-2 * abs(ref.item())
    close(x.grad, xf.grad, tol=3e-2)
    close(w.main_grad, wf.grad, tol=3e-2)
    assert w.main_grad[V:].abs().max().item() == 0.0      # padded vocabulary rows get no gradient


@pytest.mark.parametrize("rows,C", [(5, 8), (300, 256), (8192, 512), (1001, 1000)])
def test_pipelined_norm_backward_edges(rows, C):
    """The pipelined one-pass backward with column sums on its edge cases (fewer rows than warps, a partly filled last
    group of 256 columns, no incoming residual gradient) against fp32 autograd."""
    from _tol import check_close
    from incin_b200.ops import kernels as K
    g = torch.Generator().manual_seed(rows * 7 + C)
    x = torch.randn(rows, C, generator=g).bfloat16().cuda()
    dy = torch.randn(rows, C, generator=g).bfloat16().cuda()
    gamma = (torch.rand(C, generator=g) + 0.5).bfloat16().cuda()
    beta = torch.zeros(C).bfloat16().cuda()
    _, mean, rstd = K.layernorm_fwd(x, gamma, beta, 1e-5)
    dg, db, cs = (torch.zeros(C, device="cuda") for _ in range(3))
    dx = K.layernorm_bwd(dy, x, gamma, mean, rstd, None, dg, db, cs)
    xr, gr, br = x.float().requires_grad_(), gamma.float().requires_grad_(), beta.float().requires_grad_()
    torch.nn.functional.layer_norm(xr, (C,), gr, br, 1e-5).backward(dy.float())
    check_close(dx, xr.grad, rtol=1.6e-2, atol_rms=1.5e-2, what=f"dx {rows}x{C}")
    check_close(dg, gr.grad, rtol=5e-3, atol_rms=5e-3, what=f"dgamma {rows}x{C}")
    check_close(db, br.grad, rtol=5e-3, atol_rms=5e-3, what=f"dbeta {rows}x{C}")
    check_close(cs, dx.float().sum(0), rtol=1e-2, atol_rms=1e-2, what=f"column sums {rows}x{C}")


@pytest.mark.parametrize("C", [768, 1024, 2048, 100])
def test_layernorm_backward_also_returns_the_column_sums_of_dx(C):
    """The bias gradient of the linear in front of a norm is the column sum of the norm's input gradient: it comes out
    of the one-pass backward kernel (C <= 1024, C % 8 == 0) or from one column-sum launch behind it; either way it
    equals the fp32 column sums of the dx that the plain backward returns, and it accumulates."""
    from _tol import check_close
    from incin_b200.ops import kernels as K
    g = torch.Generator().manual_seed(C)
    rows = 1000
    x = torch.randn(rows, C, generator=g).bfloat16().cuda()
    dy = torch.randn(rows, C, generator=g).bfloat16().cuda()
    res = torch.randn(rows, C, generator=g).bfloat16().cuda()
    gamma = (torch.rand(C, generator=g) + 0.5).bfloat16().cuda()
    beta = torch.zeros(C).bfloat16().cuda()
    _, mean, rstd = K.layernorm_fwd(x, gamma, beta, 1e-5)
    dg0, db0 = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
    dx0 = K.layernorm_bwd(dy, x, gamma, mean, rstd, res, dg0, db0)
    dg1, db1 = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
    cs = torch.full((C,), 3.0, device="cuda")                       # accumulates on top of what is there
    dx1 = K.layernorm_bwd(dy, x, gamma, mean, rstd, res, dg1, db1, cs)
    # the one-pass kernel with column sums is its own kernel (pipelined, other summation order): close, not equal
    check_close(dx1, dx0.float(), rtol=1.6e-2, atol_rms=1e-2, what=f"dx, C={C}")
    check_close(dg1, dg0, rtol=1e-3, atol_rms=1e-3, what=f"dgamma, C={C}")
    check_close(db1, db0, rtol=1e-3, atol_rms=1e-3, what=f"dbeta, C={C}")
    want = dx0.float().sum(0) + 3.0
    check_close(cs, want, rtol=1e-2, atol_rms=1e-2, what=f"column sums of dx, C={C}")
