"""Native reductions, data-movement ops, pooling, batch norm, im2col/col2im, Q8_0 and the deterministic embedding
backward against plain PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from incin_b200.ops import tensor_ops as T  # noqa: E402

DEV = "cuda"


def _ref(x):
    return x.float()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,dim", [((37, 1000), 1), ((5, 4099), 1), ((6, 50, 33), 1), ((3, 7, 129), 0), ((2000, 8), 0)])
def test_reduce_axis(dtype, shape, dim):
    torch.manual_seed(0)
    x = torch.randn(shape, device=DEV).to(dtype)
    for op in ("sum", "mean", "max", "min"):
        got = T.reduce(x, op, dim).float()
        want = getattr(torch, op)(_ref(x), dim=dim)
        want = want if op in ("sum", "mean") else want.values
        tol = 1e-4 if dtype == torch.float32 else 2e-2
        torch.testing.assert_close(got, want, rtol=tol, atol=tol * max(1.0, float(want.abs().max())))
    for op in ("argmax", "argmin"):
        got = T.reduce(x, op, dim)
        want = getattr(torch, op)(_ref(x), dim=dim)
        # ties (bf16) may pick another index with the same value: compare the values picked
        gv = torch.gather(_ref(x), dim, got.unsqueeze(dim)).squeeze(dim)
        wv = torch.gather(_ref(x), dim, want.unsqueeze(dim)).squeeze(dim)
        assert torch.equal(gv, wv)
    k = T.reduce(x, "sum", dim, keepdim=True)
    assert k.shape[dim] == 1 and k.dim() == x.dim()


def test_reduce_prod_and_nan_propagation():
    x = (torch.rand(9, 64, device=DEV) + 0.5)
    torch.testing.assert_close(T.reduce(x, "prod", 1), torch.prod(x, 1), rtol=1e-4, atol=1e-6)
    y = torch.randn(4, 300, device=DEV)
    y[2, 17] = float("nan")
    m = T.reduce(y, "max", 1)
    assert torch.isnan(m[2]) and not torch.isnan(m[[0, 1, 3]]).any()
    assert int(T.reduce(y, "argmax", 1)[2]) == 17


@pytest.mark.parametrize("n", [1, 1000, 1 << 20, (1 << 22) + 3])
def test_reduce_all_is_deterministic(n):
    torch.manual_seed(1)
    x = torch.randn(n, device=DEV)
    a, b = T.reduce(x, "sum"), T.reduce(x, "sum")
    assert torch.equal(a, b)
    torch.testing.assert_close(a.double(), x.double().sum(), rtol=1e-5, atol=1e-2)
    torch.testing.assert_close(T.reduce(x, "max"), x.max())
    torch.testing.assert_close(T.reduce(x, "mean").double(), x.double().mean(), rtol=1e-4, atol=1e-5)
    assert int(T.reduce(x, "argmin")) == int(x.argmin())
    xb = x.bfloat16()
    torch.testing.assert_close(T.reduce(xb, "sum").float(), xb.float().sum(), rtol=2e-2, atol=2.0)


@pytest.mark.parametrize("shape,dim", [((7, 5000), 1), ((3, 100, 17), 1), ((64, 9), 0)])
def test_cumsum_var_std_norm(shape, dim):
    torch.manual_seed(2)
    x = torch.randn(shape, device=DEV)
    torch.testing.assert_close(T.cumsum(x, dim), torch.cumsum(x, dim), rtol=1e-4, atol=1e-3)
    torch.testing.assert_close(T.var(x, dim), x.var(dim), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(T.std(x, dim, unbiased=False), x.std(dim, unbiased=False), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(T.norm(x), x.norm(), rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64])
def test_strided_copies(dtype):
    torch.manual_seed(3)
    x = (torch.randn(6, 40, 72, device=DEV) * 10).to(dtype)
    assert torch.equal(T.transpose(x, 1, 2), x.transpose(1, 2).contiguous())          # tiled transpose path
    assert torch.equal(T.transpose(x, 0, 2), x.transpose(0, 2).contiguous())          # generic path
    assert torch.equal(T.narrow(x, 2, 8, 32), x.narrow(2, 8, 32).contiguous())        # vector path
    assert torch.equal(T.narrow(x, 2, 3, 31), x.narrow(2, 3, 31).contiguous())        # unaligned
    assert torch.equal(T.broadcast_to(x[:, :1, :], (6, 5, 72)), x[:, :1, :].expand(6, 5, 72).contiguous())
    assert torch.equal(T.concat([x, x[:, :3]], 1), torch.cat([x, x[:, :3]], 1))
    dst = torch.zeros(6, 50, 72, device=DEV, dtype=dtype)
    assert torch.equal(T.paste(dst, x, 1, 7)[:, 7:47], x) and float(dst[:, :7].abs().sum()) == 0
    p = T.pad(x, [(0, 0), (1, 2), (3, 0)], value=1)
    want = torch.nn.functional.pad(x, (3, 0, 1, 2), value=1)
    assert torch.equal(p, want)


def test_indexed_ops_and_bad_index_is_reported_not_dereferenced():
    torch.manual_seed(4)
    x = torch.randn(50, 24, device=DEV).bfloat16()
    idx = torch.randint(0, 50, (200,), device=DEV)
    assert torch.equal(T.index_select(x, 0, idx), x[idx])
    x3 = torch.randn(5, 50, 8, device=DEV)
    assert torch.equal(T.index_select(x3, 1, idx[:20]), torch.index_select(x3, 1, idx[:20]))
    acc = torch.zeros(50, 24, device=DEV)
    T.index_add_rows(acc, idx, x[idx])
    want = torch.zeros(50, 24, device=DEV).index_add_(0, idx, x[idx].float())
    torch.testing.assert_close(acc, want, rtol=1e-5, atol=1e-4)
    g_idx = torch.randint(0, 24, (50, 7), device=DEV)
    assert torch.equal(T.gather_last(x, g_idx), torch.gather(x, 1, g_idx))
    perm = torch.stack([torch.randperm(24, device=DEV)[:7] for _ in range(50)])
    src = torch.randn(50, 7, device=DEV).bfloat16()
    assert torch.equal(T.scatter_last(torch.zeros_like(x), perm, src), torch.zeros_like(x).scatter_(1, perm, src))
    T.check_indices(torch.device(DEV))
    bad = idx.clone()
    bad[5] = 50
    out = T.index_select(x, 0, bad)          # the bad row is skipped, the rest is right
    assert torch.equal(out[:5], x[bad[:5]])
    with pytest.raises(IndexError):
        T.check_indices(torch.device(DEV))
    T.check_indices(torch.device(DEV))       # the flag was cleared


def test_mask_where_tri():
    torch.manual_seed(5)
    x = torch.randn(3, 33, 65, device=DEV).bfloat16()
    y = torch.randn(3, 33, 65, device=DEV).bfloat16()
    m = torch.rand(3, 33, 65, device=DEV) > 0.5
    assert torch.equal(T.masked_fill(x, m, -2.0), x.masked_fill(m, -2.0))
    assert torch.equal(T.masked_fill(x, m[0], float("-inf")), x.masked_fill(m[0], float("-inf")))
    assert torch.equal(T.where(m, x, y), torch.where(m, x, y))
    for d in (-2, 0, 3):
        assert torch.equal(T.triu(x, d), torch.triu(x, d)) and torch.equal(T.tril(x, d), torch.tril(x, d))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("k,s,p", [(2, 2, 0), (3, 2, 1), (3, 1, 1)])
def test_pooling_forward_backward(dtype, k, s, p):
    torch.manual_seed(6)
    x = torch.randn(2, 5, 19, 23, device=DEV).to(dtype).requires_grad_(True)
    xr = x.detach().float().requires_grad_(True)
    for ours, ref in ((T.max_pool2d, torch.nn.functional.max_pool2d), (T.avg_pool2d, torch.nn.functional.avg_pool2d)):
        y = ours(x, k, s, p)
        yr = ref(xr, k, s, p)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        torch.testing.assert_close(y.float(), yr, rtol=tol, atol=tol)
        g = torch.randn_like(yr)
        (gx,) = torch.autograd.grad(y, x, g.to(dtype))
        (gr,) = torch.autograd.grad(yr, xr, g.to(dtype).float())
        torch.testing.assert_close(gx.float(), gr, rtol=tol, atol=tol * 4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batch_norm_train_eval_backward(dtype):
    torch.manual_seed(7)
    x = (torch.randn(8, 6, 11, 13, device=DEV) * 2 + 5).to(dtype).requires_grad_(True)
    gamma = (torch.rand(6, device=DEV) + 0.5).requires_grad_(True)
    beta = torch.randn(6, device=DEV).requires_grad_(True)
    rm, rv = torch.zeros(6, device=DEV), torch.ones(6, device=DEV)
    rm2, rv2 = rm.clone(), rv.clone()
    y = T.batch_norm(x, gamma, beta, rm, rv, True, 0.1, 1e-5)
    xr = x.detach().float().requires_grad_(True)
    gr_, br_ = gamma.detach().clone().requires_grad_(True), beta.detach().clone().requires_grad_(True)
    yr = torch.nn.functional.batch_norm(xr, rm2, rv2, gr_, br_, True, 0.1, 1e-5)
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    torch.testing.assert_close(y.float(), yr, rtol=tol, atol=tol)
    torch.testing.assert_close(rm, rm2, rtol=1e-3, atol=1e-3 if dtype == torch.float32 else 2e-2)
    torch.testing.assert_close(rv, rv2, rtol=1e-3 if dtype == torch.float32 else 2e-2, atol=1e-3)
    g = torch.randn_like(yr)
    dx, dg, db = torch.autograd.grad(y, (x, gamma, beta), g.to(dtype))
    dxr, dgr, dbr = torch.autograd.grad(yr, (xr, gr_, br_), g.to(dtype).float())
    torch.testing.assert_close(dx.float(), dxr, rtol=tol, atol=tol)
    torch.testing.assert_close(dg, dgr, rtol=tol, atol=tol * 20)
    torch.testing.assert_close(db, dbr, rtol=tol, atol=tol * 20)
    ye = T.batch_norm(x.detach(), gamma.detach(), beta.detach(), rm, rv, False)
    yer = torch.nn.functional.batch_norm(x.detach().float(), rm, rv, gamma.detach(), beta.detach(), False)
    torch.testing.assert_close(ye.float(), yer, rtol=tol, atol=tol)


@pytest.mark.parametrize("k,s,p,d", [((3, 3), (1, 1), (1, 1), (1, 1)), ((5, 3), (2, 2), (2, 1), (1, 1)), ((3, 3), (1, 2), (2, 2), (2, 2))])
def test_im2col_col2im(k, s, p, d):
    torch.manual_seed(8)
    x = torch.randn(2, 4, 17, 15, device=DEV)
    cols = T.im2col(x, k, s, p, d)
    ref = torch.nn.functional.unfold(x, k, d, p, s).transpose(1, 2).reshape(cols.shape)
    assert torch.equal(cols, ref)
    g = torch.randn_like(cols)
    back = T.col2im(g, x.shape, k, s, p, d)
    oh_ow = cols.shape[0] // 2
    ref_back = torch.nn.functional.fold(g.reshape(2, oh_ow, -1).transpose(1, 2), (17, 15), k, d, p, s)
    torch.testing.assert_close(back, ref_back, rtol=1e-5, atol=1e-5)
    assert torch.equal(T.im2col(x.bfloat16(), k, s, p, d), ref.bfloat16())


def test_q8_0_device_matches_cpu_codec():
    from incin_b200.ops import quant
    torch.manual_seed(9)
    x = torch.randn(1000 * 32 + 5) * 3
    x[64:96] = 0.0
    packed_cpu = quant.quantize_q8_0(x)
    packed = T.quantize_q8_0_cuda(x.to(DEV))
    assert torch.equal(packed.cpu(), packed_cpu)
    deq = T.dequantize_q8_0_cuda(packed, x.numel(), torch.float32)
    assert torch.equal(deq.cpu(), quant.dequantize_q8_0(packed_cpu, x.numel()))
    assert float((deq.cpu() - x).abs().max()) <= float(x.abs().max()) / 127 * 0.51
    assert T.dequantize_q8_0_cuda(packed, x.numel()).dtype == torch.bfloat16


def test_embedding_backward_deterministic_matches_atomic_version():
    torch.manual_seed(10)
    B, Tn, Cc, V = 4, 64, 96, 50
    tok = torch.randint(0, V, (B, Tn), device=DEV)
    dout = torch.randn(B, Tn, Cc, device=DEV).bfloat16()
    runs = []
    for _ in range(2):
        dwte, dwpe = torch.zeros(V, Cc, device=DEV), torch.zeros(Tn, Cc, device=DEV)
        T.embedding_bwd_deterministic(dout, tok, dwte, dwpe, Tn)
        runs.append((dwte, dwpe))
    assert torch.equal(runs[0][0], runs[1][0]) and torch.equal(runs[0][1], runs[1][1])
    want = torch.zeros(V, Cc, device=DEV).index_add_(0, tok.reshape(-1), dout.reshape(-1, Cc).float())
    torch.testing.assert_close(runs[0][0], want, rtol=1e-5, atol=1e-4)
    torch.testing.assert_close(runs[0][1], dout.float().sum(0), rtol=1e-5, atol=1e-4)
