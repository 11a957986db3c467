"""tcgen05 GEMM against a plain PyTorch fp32 reference of the same product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_inputs(shape, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(*shape, generator=g).to(torch.bfloat16).cuda()


def _close(out, ref, tol=2e-2):
    from _tol import check_close
    fp32_out = out.dtype == torch.float32
    out, ref = out.float(), ref.float()
    err = (out - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err <= tol * scale, f"max abs err {err} vs scale {scale}"
    # elementwise: bf16 outputs carry two ulps of rounding, fp32 outputs only the accumulation order
    check_close(out, ref, rtol=4e-3 if fp32_out else 1.6e-2, atol_rms=4e-3 if fp32_out else 1.5e-2, what="gemm")


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 256), (300, 200, 136), (1024, 768, 768), (77, 50, 8)])
@pytest.mark.parametrize("tile_n", [0, 64, 128, 192, 256])
def test_nt(M, N, K, tile_n):
    from incin_b200.ops import gemm as G
    x, w = _ref_inputs((M, K), 1), _ref_inputs((N, K), 2)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    G.gemm(x, w, out, M=M, N=N, K=K, lda=K, ldb=K, ldc=N, tile_n=tile_n)
    _close(out, x.float() @ w.float().T)
    G.check_status()


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (300, 200, 136), (512, 768, 3072)])
def test_nn_dgrad(M, N, K):
    from incin_b200.ops import gemm as G
    dy, w = _ref_inputs((M, N), 3), _ref_inputs((N, K), 4)
    dx = G.mm_nn(dy, w)
    _close(dx, dy.float() @ w.float())
    G.check_status()


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (1000, 200, 136), (4096, 768, 768)])
@pytest.mark.parametrize("splits", [1, 4, None])
def test_tn_wgrad_accumulate(M, N, K, splits):
    from incin_b200.ops import gemm as G
    dy, x = _ref_inputs((M, N), 5), _ref_inputs((M, K), 6)
    grad = torch.ones(N, K, dtype=torch.float32, device="cuda")
    G.mm_tn_accum(dy, x, grad, splits=splits)
    _close(grad, 1.0 + dy.float().T @ x.float(), tol=1e-2)
    G.check_status()


def test_mn_major_a_only_and_b_only():
    from incin_b200.ops import gemm as G
    M, N, K = 256, 192, 320
    at, b = _ref_inputs((K, M), 7), _ref_inputs((N, K), 8)  # A stored transposed
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    G.gemm(at, b, out, M=M, N=N, K=K, lda=M, ldb=K, ldc=N, a_mn=True)
    _close(out, at.float().T @ b.float().T)
    a, bt = _ref_inputs((M, K), 9), _ref_inputs((K, N), 10)
    G.gemm(a, bt, out, M=M, N=N, K=K, lda=K, ldb=N, ldc=N, b_mn=True)
    _close(out, a.float() @ bt.float())
    G.check_status()


def test_epilogues():
    from incin_b200 import _native as nat
    from incin_b200.ops import gemm as G
    M, N, K = 384, 320, 256
    x, w = _ref_inputs((M, K), 11), _ref_inputs((N, K), 12)
    bias, res = _ref_inputs((N,), 13), _ref_inputs((M, N), 14)
    ref = x.float() @ w.float().T * 0.125
    y = G.mm_nt(x, w, bias=bias, alpha=0.125)
    _close(y, ref + bias.float())
    y = G.mm_nt(x, w, bias=bias, residual=res, alpha=0.125)
    _close(y, ref + bias.float() + res.float())
    aux = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    y = G.mm_nt(x, w, bias=bias, act=nat.ACT_GELU, aux=aux, alpha=0.125)
    pre = ref + bias.float()
    _close(aux, pre)
    _close(y, torch.nn.functional.gelu(pre))
    # dgelu mask
    dy, w2 = _ref_inputs((M, K), 15), _ref_inputs((K, N), 16)
    out = G.mm_nn(dy, w2, act=nat.ACT_DGELU, aux=aux)
    a = aux.float().requires_grad_()
    torch.nn.functional.gelu(a).backward(dy.float() @ w2.float())
    _close(out, a.grad)
    G.check_status()


def test_batched_strided_heads():
    from incin_b200.ops import gemm as G
    B, T, H, D = 2, 256, 3, 64
    C = H * D
    qkv = _ref_inputs((B, T, 3 * C), 17)
    S = torch.empty(B * H, T, T, dtype=torch.bfloat16, device="cuda")
    ld = 3 * C
    G.gemm(qkv, qkv, S, M=T, N=T, K=D, lda=ld, ldb=ld, ldc=T, batch=(H, B), a_strides=(D, T * ld),
           b_strides=(D, T * ld), c_strides=(T * T, H * T * T), b_offset=C)
    q, k, v = qkv.float().view(B, T, 3, H, D).permute(2, 0, 3, 1, 4)
    _close(S.view(B, H, T, T), q @ k.transpose(-1, -2))
    G.check_status()


def test_general_matmul():
    from incin_b200.ops import gemm as G
    a, b = _ref_inputs((4, 96, 160), 18), _ref_inputs((4, 160, 72), 19)
    _close(G.matmul(a, b), a.float() @ b.float())


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 2e-3), (torch.float32, 2e-3), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (300, 200, 136), (1024, 768, 772), (77, 50, 12)])
def test_fp16_and_tf32_operands(dtype, tol, M, N, K):
    """fp16 operands and fp32 operands multiplied as tf32 run on the same kernel with fp32 output (K need not fill
    a 128-byte k-block: the tail is zero filled)."""
    from incin_b200.ops import gemm as G
    if dtype != torch.float32 and K % 8:
        K += 8 - K % 8
    g = torch.Generator(device="cpu").manual_seed(5)
    x = torch.randn(M, K, generator=g).to(dtype).cuda()
    w = torch.randn(N, K, generator=g).to(dtype).cuda()
    out = G.mm_nt_f32out(x, w, alpha=0.5)
    assert out.dtype == torch.float32
    _close(out, 0.5 * (x.double() @ w.double().T), tol=tol)
    G.check_status()


def test_linear_fp16_and_tf32_autograd():
    from incin_b200.core.policy import MathMode, policy_scope
    from incin_b200.ops import functional as F
    g = torch.Generator(device="cpu").manual_seed(9)
    for dtype, fast in ((torch.float16, False), (torch.float32, True)):
        x = torch.randn(4, 64, 96, generator=g).to(dtype).cuda().requires_grad_()
        w = (torch.randn(80, 96, generator=g) * 0.1).to(dtype).cuda().requires_grad_()
        b = torch.randn(80, generator=g).to(dtype).cuda().requires_grad_()
        dy = torch.randn(4, 64, 80, generator=g).to(dtype).cuda()
        with policy_scope(math=MathMode.FAST if fast else MathMode.PRECISE):
            assert F._f32acc_native(x, w)
            y = F.linear(x, w, b)
            y.backward(dy)
        xr, wr, br = (t.detach().double().requires_grad_() for t in (x, w, b))
        yr = xr @ wr.T + br
        yr.backward(dy.double())
        _close(y, yr, tol=4e-3)
        _close(x.grad, xr.grad, tol=4e-3)
        _close(w.grad, wr.grad, tol=4e-3)
        _close(b.grad, br.grad, tol=4e-3)
    # fp32 without the fast-math policy keeps full precision (library path)
    assert not F._f32acc_native(torch.zeros(8, 8, device="cuda"), torch.zeros(8, 8, device="cuda"))
