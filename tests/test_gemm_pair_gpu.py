"""CTA-pair (cta_group::2) tcgen05 GEMM, selected with ``tile_n=512``, against plain PyTorch fp32 products."""
import pytest
import torch

pytestmark = pytest.mark.gpu
PAIR = 512


def _rand(shape, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(*shape, generator=g).to(torch.bfloat16).cuda()


def _close(out, ref, tol=2e-2):
    from _tol import check_close
    fp32_out = out.dtype == torch.float32
    out, ref = out.float(), ref.float()
    err = (out - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err <= tol * scale, f"max abs err {err} vs scale {scale}"
    check_close(out, ref, rtol=4e-3 if fp32_out else 1.6e-2, atol_rms=4e-3 if fp32_out else 1.5e-2, what="gemm pair")


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (256, 256, 512), (512, 768, 768), (300, 200, 136), (2048, 2304, 768),
                                   (77, 50, 8), (128, 512, 256), (4096, 4096, 1024)])
def test_pair_nt(M, N, K):
    from incin_b200.ops import gemm as G
    x, w = _rand((M, K), 1), _rand((N, K), 2)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    G.gemm(x, w, out, M=M, N=N, K=K, lda=K, ldb=K, ldc=N, tile_n=PAIR)
    G.check_status()
    _close(out, x.float() @ w.float().T)


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (304, 200, 136), (1024, 768, 3072)])
def test_pair_nn_and_tn(M, N, K):
    from incin_b200.ops import gemm as G
    a, bt = _rand((M, K), 3), _rand((K, N), 4)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    G.gemm(a, bt, out, M=M, N=N, K=K, lda=K, ldb=N, ldc=N, b_mn=True, tile_n=PAIR)
    G.check_status()
    _close(out, a.float() @ bt.float())
    at = _rand((K, M), 5)
    acc = torch.ones(M, N, dtype=torch.float32, device="cuda")
    G.gemm(at, bt, acc, M=M, N=N, K=K, lda=M, ldb=N, ldc=N, a_mn=True, b_mn=True, accumulate=True, splits=2, tile_n=PAIR)
    G.check_status()
    _close(acc, 1.0 + at.float().T @ bt.float(), tol=1e-2)


def test_pair_epilogues_match_single_cta_kernel():
    from incin_b200 import _native as nat
    from incin_b200.ops import gemm as G
    M, N, K = 512, 1024, 256
    x, w = _rand((M, K), 6), _rand((N, K), 7)
    bias, res = _rand((N,), 8), _rand((M, N), 9)
    outs = {}
    for tile in (256, PAIR):
        out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        aux = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        G.gemm(x, w, out, M=M, N=N, K=K, lda=K, ldb=K, ldc=N, bias=bias, act=nat.ACT_GELU,
               aux=aux, residual=res, alpha=0.5, tile_n=tile)
        G.check_status()
        outs[tile] = (out, aux)
    assert torch.equal(outs[256][0], outs[PAIR][0]) and torch.equal(outs[256][1], outs[PAIR][1])
    pre = 0.5 * (x.float() @ w.float().T) + bias.float()
    _close(outs[PAIR][0], torch.nn.functional.gelu(pre) + res.float(), tol=3e-2)


def test_pair_batched():
    from incin_b200.ops import gemm as G
    B, M, N, K = 3, 256, 256, 128
    a, b = _rand((B, M, K), 10), _rand((B, N, K), 11)
    out = torch.empty(B, M, N, dtype=torch.bfloat16, device="cuda")
    G.gemm(a, b, out, M=M, N=N, K=K, lda=K, ldb=K, ldc=N, batch=(B, 1), a_strides=(M * K, 0), b_strides=(N * K, 0),
           c_strides=(M * N, 0), tile_n=PAIR)
    G.check_status()
    _close(out, torch.bmm(a.float(), b.float().transpose(1, 2)))
