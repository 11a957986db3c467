"""tcgen05 flash attention forward/backward against an fp32 PyTorch reference of the same math."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, scale):
    # q [B,T,Hq,D], k/v [B,T,Hkv,D] in fp32
    B, T, Hq, D = q.shape
    g = Hq // k.shape[2]
    k = k.repeat_interleave(g, dim=2)
    v = v.repeat_interleave(g, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, k) * scale
    mask = torch.ones(T, T, device=q.device, dtype=torch.bool).tril()
    p = torch.softmax(s.masked_fill(~mask, float("-inf")), dim=-1)
    return torch.einsum("bhqk,bkhd->bqhd", p, v)


def _err(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


def _elementwise(a, b, what):
    from _tol import check_close
    # P and dS are rounded to bf16 before the second products, so gradients carry a few bf16 ulps of noise
    check_close(a, b, rtol=3e-2, atol_rms=8e-2, min_cos=0.9998, what=what)


@pytest.mark.parametrize("B,T,Hq,Hkv,D", [(1, 128, 1, 1, 64), (2, 256, 2, 2, 64), (1, 384, 4, 2, 64), (2, 200, 2, 1, 64),
                                          (1, 128, 1, 1, 128), (1, 512, 2, 2, 128), (1, 320, 4, 1, 128),
                                          (1, 1024, 2, 2, 64), (2, 640, 6, 2, 64),
                                          (1, 2048, 2, 1, 128), (2, 1000, 4, 2, 128), (1, 64, 2, 2, 128),
                                          (1, 2304, 1, 1, 128)])
def test_flash_fwd_bwd(B, T, Hq, Hkv, D):
    from incin_b200.ops import attention as A
    from incin_b200.ops import gemm as G
    g = torch.Generator().manual_seed(T + D)
    mk = lambda h: (torch.randn(B, T, h, D, generator=g) * 0.8).to(torch.bfloat16).cuda()
    q, k, v, do = mk(Hq), mk(Hkv), mk(Hkv), mk(Hq)
    scale = 1.0 / math.sqrt(D)
    qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
    ref = _ref(qf, kf, vf, scale)
    ref.backward(do.float())
    q1, k1, v1 = (t.clone().requires_grad_() for t in (q, k, v))
    out = A.flash_attention(q1, k1, v1, scale)
    G.check_status()
    assert _err(out, ref) < 2e-2, _err(out, ref)
    out.backward(do)
    G.check_status()
    assert _err(q1.grad, qf.grad) < 3e-2, ("dq", _err(q1.grad, qf.grad))
    assert _err(k1.grad, kf.grad) < 3e-2, ("dk", _err(k1.grad, kf.grad))
    assert _err(v1.grad, vf.grad) < 3e-2, ("dv", _err(v1.grad, vf.grad))
    _elementwise(out, ref, f"attn out T{T} D{D}")
    _elementwise(q1.grad, qf.grad, f"attn dq T{T} D{D}")
    _elementwise(k1.grad, kf.grad, f"attn dk T{T} D{D}")
    _elementwise(v1.grad, vf.grad, f"attn dv T{T} D{D}")


def test_flash_packed_matches_composed():
    from incin_b200.ops import functional as F
    B, T, H, D = 2, 256, 4, 64
    g = torch.Generator().manual_seed(0)
    qkv = (torch.randn(B, T, 3 * H * D, generator=g) * 0.7).to(torch.bfloat16).cuda()
    do = torch.randn(B, T, H * D, generator=g).to(torch.bfloat16).cuda()
    outs = {}
    for impl in ("composed", "flash"):
        F.set_attention_impl(impl)
        x = qkv.clone().requires_grad_()
        o = F.causal_attention(x, H, D)
        o.backward(do)
        outs[impl] = (o.detach(), x.grad)
    F.set_attention_impl("auto")
    assert _err(outs["flash"][0], outs["composed"][0]) < 2e-2
    assert _err(outs["flash"][1], outs["composed"][1]) < 4e-2
