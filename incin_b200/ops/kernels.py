"""One thin Python wrapper per native sm_100a kernel (tensor in, tensor out, no autograd).

These are the leaves the autograd functions in :mod:`incin_b200.ops.functional`
are built from.  Every wrapper launches on the current CUDA stream and never
synchronises, so a whole training step made of them can be captured in a CUDA
graph.  They require CUDA tensors: the CPU path of each op lives in
``functional`` (PyTorch CPU math) and in the C++ oracle.
"""
from __future__ import annotations

import torch

from .. import _native as nat

BF16 = torch.bfloat16
F32 = torch.float32


def _s() -> int:
    return nat.stream_ptr()


def layernorm_fwd(x, gamma, beta, eps):
    C = x.shape[-1]
    rows = x.numel() // C
    y = torch.empty_like(x)
    mean = torch.empty(rows, dtype=F32, device=x.device)
    rstd = torch.empty(rows, dtype=F32, device=x.device)
    nat.check(nat.cuda().incin_layernorm_fwd(x.data_ptr(), gamma.data_ptr(), nat.ptr(beta), y.data_ptr(),
                                            mean.data_ptr(), rstd.data_ptr(), rows, C, eps, _s()), "layernorm_fwd")
    return y, mean, rstd


def norm_bwd_scratch(rows: int, C: int, device) -> torch.Tensor:
    n = nat.cuda().incin_layernorm_bwd_scratch_floats(rows, C)
    return torch.empty(n, dtype=F32, device=device)


def layernorm_bwd(dy, x, gamma, mean, rstd, dx_add, dgamma, dbeta, dx_colsum=None):
    """``dx_colsum`` (fp32 ``[C]``, accumulated into): the column sums of the returned dx, i.e. the bias gradient of the
    linear layer in front of this norm on the residual stream.  They come out of the one-pass kernel for free
    (C % 8 == 0, C <= 1024, parameter gradients requested); otherwise one column-sum launch follows."""
    C = x.shape[-1]
    rows = x.numel() // C
    dx = torch.empty_like(x)
    if dx_colsum is not None:
        if dgamma is not None and C % 8 == 0 and C <= 1024:
            n = nat.cuda().incin_layernorm_bwd_colsum_scratch_floats(rows, C)
            scratch = torch.empty(n, dtype=F32, device=x.device)
            nat.check(nat.cuda().incin_layernorm_bwd_colsum(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(),
                                                           rstd.data_ptr(), nat.ptr(dx_add), dx.data_ptr(), nat.ptr(dgamma),
                                                           nat.ptr(dbeta), dx_colsum.data_ptr(), scratch.data_ptr(), rows, C,
                                                           _s()), "layernorm_bwd_colsum")
            return dx
        dx = layernorm_bwd(dy, x, gamma, mean, rstd, dx_add, dgamma, dbeta)
        colsum_accum(dx, dx_colsum)
        return dx
    scratch = norm_bwd_scratch(rows, C, x.device) if dgamma is not None else None
    nat.check(nat.cuda().incin_layernorm_bwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(),
                                            rstd.data_ptr(), nat.ptr(dx_add), dx.data_ptr(), nat.ptr(dgamma),
                                            nat.ptr(dbeta), nat.ptr(scratch), rows, C, _s()), "layernorm_bwd")
    return dx


def rmsnorm_fwd(x, gamma, eps):
    C = x.shape[-1]
    rows = x.numel() // C
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=F32, device=x.device)
    nat.check(nat.cuda().incin_rmsnorm_fwd(x.data_ptr(), gamma.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, C, eps,
                                          _s()), "rmsnorm_fwd")
    return y, rstd


def rmsnorm_bwd(dy, x, gamma, rstd, dx_add, dgamma):
    C = x.shape[-1]
    rows = x.numel() // C
    dx = torch.empty_like(x)
    scratch = norm_bwd_scratch(rows, C, x.device) if dgamma is not None else None
    nat.check(nat.cuda().incin_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), rstd.data_ptr(),
                                          nat.ptr(dx_add), dx.data_ptr(), nat.ptr(dgamma), nat.ptr(scratch), rows, C,
                                          _s()), "rmsnorm_bwd")
    return dx


def embedding_fwd(tokens, wte, wpe):
    B, T = tokens.shape
    C = wte.shape[1]
    out = torch.empty(B, T, C, dtype=BF16, device=wte.device)
    nat.check(nat.cuda().incin_embedding_fwd(tokens.data_ptr(), wte.data_ptr(), nat.ptr(wpe), out.data_ptr(), B, T, C,
                                            _s()), "embedding_fwd")
    return out


def embedding_bwd(dout, tokens, dwte, dwpe):
    B, T = tokens.shape
    C = dout.shape[-1]
    nat.check(nat.cuda().incin_embedding_bwd(dout.data_ptr(), tokens.data_ptr(), dwte.data_ptr(), nat.ptr(dwpe), B, T,
                                            C, _s()), "embedding_bwd")


def xent_fwd(logits2d, targets, V):
    rows, ld = logits2d.shape[0], logits2d.stride(0)
    loss = torch.empty(rows, dtype=F32, device=logits2d.device)
    lse = torch.empty(rows, dtype=F32, device=logits2d.device)
    nat.check(nat.cuda().incin_xent_fwd(logits2d.data_ptr(), targets.data_ptr(), loss.data_ptr(), lse.data_ptr(), rows,
                                       V, ld, _s()), "xent_fwd")
    return loss, lse


def xent_bwd_(logits2d, targets, lse, dloss, scale, V):
    rows, ld = logits2d.shape[0], logits2d.stride(0)
    nat.check(nat.cuda().incin_xent_bwd(logits2d.data_ptr(), targets.data_ptr(), lse.data_ptr(), nat.ptr(dloss), scale,
                                       rows, V, ld, _s()), "xent_bwd")
    return logits2d


def xent_fused_(logits2d, targets, scale, V):
    """Per-row loss and log-sum-exp; ``logits2d`` is overwritten by ``(softmax - onehot) * scale``."""
    rows, ld = logits2d.shape[0], logits2d.stride(0)
    loss = torch.empty(rows, dtype=F32, device=logits2d.device)
    lse = torch.empty(rows, dtype=F32, device=logits2d.device)
    nat.check(nat.cuda().incin_xent_fused(logits2d.data_ptr(), targets.data_ptr(), loss.data_ptr(), lse.data_ptr(), scale,
                                         rows, V, ld, _s()), "xent_fused")
    return loss, lse


def mean_f32(x):
    out = torch.empty((), dtype=F32, device=x.device)
    nat.check(nat.cuda().incin_mean_f32(x.data_ptr(), out.data_ptr(), x.numel(), _s()), "mean")
    return out


def causal_softmax_fwd_(scores, T, scale):
    nat.check(nat.cuda().incin_causal_softmax_fwd(scores.data_ptr(), scores.numel() // (T * T), T, scale, _s()),
              "causal_softmax_fwd")
    return scores


def causal_softmax_bwd_(dp, p, T, scale):
    nat.check(nat.cuda().incin_causal_softmax_bwd(dp.data_ptr(), p.data_ptr(), p.numel() // (T * T), T, scale, _s()),
              "causal_softmax_bwd")
    return dp


def colsum_accum(dy, dbias):
    N = dy.shape[-1]
    rows = dy.numel() // N
    nat.check(nat.cuda().incin_colsum_accum(dy.data_ptr(), dbias.data_ptr(), rows, N, N, _s()), "colsum")


def sumsq_nonfinite(x, out):
    nat.check(nat.cuda().incin_sumsq_nonfinite_f32(x.data_ptr(), x.numel(), out.data_ptr(), _s()), "sumsq")


def fill_f32_(x, value):
    nat.check(nat.cuda().incin_fill_f32(x.data_ptr(), value, x.numel(), _s()), "fill")
    return x


def cast_to_bf16(x, out=None):
    out = torch.empty(x.shape, dtype=BF16, device=x.device) if out is None else out
    nat.check(nat.cuda().incin_cast_f32_to_bf16(x.data_ptr(), out.data_ptr(), x.numel(), _s()), "cast")
    return out


def cast_to_f32(x, out=None):
    out = torch.empty(x.shape, dtype=F32, device=x.device) if out is None else out
    nat.check(nat.cuda().incin_cast_bf16_to_f32(x.data_ptr(), out.data_ptr(), x.numel(), _s()), "cast")
    return out


def act_fwd(x, act):
    y = torch.empty_like(x)
    nat.check(nat.cuda().incin_act_fwd(x.data_ptr(), y.data_ptr(), x.numel(), act, _s()), "act_fwd")
    return y


def act_bwd(dy, pre, act):
    dx = torch.empty_like(dy)
    nat.check(nat.cuda().incin_act_bwd(dy.data_ptr(), pre.data_ptr(), dx.data_ptr(), dy.numel(), act, _s()), "act_bwd")
    return dx


def swiglu_fwd(gate_up):
    F = gate_up.shape[-1] // 2
    rows = gate_up.numel() // (2 * F)
    y = torch.empty(*gate_up.shape[:-1], F, dtype=BF16, device=gate_up.device)
    nat.check(nat.cuda().incin_swiglu_fwd(gate_up.data_ptr(), y.data_ptr(), rows, F, _s()), "swiglu_fwd")
    return y


def swiglu_bwd(dy, gate_up):
    F = gate_up.shape[-1] // 2
    rows = gate_up.numel() // (2 * F)
    d = torch.empty_like(gate_up)
    nat.check(nat.cuda().incin_swiglu_bwd(dy.data_ptr(), gate_up.data_ptr(), d.data_ptr(), rows, F, _s()), "swiglu_bwd")
    return d


def rope_(x, B, T, H, D, stride_b, stride_t, stride_h, theta, inverse, offset=0):
    nat.check(nat.cuda().incin_rope(x.data_ptr() + 2 * offset, B, T, H, D, stride_b, stride_t, stride_h, theta,
                                   int(inverse), _s()), "rope")
    return x


def adamw_flat(master, m, v, grad, shadow, n_decay, hyper):
    nat.check(nat.cuda().incin_adamw_flat(master.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(),
                                         nat.ptr(shadow), master.numel(), n_decay, hyper.data_ptr(), _s()), "adamw")


def sgd_flat(master, mom, grad, shadow, n_decay, hyper):
    nat.check(nat.cuda().incin_sgd_flat(master.data_ptr(), nat.ptr(mom), grad.data_ptr(), nat.ptr(shadow),
                                       master.numel(), n_decay, hyper.data_ptr(), _s()), "sgd")


def philox_uniform(shape, seed, offset, device):
    out = torch.empty(shape, dtype=F32, device=device)
    nat.check(nat.cuda().incin_philox_uniform_f32(out.data_ptr(), out.numel(), seed, offset, _s()), "philox")
    return out


def philox_normal(shape, seed, offset, device, mean=0.0, std=1.0, dtype=F32):
    out = torch.empty(shape, dtype=dtype, device=device)
    fn = nat.cuda().incin_philox_normal_f32 if dtype == F32 else nat.cuda().incin_philox_normal_bf16
    nat.check(fn(out.data_ptr(), out.numel(), seed, offset, mean, std, _s()), "philox")
    return out


def dropout(x, p, seed, offset):
    y = torch.empty_like(x)
    nat.check(nat.cuda().incin_dropout_bf16(x.data_ptr(), y.data_ptr(), x.numel(), p, seed, offset, _s()), "dropout")
    return y
