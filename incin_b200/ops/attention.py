"""Causal online-softmax (flash) attention on tcgen05 — Python front end.

``flash_attention(q, k, v)`` takes ``[B, T, H, D]`` views (any strides whose innermost dimension is
contiguous, so slices of a packed QKV projection work in place), supports grouped-query attention
(``Hq`` a multiple of ``Hkv``) and head_dim 64 / 128, and is differentiable.  The forward keeps only
O and the per-row log-sum-exp; the backward recomputes the probabilities tile by tile.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from .. import _native as nat
from .gemm import status_word

c_void_p, c_int, c_ll, c_float = C.c_void_p, C.c_int, C.c_longlong, C.c_float


class AttnDesc(C.Structure):
    _fields_ = (
        [("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("o", c_void_p), ("lse", c_void_p),
         ("B", c_int), ("T", c_int), ("Hq", c_int), ("Hkv", c_int), ("D", c_int), ("scale", c_float)]
        + [(f"{n}_stride_{a}", c_ll) for n in ("q", "k", "v", "o") for a in ("b", "t", "h")]
        + [("d_o", c_void_p)] + [(f"do_stride_{a}", c_ll) for a in ("b", "t", "h")]
        + [("dq", c_void_p), ("dk", c_void_p), ("dv", c_void_p)]
        + [(f"{n}_stride_{a}", c_ll) for n in ("dq", "dk", "dv") for a in ("b", "t", "h")]
        + [("delta", c_void_p), ("dq_accum", c_void_p), ("status", c_void_p)]
    )


nat.register_cuda_signatures({
    "incin_flash_attn_fwd": (c_int, [C.POINTER(AttnDesc), c_void_p]),
    "incin_flash_attn_bwd": (c_int, [C.POINTER(AttnDesc), c_void_p]),
})


def _ok_view(t: torch.Tensor) -> bool:
    return (t.dim() == 4 and t.stride(3) == 1 and all(s % 8 == 0 for s in t.stride()[:3])
            and t.data_ptr() % 16 == 0 and t.dtype == torch.bfloat16)


def _set(d: AttnDesc, name: str, t: torch.Tensor) -> None:
    setattr(d, name if name != "do" else "d_o", t.data_ptr())
    sb, st, sh, _ = t.stride()
    setattr(d, f"{name}_stride_b", sb)
    setattr(d, f"{name}_stride_t", st)
    setattr(d, f"{name}_stride_h", sh)


def flash_shape_supported(T: int, head_dim: int, hq: int, hkv: int) -> bool:
    return head_dim in (64, 128) and hq % hkv == 0


class _Flash(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale):
        B, T, Hq, D = q.shape
        Hkv = k.shape[2]
        o = torch.empty(B, T, Hq, D, dtype=torch.bfloat16, device=q.device)
        lse = torch.empty(B, Hq, (T + 127) // 128 * 128, dtype=torch.float32, device=q.device)
        d = AttnDesc()
        d.B, d.T, d.Hq, d.Hkv, d.D, d.scale = B, T, Hq, Hkv, D, scale
        _set(d, "q", q), _set(d, "k", k), _set(d, "v", v), _set(d, "o", o)
        d.lse = lse.data_ptr()
        d.status = status_word(q.device).data_ptr()
        nat.check(nat.cuda().incin_flash_attn_fwd(C.byref(d), nat.stream_ptr()), "flash_attn_fwd")
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        B, T, Hq, D = q.shape
        Hkv = k.shape[2]
        if not _ok_view(do):
            do = do.contiguous()
        # gradients are produced in one packed [B, T, Hq + 2 Hkv, D] buffer so that a packed-QKV caller
        # gets a single contiguous gradient back through autograd's view backward with no concatenation
        packed = torch.empty(B, T, Hq + 2 * Hkv, D, dtype=torch.bfloat16, device=q.device)
        dq, dk, dv = packed[:, :, :Hq], packed[:, :, Hq:Hq + Hkv], packed[:, :, Hq + Hkv:]
        delta = torch.empty_like(lse)
        acc = torch.empty(B, T, Hq, D, dtype=torch.float32, device=q.device)
        d = AttnDesc()
        d.B, d.T, d.Hq, d.Hkv, d.D, d.scale = B, T, Hq, Hkv, D, ctx.scale
        _set(d, "q", q), _set(d, "k", k), _set(d, "v", v), _set(d, "o", o), _set(d, "do", do)
        _set(d, "dq", dq), _set(d, "dk", dk), _set(d, "dv", dv)
        d.lse, d.delta, d.dq_accum = lse.data_ptr(), delta.data_ptr(), acc.data_ptr()
        d.status = status_word(q.device).data_ptr()
        nat.check(nat.cuda().incin_flash_attn_bwd(C.byref(d), nat.stream_ptr()), "flash_attn_bwd")
        return dq, dk, dv, None


def flash_attention(q, k, v, scale: float | None = None):
    """Causal attention; q ``[B,T,Hq,D]``, k/v ``[B,T,Hkv,D]`` -> ``[B,T,Hq,D]`` (bf16, CUDA)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    q, k, v = (t if _ok_view(t) else t.contiguous() for t in (q, k, v))
    return _Flash.apply(q, k, v, scale)


class _FlashPacked(torch.autograd.Function):
    """Packed ``[B, T, (Hq + 2 Hkv) * D]`` QKV in, ``[B, T, Hq * D]`` out; the gradient is one packed tensor."""

    @staticmethod
    def forward(ctx, qkv, Hq, Hkv, D, scale):
        B, T, _ = qkv.shape
        x = qkv.view(B, T, Hq + 2 * Hkv, D)
        q, k, v = x[:, :, :Hq], x[:, :, Hq:Hq + Hkv], x[:, :, Hq + Hkv:]
        o = torch.empty(B, T, Hq, D, dtype=torch.bfloat16, device=qkv.device)
        lse = torch.empty(B, Hq, (T + 127) // 128 * 128, dtype=torch.float32, device=qkv.device)
        d = AttnDesc()
        d.B, d.T, d.Hq, d.Hkv, d.D, d.scale = B, T, Hq, Hkv, D, scale
        _set(d, "q", q), _set(d, "k", k), _set(d, "v", v), _set(d, "o", o)
        d.lse = lse.data_ptr()
        d.status = status_word(qkv.device).data_ptr()
        nat.check(nat.cuda().incin_flash_attn_fwd(C.byref(d), nat.stream_ptr()), "flash_attn_fwd")
        ctx.save_for_backward(qkv, o, lse)
        ctx.dims = (Hq, Hkv, D, scale)
        return o.view(B, T, Hq * D)

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse = ctx.saved_tensors
        Hq, Hkv, D, scale = ctx.dims
        B, T, _ = qkv.shape
        do = do.contiguous().view(B, T, Hq, D)
        x = qkv.view(B, T, Hq + 2 * Hkv, D)
        q, k, v = x[:, :, :Hq], x[:, :, Hq:Hq + Hkv], x[:, :, Hq + Hkv:]
        dqkv = torch.empty_like(x)
        dq, dk, dv = dqkv[:, :, :Hq], dqkv[:, :, Hq:Hq + Hkv], dqkv[:, :, Hq + Hkv:]
        delta = torch.empty_like(lse)
        acc = torch.empty(B, T, Hq, D, dtype=torch.float32, device=qkv.device)
        d = AttnDesc()
        d.B, d.T, d.Hq, d.Hkv, d.D, d.scale = B, T, Hq, Hkv, D, scale
        _set(d, "q", q), _set(d, "k", k), _set(d, "v", v), _set(d, "o", o), _set(d, "do", do)
        _set(d, "dq", dq), _set(d, "dk", dk), _set(d, "dv", dv)
        d.lse, d.delta, d.dq_accum = lse.data_ptr(), delta.data_ptr(), acc.data_ptr()
        d.status = status_word(qkv.device).data_ptr()
        nat.check(nat.cuda().incin_flash_attn_bwd(C.byref(d), nat.stream_ptr()), "flash_attn_bwd")
        return dqkv.view(B, T, -1), None, None, None, None


def flash_supported(qkv: torch.Tensor, n_heads: int, head_dim: int, n_kv_heads: int | None = None) -> bool:
    hkv = n_kv_heads or n_heads
    return (qkv.is_cuda and qkv.dtype == torch.bfloat16 and head_dim in (64, 128) and n_heads % hkv == 0
            and qkv.shape[-1] == (n_heads + 2 * hkv) * head_dim)


def flash_attention_packed(qkv, n_heads, head_dim, scale, n_kv_heads: int | None = None):
    qkv = qkv if qkv.is_contiguous() else qkv.contiguous()
    return _FlashPacked.apply(qkv, n_heads, n_kv_heads or n_heads, head_dim, scale)
