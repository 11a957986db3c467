"""Q8_0 block quantisation: blocks of 32 values share one f16 scale (34 bytes per block).

Counterpart of ``QuantizedOps`` (crates/incin-core/src/tensor/backend.rs:817-829) and the CPU/CUDA
quantise / dequantise kernels (crates/incin-backends/src/cpu/ops/quant.rs, cuda/ops/kernels/quant.cu).
The packed layout is the GGUF ``Q8_0`` layout, so exported files are readable by GGML tools.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as nat
from ..core.dtype import DTypeId, size_bytes


def _host():
    h = nat.host()
    h.incin_cpu_quantize_q8_0.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
    h.incin_cpu_dequantize_q8_0.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
    return h


def quantize_q8_0(x: torch.Tensor) -> torch.Tensor:
    """fp32 values -> packed uint8 blocks (last block zero-padded)."""
    if x.is_cuda and x.dtype in (torch.float32, torch.bfloat16):
        from .tensor_ops import quantize_q8_0_cuda
        return quantize_q8_0_cuda(x.detach().reshape(-1))
    xf = x.detach().float().cpu().contiguous().reshape(-1)
    out = torch.empty(size_bytes(DTypeId.Q8_0, xf.numel()), dtype=torch.uint8)
    _host().incin_cpu_quantize_q8_0(xf.data_ptr(), out.data_ptr(), xf.numel())
    return out


def dequantize_q8_0(packed: torch.Tensor, numel: int) -> torch.Tensor:
    if packed.numel() != size_bytes(DTypeId.Q8_0, numel):
        raise ValueError("packed buffer size does not match the element count")
    if packed.is_cuda:
        from .tensor_ops import dequantize_q8_0_cuda
        return dequantize_q8_0_cuda(packed, numel, torch.float32)
    out = torch.empty(numel, dtype=torch.float32)
    _host().incin_cpu_dequantize_q8_0(packed.contiguous().data_ptr(), out.data_ptr(), numel)
    return out


def quantized_matmul(x: torch.Tensor, w_packed: torch.Tensor, out_features: int, in_features: int) -> torch.Tensor:
    """``x @ dequant(W)^T`` for a Q8_0-packed ``[out, in]`` weight (dequantise, then the regular matmul path:
    the tcgen05 GEMM for bf16 CUDA inputs)."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        from .tensor_ops import dequantize_q8_0_cuda
        w = dequantize_q8_0_cuda(w_packed.to(x.device), out_features * in_features).view(out_features, in_features)
    else:
        w = dequantize_q8_0(w_packed.cpu(), out_features * in_features).reshape(out_features, in_features)
        w = w.to(device=x.device, dtype=x.dtype)
    from .functional import linear
    return linear(x, w)
