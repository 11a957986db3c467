"""Online-softmax (flash) causal attention on tcgen05 — front end.

``flash_supported`` reports whether the fused kernel covers a shape; callers fall
back to the composed GEMM + softmax path otherwise.
"""
from __future__ import annotations

import torch


def flash_supported(qkv: torch.Tensor, n_heads: int, head_dim: int) -> bool:
    return False


def flash_attention_packed(qkv, n_heads, head_dim, scale):
    raise NotImplementedError
