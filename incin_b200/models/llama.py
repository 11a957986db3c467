"""Llama-style decoder-only LM: RMSNorm, rotary positions, grouped-query attention, SwiGLU FFN, untied LM head.

New model code on the framework's op surface (the reference has no RoPE, SwiGLU layer, GQA or causal-mask
helper).  Presets match the tensor-parallel and 2-D-mesh benchmark configurations:

* ``llama_1b``: 22 layers, d_model 2048, 32 query / 4 KV heads, head_dim 64, FFN 5632, vocab 32000;
* ``llama_3b``: 26 layers, d_model 3072, 24 query / 8 KV heads, head_dim 128, FFN 8192, vocab 32000.

Per block on CUDA: RMSNorm -> fused QKV GEMM -> RoPE (q and k heads, in place) -> flash attention (GQA) ->
output GEMM (+residual) -> RMSNorm -> fused gate/up GEMM -> SwiGLU -> down GEMM (+residual).  With a
:class:`~incin_b200.parallel.tp.TensorParallel` context the four GEMMs become the fused
all-gather->GEMM / GEMM->reduce-scatter kernels and activations between blocks stay sharded over tokens.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from ..ops import functional as F


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    n_layer: int = 22
    d_model: int = 2048
    n_head: int = 32
    n_kv_head: int = 4
    head_dim: int = 64
    d_ffn: int = 5632
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    init_std: float = 0.02
    max_seq: int = 4096

    @staticmethod
    def llama_1b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def llama_3b() -> "LlamaConfig":
        return LlamaConfig(n_layer=26, d_model=3072, n_head=24, n_kv_head=8, head_dim=128, d_ffn=8192)

    @staticmethod
    def tiny() -> "LlamaConfig":
        return LlamaConfig(vocab_size=512, n_layer=2, d_model=256, n_head=4, n_kv_head=2, head_dim=64, d_ffn=512,
                           max_seq=256)

    @property
    def qkv_dim(self) -> int:
        return (self.n_head + 2 * self.n_kv_head) * self.head_dim

    def num_params(self) -> int:
        c = self.d_model
        per = c * self.qkv_dim + self.n_head * self.head_dim * c + 3 * c * self.d_ffn + 2 * c
        return 2 * self.vocab_size * c + self.n_layer * per + c

    def flops_per_token(self, seq: int) -> float:
        c = self.d_model
        mat = self.n_layer * (c * self.qkv_dim + self.n_head * self.head_dim * c + 3 * c * self.d_ffn) + self.vocab_size * c
        attn = self.n_layer * 2 * seq * self.n_head * self.head_dim
        return 6.0 * mat + 6.0 * attn


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        c = cfg.d_model
        self.cfg = cfg
        self.attn_norm = nn.Parameter(torch.ones(c))
        self.qkv_w = nn.Parameter(torch.empty(cfg.qkv_dim, c))
        self.o_w = nn.Parameter(torch.empty(c, cfg.n_head * cfg.head_dim))
        self.ffn_norm = nn.Parameter(torch.ones(c))
        self.gate_up_w = nn.Parameter(torch.empty(2 * cfg.d_ffn, c))
        self.down_w = nn.Parameter(torch.empty(c, cfg.d_ffn))

    def forward(self, x):
        cfg = self.cfg
        B, T, _ = x.shape
        res, h = F.rmsnorm_fork(x, self.attn_norm, cfg.rms_eps)
        qkv = F.linear(h, self.qkv_w)
        qkv = F.rope(qkv.view(B, T, cfg.n_head + 2 * cfg.n_kv_head, cfg.head_dim), cfg.n_head + cfg.n_kv_head,
                     cfg.head_dim, cfg.rope_theta).view(B, T, cfg.qkv_dim)
        a = F.gqa_attention(qkv, cfg.n_head, cfg.n_kv_head, cfg.head_dim)
        x = F.linear(a, self.o_w, residual=res)
        res, h = F.rmsnorm_fork(x, self.ffn_norm, cfg.rms_eps)
        g = F.swiglu(F.linear(h, self.gate_up_w))
        return F.linear(g, self.down_w, residual=res)


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig, seed: int = 0):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.d_model))
        self.blocks = nn.ModuleList([LlamaBlock(cfg) for _ in range(cfg.n_layer)])
        self.final_norm = nn.Parameter(torch.ones(cfg.d_model))
        self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.d_model))
        self.reset_parameters(seed)

    def reset_parameters(self, seed: int = 0) -> None:
        g = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for p in self.parameters():
                if p.dim() >= 2:
                    p.normal_(0.0, self.cfg.init_std, generator=g)

    def forward(self, tokens, targets=None):
        cfg = self.cfg
        x = F.embedding(tokens, self.embed, None)
        for b in self.blocks:
            x = b(x)
        h = F.rms_norm(x, self.final_norm, cfg.rms_eps)
        if targets is None:
            return F.linear(h, self.lm_head)
        return F.linear_cross_entropy(h, self.lm_head, targets, cfg.vocab_size)
