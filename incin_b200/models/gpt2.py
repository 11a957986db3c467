"""GPT-2 style decoder-only LM (pre-LayerNorm, learned positions, GELU MLP, tied LM head).

The reference ships no transformer model; this is new model code on the
framework's op surface for the data-parallel training benchmark
(GPT-2-small: 12 layers, d_model 768, 12 heads, MLP 3072, vocab 50257).

Per block the CUDA path launches: LayerNorm, QKV GEMM (+bias), attention,
projection GEMM (+bias +residual), LayerNorm, FC GEMM (+bias +GELU), FC GEMM
(+bias +residual) — all elementwise work rides in GEMM epilogues or the norm
kernels.  The vocabulary is padded to a multiple of 128 rows so LM-head tiles
are full; padded classes are masked inside the cross-entropy kernel.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import nn

from ..ops import functional as F


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_layer: int = 12
    n_head: int = 12
    d_model: int = 768
    d_mlp: int = 3072
    max_seq: int = 1024
    ln_eps: float = 1e-5
    init_std: float = 0.02

    @property
    def padded_vocab(self) -> int:
        return (self.vocab_size + 127) // 128 * 128

    @staticmethod
    def small() -> "GPT2Config":
        return GPT2Config()

    @staticmethod
    def tiny() -> "GPT2Config":
        return GPT2Config(vocab_size=509, n_layer=2, n_head=2, d_model=128, d_mlp=512, max_seq=128)

    def num_params(self) -> int:
        c, m = self.d_model, self.d_mlp
        per = 2 * 2 * c + (3 * c * c + 3 * c) + (c * c + c) + (m * c + m) + (c * m + c)
        return self.vocab_size * c + self.max_seq * c + self.n_layer * per + 2 * c

    def flops_per_token(self, seq: int) -> float:
        """Training FLOPs per token: 6 x matmul parameters + causal attention (fwd + bwd)."""
        c, m = self.d_model, self.d_mlp
        mat = self.n_layer * (4 * c * c + 2 * c * m) + self.vocab_size * c
        attn = self.n_layer * 2 * seq * c  # QK^T and PV, causal half
        return 6.0 * mat + 6.0 * attn


class Block(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        c, m = cfg.d_model, cfg.d_mlp
        self.ln1_g = nn.Parameter(torch.ones(c))
        self.ln1_b = nn.Parameter(torch.zeros(c))
        self.qkv_w = nn.Parameter(torch.empty(3 * c, c))
        self.qkv_b = nn.Parameter(torch.zeros(3 * c))
        self.proj_w = nn.Parameter(torch.empty(c, c))
        self.proj_b = nn.Parameter(torch.zeros(c))
        self.ln2_g = nn.Parameter(torch.ones(c))
        self.ln2_b = nn.Parameter(torch.zeros(c))
        self.fc_w = nn.Parameter(torch.empty(m, c))
        self.fc_b = nn.Parameter(torch.zeros(m))
        self.out_w = nn.Parameter(torch.empty(c, m))
        self.out_b = nn.Parameter(torch.zeros(c))
        self.cfg = cfg

    def forward(self, x, bias_of_input=None, defer_out_bias: bool = False):
        """``bias_of_input``: the bias of the linear layer that produced ``x`` (the previous block's ``out_b``) when that
        layer left its bias gradient to the norm that consumes its output; ``defer_out_bias``: this block's ``out_b``
        gradient is left to whoever normalises the block's output.  The gradient that a norm's backward returns IS the
        output gradient of the linear in front of it, so its column sums cost no extra pass there, where the linear
        would need a launch that reads the whole gradient again."""
        cfg = self.cfg
        res, h = F.layernorm_fork(x, self.ln1_g, self.ln1_b, cfg.ln_eps, bias_of_input=bias_of_input)
        qkv = F.linear(h, self.qkv_w, self.qkv_b)
        a = F.causal_attention(qkv, cfg.n_head, cfg.d_model // cfg.n_head)
        x = F.linear(a, self.proj_w, self.proj_b, residual=res, defer_bias_grad=True)
        res, h = F.layernorm_fork(x, self.ln2_g, self.ln2_b, cfg.ln_eps, bias_of_input=self.proj_b)
        return F.mlp(h, self.fc_w, self.fc_b, self.out_w, self.out_b, act="gelu", residual=res,
                     defer_b2_grad=defer_out_bias)


class GPT2(nn.Module):
    def __init__(self, cfg: GPT2Config, seed: int = 0):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Parameter(torch.zeros(cfg.padded_vocab, cfg.d_model))
        self.wpe = nn.Parameter(torch.empty(cfg.max_seq, cfg.d_model))
        self.blocks = nn.ModuleList([Block(cfg) for _ in range(cfg.n_layer)])
        self.lnf_g = nn.Parameter(torch.ones(cfg.d_model))
        self.lnf_b = nn.Parameter(torch.zeros(cfg.d_model))
        self.wte._grad_uses = 2  # embedding and tied LM head both contribute to its gradient
        self.reset_parameters(seed)

    def reset_parameters(self, seed: int = 0) -> None:
        """Weights ~ N(0, init_std) from a seeded CPU generator (biases 0, norm gains 1)."""
        g = torch.Generator().manual_seed(seed)
        cfg = self.cfg
        with torch.no_grad():
            self.wte.zero_()
            self.wte[: cfg.vocab_size].normal_(0.0, cfg.init_std, generator=g)
            self.wpe.normal_(0.0, cfg.init_std, generator=g)
            for b in self.blocks:
                for w in (b.qkv_w, b.proj_w, b.fc_w, b.out_w):
                    w.normal_(0.0, cfg.init_std, generator=g)

    def forward(self, tokens: torch.Tensor, targets: torch.Tensor | None = None):
        cfg = self.cfg
        T = tokens.shape[1]
        assert T <= cfg.max_seq
        x = F.embedding(tokens, self.wte, self.wpe)
        prev_bias = None
        for b in self.blocks:       # every block's output is normalised next (by the next block or by the final norm)
            x = b(x, prev_bias, True)
            prev_bias = b.out_b
        h = F.layer_norm(x, self.lnf_g, self.lnf_b, cfg.ln_eps, bias_of_input=prev_bias)
        if targets is None:
            return F.linear(h, self.wte)[..., : cfg.vocab_size]   # tied LM head over the padded vocabulary
        return F.linear_cross_entropy(h, self.wte, targets, cfg.vocab_size)
