"""Baseline arm, NOT the product path: the same GPT-2 training step written with stock PyTorch —
cuBLAS GEMMs, SDPA attention, ATen LayerNorm/GELU/cross-entropy, fused torch AdamW, bf16 autocast
with fp32 parameters, DistributedDataParallel over NCCL (bucketed all-reduce overlapped with
backward).  It exists so every number of the hand-written sm_100a path is reported next to what the
vendor libraries do on the same box, same shapes, same synthetic data.
"""
from __future__ import annotations

import torch
import torch.nn.functional as TF
from torch import nn


class _Block(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        c = cfg.d_model
        self.ln1, self.ln2 = nn.LayerNorm(c, eps=cfg.ln_eps), nn.LayerNorm(c, eps=cfg.ln_eps)
        self.qkv, self.proj = nn.Linear(c, 3 * c), nn.Linear(c, c)
        self.fc, self.out = nn.Linear(c, cfg.d_mlp), nn.Linear(cfg.d_mlp, c)
        self.h = cfg.n_head

    def forward(self, x):
        B, T, C = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, T, 3, self.h, C // self.h).permute(2, 0, 3, 1, 4)
        a = TF.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, C)
        x = x + self.proj(a)
        return x + self.out(TF.gelu(self.fc(self.ln2(x))))


class TorchGPT2(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Embedding(cfg.padded_vocab, cfg.d_model)
        self.wpe = nn.Embedding(cfg.max_seq, cfg.d_model)
        self.blocks = nn.ModuleList([_Block(cfg) for _ in range(cfg.n_layer)])
        self.lnf = nn.LayerNorm(cfg.d_model, eps=cfg.ln_eps)
        for p in self.parameters():
            if p.dim() >= 2:
                nn.init.normal_(p, 0.0, cfg.init_std)

    def forward(self, tok, tgt):
        T = tok.shape[1]
        x = self.wte(tok) + self.wpe.weight[:T]
        for b in self.blocks:
            x = b(x)
        logits = TF.linear(self.lnf(x), self.wte.weight)[..., : self.cfg.vocab_size]
        return TF.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), tgt.reshape(-1))


def build_torch_baseline(cfg, device, world: int):
    torch.manual_seed(0)
    model = TorchGPT2(cfg).to(device)
    net = model
    if world > 1:
        from torch.nn.parallel import DistributedDataParallel as DDP
        net = DDP(model, device_ids=[device.index], gradient_as_bucket_view=True)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)

    def step(tok, tgt):
        opt.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = net(tok, tgt)
        loss.backward()
        opt.step()
        return loss.detach()

    return step, ("nccl-ddp" if world > 1 else "none")
