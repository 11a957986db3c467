"""Tensor-parallel (and data x tensor parallel) Llama: the same network as :mod:`incin_b200.models.llama`, with
parameters placed on a mesh and activations sharded over tokens between layers.

Placements (tensor-parallel axis):
  q / gate / up projection rows      Sharded(0)   (column-parallel: fused all-gather -> GEMM)
  attention-output / down columns    Sharded(1)   (row-parallel: fused GEMM -> reduce-scatter)
  K/V projection rows                Sharded(0) when ``n_kv_head >= tp``; otherwise every KV head is shared by
                                     ``tp / n_kv_head`` neighbouring ranks, which keep identical copies and sum its
                                     gradient among themselves each step
  embedding, LM head, norm gains     Replicated; every rank works on its own rows of the token batch, so their
                                     gradients are Partial(Sum) and are reduced + updated by the fused
                                     reduce-scatter/AdamW/all-gather kernel over the tensor-parallel group
Each rank computes the loss of its own ``M / tp`` rows scaled by ``1 / tp``; the sum over ranks is the global mean.
"""
from __future__ import annotations

import torch
from torch import nn

from ..ops import functional as F
from ..parallel.tp import PeerRangeSum, TensorParallel, column_parallel_linear, row_parallel_linear
from .llama import Llama, LlamaConfig


class LlamaBlockTP(nn.Module):
    def __init__(self, cfg: LlamaConfig, tp_world: int):
        super().__init__()
        c, D = cfg.d_model, cfg.head_dim
        assert cfg.n_head % tp_world == 0 and cfg.d_ffn % tp_world == 0
        assert cfg.n_kv_head % tp_world == 0 or tp_world % cfg.n_kv_head == 0
        self.cfg, self.tp_world = cfg, tp_world
        self.hq = cfg.n_head // tp_world
        self.hkv = max(1, cfg.n_kv_head // tp_world)
        self.fl = cfg.d_ffn // tp_world
        self.attn_norm = nn.Parameter(torch.ones(c))
        self.q_w = nn.Parameter(torch.empty(self.hq * D, c))
        self.kv_w = nn.Parameter(torch.empty(2 * self.hkv * D, c))
        self.o_w = nn.Parameter(torch.empty(c, self.hq * D))
        self.ffn_norm = nn.Parameter(torch.ones(c))
        self.gate_up_w = nn.Parameter(torch.empty(2 * self.fl, c))
        self.down_w = nn.Parameter(torch.empty(c, self.fl))

    def load_from(self, full, rank: int) -> None:
        """Slice this rank's shards out of a full :class:`LlamaBlock`."""
        cfg, D, tp = self.cfg, self.cfg.head_dim, self.tp_world
        Hq, Hkv = cfg.n_head, cfg.n_kv_head
        qkv = full.qkv_w.detach()
        q, k, v = qkv[: Hq * D], qkv[Hq * D:(Hq + Hkv) * D], qkv[(Hq + Hkv) * D:]
        kv_first = rank * self.hkv if Hkv >= tp else rank // (tp // Hkv)
        with torch.no_grad():
            self.attn_norm.copy_(full.attn_norm)
            self.ffn_norm.copy_(full.ffn_norm)
            self.q_w.copy_(q[rank * self.hq * D:(rank + 1) * self.hq * D])
            self.kv_w.copy_(torch.cat([k[kv_first * D:(kv_first + self.hkv) * D], v[kv_first * D:(kv_first + self.hkv) * D]]))
            self.o_w.copy_(full.o_w.detach()[:, rank * self.hq * D:(rank + 1) * self.hq * D])
            gu, Fd = full.gate_up_w.detach(), cfg.d_ffn
            self.gate_up_w.copy_(torch.cat([gu[rank * self.fl:(rank + 1) * self.fl], gu[Fd + rank * self.fl:Fd + (rank + 1) * self.fl]]))
            self.down_w.copy_(full.down_w.detach()[:, rank * self.fl:(rank + 1) * self.fl])

    def forward(self, x_shard, tp: TensorParallel, B: int, T: int, layer: int = 0):
        cfg, D = self.cfg, self.cfg.head_dim
        i = 4 * layer                                                                  # plan ids of this block's four linears
        res, h = F.rmsnorm_fork(x_shard, self.attn_norm, cfg.rms_eps)
        qkv = column_parallel_linear(h, tp, self.q_w, self.kv_w, tp_id=i)              # [B*T, (hq + 2 hkv) D]
        qkv = F.rope(qkv.view(B, T, self.hq + 2 * self.hkv, D), self.hq + self.hkv, D, cfg.rope_theta)
        a = F.gqa_attention(qkv.view(B, T, -1), self.hq, self.hkv, D)                  # [B, T, hq D]
        x_shard = row_parallel_linear(a.view(B * T, self.hq * D), tp, self.o_w, res, tp_id=i + 1)   # [B*T / tp, C]
        res, h = F.rmsnorm_fork(x_shard, self.ffn_norm, cfg.rms_eps)
        g = F.swiglu(column_parallel_linear(h, tp, self.gate_up_w, tp_id=i + 2))       # [B*T, F / tp]
        return row_parallel_linear(g, tp, self.down_w, res, tp_id=i + 3)


def tensor_parallel_plan(cfg: LlamaConfig, mesh, rank: int, tokens: int):
    """The tensor-parallel collectives of ONE training step of :class:`LlamaTP` in launch order, as a
    :class:`~incin_b200.parallel.plan.CollectivePlan`: per block, forward = all-gather (QKV), reduce-scatter
    (attention output), all-gather (gate / up), reduce-scatter (down); then the backward pass block by block in
    reverse, every linear running the adjoint of its forward collective.  ``tokens`` = B * T of the group.
    Linear ``k`` of block ``l`` has plan id ``4 l + k``; ids ``2 id`` / ``2 id + 1`` tag its forward / backward launch."""
    from ..parallel.strategies import TensorParallelPlanBuilder
    b = TensorParallelPlanBuilder(mesh, rank)
    c = cfg.d_model
    col_in = (tokens, c)                       # gathered activation of both column-parallel linears
    row_out = (tokens, c)                      # partial product of both row-parallel linears
    for layer in range(cfg.n_layer):
        i = 4 * layer
        b.push_column(2 * i, col_in, 0)
        b.push_row_scatter(2 * (i + 1), row_out, 0)
        b.push_column(2 * (i + 2), col_in, 0)
        b.push_row_scatter(2 * (i + 3), row_out, 0)
    for layer in reversed(range(cfg.n_layer)):
        i = 4 * layer
        b.push_column(2 * (i + 3) + 1, (tokens, c), 0)           # d(down): all-gather of the output-gradient shards
        b.push_row_scatter(2 * (i + 2) + 1, (tokens, c), 0)      # d(gate / up): reduce-scatter of the input gradient
        b.push_column(2 * (i + 1) + 1, (tokens, c), 0)           # d(attention output)
        b.push_row_scatter(2 * i + 1, (tokens, c), 0)            # d(QKV)
    return b.finish()


class LlamaTP(nn.Module):
    def __init__(self, cfg: LlamaConfig, tp_world: int, tp_rank: int):
        super().__init__()
        self.cfg, self.tp_world, self.tp_rank = cfg, tp_world, tp_rank
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.d_model))
        self.blocks = nn.ModuleList([LlamaBlockTP(cfg, tp_world) for _ in range(cfg.n_layer)])
        self.final_norm = nn.Parameter(torch.ones(cfg.d_model))
        self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.d_model))
        self.tp: TensorParallel | None = None

    @staticmethod
    def from_seed(cfg: LlamaConfig, tp_world: int, tp_rank: int, seed: int = 0) -> "LlamaTP":
        """Same weights as ``Llama(cfg, seed)``, sliced for this rank (built layer by layer on the host)."""
        full = Llama(cfg, seed)
        m = LlamaTP(cfg, tp_world, tp_rank)
        with torch.no_grad():
            m.embed.copy_(full.embed)
            m.lm_head.copy_(full.lm_head)
            m.final_norm.copy_(full.final_norm)
        for b, fb in zip(m.blocks, full.blocks):
            b.load_from(fb, tp_rank)
        return m

    def replicated_parameters(self):
        out = [("embed", self.embed), ("lm_head", self.lm_head), ("final_norm", self.final_norm)]
        for i, b in enumerate(self.blocks):
            out += [(f"blocks.{i}.attn_norm", b.attn_norm), (f"blocks.{i}.ffn_norm", b.ffn_norm)]
        return out

    def sharded_parameters(self):
        out = []
        for i, b in enumerate(self.blocks):
            out += [(f"blocks.{i}.{n}", getattr(b, n)) for n in ("q_w", "kv_w", "o_w", "gate_up_w", "down_w")]
        return out

    def kv_shared(self) -> int:
        """Number of neighbouring ranks that hold the same K/V head (1 = K/V projections are plainly sharded)."""
        return max(1, self.tp_world // self.cfg.n_kv_head)

    def forward(self, tokens, targets):
        """tokens/targets: the FULL ``[B, T]`` batch of this tensor-parallel group (identical on its ranks)."""
        cfg, tp = self.cfg, self.tp
        B, T = tokens.shape
        M = B * T
        Ml = M // tp.world
        lo = tp.rank * Ml
        tok = tokens.reshape(-1)[lo:lo + Ml].reshape(1, Ml)
        x = F.embedding(tok, self.embed, None).view(Ml, cfg.d_model)
        tp.begin_step()
        for li, b in enumerate(self.blocks):
            x = b(x, tp, B, T, li)
        h = F.rms_norm(x, self.final_norm, cfg.rms_eps)
        loss = F.linear_cross_entropy(h, self.lm_head, targets.reshape(-1)[lo:lo + Ml], cfg.vocab_size)
        return loss * (1.0 / tp.world)


class TPOptimizer:
    """Drives the two parameter groups of a tensor-parallel model behind the optimiser interface the training
    step expects: replicated parameters go through the fused reduce-scatter + AdamW + all-gather kernel over the
    reduction group; sharded parameters get the local flat AdamW (after the K/V pair sum, and after the
    data-parallel reduction when there is a data axis)."""

    def __init__(self, model: LlamaTP, tp: TensorParallel, device, *, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1,
                 dp_group=None, world_group=None, session=None, dp_ranks=None):
        """``session``: the collective session of the job (plan agreement before peer mappings, handles over its
        control channel); the reducers take it with the ranks of their groups (``tp.ranks``, ``dp_ranks``)."""
        from ..optim.flat import AdamW, ParamStore
        from ..parallel.dp import FusedReducer
        import torch.distributed as dist
        self.model, self.tp, self.device = model, tp, device
        dp = dist.get_world_size(dp_group) if dp_group is not None else 1
        # replicated group: reduced over every rank that holds a copy (tp x dp)
        from ..parallel.mesh import Axis
        rep_ranks = None
        if session is not None and session.ctx is not None:
            rep_ranks = list(range(session.ctx.world)) if dp > 1 else tp.ranks
        self.rep_reducer = FusedReducer(device, world_group if dp > 1 else tp.group, overlap=False, session=session,
                                        ranks=rep_ranks, axis=Axis.TENSOR, plan_ranks=tp.ranks)
        self.rep_store = ParamStore(model.replicated_parameters(), allocator=self.rep_reducer.allocator)
        self.rep_opt = AdamW(self.rep_store, lr=lr, betas=betas, weight_decay=weight_decay)
        self.rep_reducer.attach(self.rep_store, self.rep_opt)
        self.rep_opt.grad_scale = float(tp.world)          # sum over tp (local losses carry 1/tp), mean over dp
        # sharded group
        self.dp_reducer = FusedReducer(device, dp_group, overlap=False, session=session, ranks=dp_ranks) if dp > 1 else None
        alloc = self.dp_reducer.allocator if self.dp_reducer else None
        self.kv_share = model.kv_shared()
        self._grad_buf = None
        if self.kv_share > 1 and alloc is None:
            from ..parallel.symm import SymmetricBuffer
            holder = {}
            def alloc(n, dtype, dev):   # gradients must be peer-mapped for the K/V pair sum
                if dtype == torch.float32:
                    holder["g"] = SymmetricBuffer(n * 4, torch.device(dev))
                    return holder["g"].typed(torch.float32, n)
                return torch.zeros(n, dtype=dtype, device=dev)
            self.sh_store = ParamStore(model.sharded_parameters(), allocator=alloc)
            self._grad_buf = holder["g"].exchange(tp.group, session=session, ranks=tp.ranks)
        else:
            self.sh_store = ParamStore(model.sharded_parameters(), allocator=alloc)
            if self.dp_reducer is not None and self.kv_share > 1:
                # the reducer mapped the gradient buffer over the data axis; the K/V pair sum needs the mappings of the
                # tensor-parallel neighbours, so the same memory is mapped a second time over that group
                mine = next(b for b in self.dp_reducer._bufs if b.ptr == self.sh_store.grad.data_ptr())
                self._grad_buf = mine.mapped_over(tp.group, session=session, ranks=tp.ranks)
        self.sh_opt = AdamW(self.sh_store, lr=lr, betas=betas, weight_decay=weight_decay)
        if self.dp_reducer is not None:
            self.dp_reducer.attach(self.sh_store, self.sh_opt)
        if self.kv_share > 1:
            ranges = [(o, k) for n, p, o, k in self.sh_store.entries if n.endswith("kv_w")]
            base = (tp.rank // self.kv_share) * self.kv_share
            self._kv_sum = PeerRangeSum(self._grad_buf, ranges, list(range(base, base + self.kv_share)), tp.rank, tp,
                                        device)
        self.store = self
        self.lr, self.step_count = lr, 0

    # ParamStore-like face used by the training step
    def zero_grad(self) -> None:
        self.rep_store.zero_grad()
        self.sh_store.zero_grad()

    def collect_autograd_grads(self) -> None:
        pass

    @property
    def device(self):
        return self._device

    @device.setter
    def device(self, d):
        self._device = d

    def set_lr(self, lr: float) -> None:
        self.lr = lr
        self.rep_opt.set_lr(lr)
        self.sh_opt.set_lr(lr)

    def prepare_step(self) -> None:
        self.step_count += 1
        self.rep_opt.prepare_step()
        self.sh_opt.prepare_step()

    def launch(self) -> None:
        if self.kv_share > 1:
            self._kv_sum.run()
        self.rep_reducer.begin_step()
        self.rep_reducer.finish_step(self.rep_opt)
        if self.dp_reducer is not None:
            self.dp_reducer.begin_step()
            self.dp_reducer.finish_step(self.sh_opt)
        else:
            self.sh_opt.launch()
