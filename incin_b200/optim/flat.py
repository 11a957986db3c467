"""Flat parameter storage and the fused optimisers that run over it.

All parameters of a model live in three contiguous device buffers — a bf16
"shadow" the forward/backward kernels read, fp32 master weights, and an fp32
gradient buffer the backward kernels accumulate into — so one optimiser launch
covers the whole model and the data-parallel reduction works on large
contiguous buckets instead of one collective per parameter (the reference
issues one ncclAllReduce per parameter tensor after backward:
crates/incin-backends/src/dist/nccl.rs:606-632).

Layout: parameters that receive weight decay first, then the rest, each
sub-range padded to 64 elements so every view is 128-byte aligned (TMA needs
16).  Within each group parameters are stored in reverse registration order,
which is the order their gradients complete during backward, so gradient
buckets become ready front to back.

Optimiser arithmetic follows the reference's CPU contract
(crates/incin-backends/src/cpu/ops/optimizer.rs:10-75,
crates/incin-core/src/optim/mod.rs:39-261): SGD ``w -= lr * g``; AdamW with
bias-corrected moments and decoupled decay, defaults beta=(0.9, 0.999),
eps=1e-8, weight_decay=0.01; state-dict keys ``m.<name>`` / ``v.<name>`` plus
``step_count``.
"""
from __future__ import annotations

from typing import Callable, Iterable

import torch

from ..ops import kernels as K

ALIGN = 64


def _default_decay(name: str, p: torch.Tensor) -> bool:
    return p.dim() >= 2


class ParamStore:
    def __init__(self, named_params: Iterable[tuple[str, torch.nn.Parameter]], *, device=None,
                 compute_dtype=torch.bfloat16, decay_filter: Callable[[str, torch.Tensor], bool] = _default_decay,
                 allocator: Callable[[int, torch.dtype, torch.device], torch.Tensor] | None = None):
        seen: dict[int, str] = {}
        params: list[tuple[str, torch.nn.Parameter]] = []
        for name, p in named_params:
            if id(p) in seen:
                continue  # tied weights appear once
            seen[id(p)] = name
            params.append((name, p))
        if not params:
            raise ValueError("no parameters")
        self.device = torch.device(device) if device is not None else params[0][1].device
        self.compute_dtype = compute_dtype
        decay = [(n, p) for n, p in params if decay_filter(n, p)][::-1]
        rest = [(n, p) for n, p in params if not decay_filter(n, p)][::-1]
        self.entries: list[tuple[str, torch.nn.Parameter, int, int]] = []  # name, param, offset, numel
        off = 0
        for group in (decay, rest):
            for n, p in group:
                self.entries.append((n, p, off, p.numel()))
                off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
            if group is decay:
                self.n_decay = off
        self.numel = off
        alloc = allocator or (lambda n, dt, dev: torch.zeros(n, dtype=dt, device=dev))
        self.shadow = alloc(self.numel, compute_dtype, self.device)
        self.grad = alloc(self.numel, torch.float32, self.device)
        self.master = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
        for n, p, o, k in self.entries:
            self.master[o:o + k].copy_(p.detach().reshape(-1).to(device=self.device, dtype=torch.float32))
        self.shadow.copy_(self.master.to(compute_dtype))
        for n, p, o, k in self.entries:
            p.data = self.shadow[o:o + k].view(p.shape)
            p.main_grad = self.grad[o:o + k].view(p.shape)
        self.by_name = {n: (p, o, k) for n, p, o, k in self.entries}

    def zero_grad(self) -> None:
        if self.grad.is_cuda:
            K.fill_f32_(self.grad, 0.0)
        else:
            self.grad.zero_()

    def collect_autograd_grads(self) -> None:
        """Fold ``param.grad`` produced by stock autograd (the CPU backend path) into the flat buffer."""
        for n, p, o, k in self.entries:
            if p.grad is not None:
                self.grad[o:o + k].add_(p.grad.reshape(-1).to(torch.float32))
                p.grad = None

    def named_master(self):
        for n, p, o, k in self.entries:
            yield n, self.master[o:o + k].view(p.shape)

    def sync_shadow_from_master(self) -> None:
        self.shadow.copy_(self.master.to(self.compute_dtype))

    def grad_norm_and_finite(self) -> tuple[torch.Tensor, torch.Tensor]:
        """(l2 norm of the flat gradient, 1.0 if any element is NaN/Inf) computed on the device."""
        if self.grad.is_cuda:
            out = torch.zeros(2, dtype=torch.float32, device=self.device)
            K.sumsq_nonfinite(self.grad, out)
            return out[0].sqrt(), out[1]
        g = self.grad
        return g.norm(), (~torch.isfinite(g)).any().float()


class _FlatOptimizer:
    """Shared hyper-parameter plumbing: values live in an 8-float device tensor that the kernel reads, so a
    captured CUDA graph of the step stays valid while lr and the step counter change between replays."""

    HYPER_RING = 8   # host-side staging slots: at most this many steps may be enqueued ahead of the device

    def __init__(self, store: ParamStore, lr: float):
        self.store = store
        self.lr = float(lr)
        self.step_count = 0
        # The host-to-device copy of the hyper-parameters reads pinned memory when it EXECUTES, not when it is
        # enqueued, so a single staging buffer would let step N pick up step N+1's lr and step count whenever the
        # host runs ahead (graph replay, pipelined steps).  Each step therefore gets its own slot of a small ring;
        # a slot is rewritten only after the event recorded behind its previous copy has completed.
        self._hyper_ring = [torch.zeros(8, dtype=torch.float32) for _ in range(self.HYPER_RING)]
        self._hyper_events: list = [None] * self.HYPER_RING
        if store.device.type == "cuda":
            self._hyper_ring = [h.pin_memory() for h in self._hyper_ring]
        self._hyper_host = self._hyper_ring[0]
        self.hyper = torch.zeros(8, dtype=torch.float32, device=store.device)
        self.grad_scale = 1.0

    def _fill_hyper(self) -> None:
        raise NotImplementedError

    def prepare_step(self) -> None:
        """Advance the step counter and push hyper-parameters to the device (outside any graph capture)."""
        self.step_count += 1
        slot = self.step_count % self.HYPER_RING
        ev = self._hyper_events[slot]
        if ev is not None:
            ev.synchronize()      # the copy that last read this slot has run
        self._hyper_host = self._hyper_ring[slot]
        self._fill_hyper()
        self.hyper.copy_(self._hyper_host, non_blocking=True)
        if self.hyper.is_cuda:
            if ev is None:
                ev = self._hyper_events[slot] = torch.cuda.Event()
            ev.record()

    def launch(self) -> None:
        """Enqueue the update kernel on the current stream (capturable)."""
        raise NotImplementedError

    def step(self) -> None:
        self.prepare_step()
        self.launch()

    def zero_grad(self) -> None:
        self.store.zero_grad()

    def set_lr(self, lr: float) -> None:
        self.lr = float(lr)


class AdamW(_FlatOptimizer):
    def __init__(self, store: ParamStore, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01):
        super().__init__(store, lr)
        self.betas, self.eps, self.weight_decay = betas, eps, weight_decay
        self.m = torch.zeros_like(store.master)
        self.v = torch.zeros_like(store.master)

    def _fill_hyper(self) -> None:
        h = self._hyper_host
        h[0], h[1], h[2], h[3] = self.lr, self.betas[0], self.betas[1], self.eps
        h[4], h[5], h[6] = self.weight_decay, float(self.step_count), self.grad_scale

    def launch(self) -> None:
        s = self.store
        if s.master.is_cuda:
            K.adamw_flat(s.master, self.m, self.v, s.grad, s.shadow, s.n_decay, self.hyper)
            return
        lr, b1, b2, eps, wd, t, gs = [float(x) for x in self.hyper[:7]]
        g = s.grad * gs
        self.m.mul_(b1).add_(g, alpha=1 - b1)
        self.v.mul_(b2).addcmul_(g, g, value=1 - b2)
        mh = self.m / (1 - b1 ** t)
        vh = self.v / (1 - b2 ** t)
        decay = torch.zeros_like(s.master)
        decay[: s.n_decay] = wd
        s.master.sub_(lr * decay * s.master + lr * mh / (vh.sqrt() + eps))
        s.sync_shadow_from_master()

    def state_dict(self) -> dict:
        out = {"step_count": self.step_count}
        for n, p, o, k in self.store.entries:
            out[f"m.{n}"] = self.m[o:o + k].view(p.shape).clone()
            out[f"v.{n}"] = self.v[o:o + k].view(p.shape).clone()
        return out

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd.get("step_count", 0))
        for n, p, o, k in self.store.entries:
            if f"m.{n}" in sd:
                self.m[o:o + k].copy_(sd[f"m.{n}"].reshape(-1))
                self.v[o:o + k].copy_(sd[f"v.{n}"].reshape(-1))


class SGD(_FlatOptimizer):
    def __init__(self, store: ParamStore, lr: float = 1e-2, momentum: float = 0.0, weight_decay: float = 0.0):
        super().__init__(store, lr)
        self.momentum, self.weight_decay = momentum, weight_decay
        self.mom = torch.zeros_like(store.master) if momentum else None

    def _fill_hyper(self) -> None:
        h = self._hyper_host
        h[0], h[1], h[4], h[6] = self.lr, self.momentum, self.weight_decay, self.grad_scale

    def launch(self) -> None:
        s = self.store
        if s.master.is_cuda:
            K.sgd_flat(s.master, self.mom, s.grad, s.shadow, s.n_decay, self.hyper)
            return
        lr, mu, wd, gs = float(self.hyper[0]), float(self.hyper[1]), float(self.hyper[4]), float(self.hyper[6])
        g = s.grad * gs
        if wd:
            g[: s.n_decay] += wd * s.master[: s.n_decay]
        if self.mom is not None:
            self.mom.mul_(mu).add_(g)
            g = self.mom
        s.master.sub_(lr * g)
        s.sync_shadow_from_master()

    def state_dict(self) -> dict:
        out = {"step_count": self.step_count}
        if self.mom is not None:
            for n, p, o, k in self.store.entries:
                out[f"momentum.{n}"] = self.mom[o:o + k].view(p.shape).clone()
        return out


class Adam(AdamW):
    """Adam = AdamW without decoupled weight decay (crates/incin-core/src/optim/mod.rs:93-124)."""

    def __init__(self, store: ParamStore, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8):
        super().__init__(store, lr, betas, eps, weight_decay=0.0)


def make_store(module, device=None, compute_dtype=None, **kw) -> ParamStore:
    """Flat store for a module: bf16 shadow on CUDA, fp32 on the CPU backend."""
    import torch
    params = list(module.named_parameters())
    dev = torch.device(device) if device is not None else params[0][1].device
    if compute_dtype is None:
        compute_dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    return ParamStore(params, device=dev, compute_dtype=compute_dtype, **kw)
