"""Collective transports behind one interface.

``CollectiveBackend`` is the counterpart of the reference's trait of the same name
(crates/incin-backends/src/dist/collective.rs:41-94: all_reduce / all_gather / reduce_scatter /
all_to_all / send_recv over dtype-indexed buffers).  Two implementations:

* :class:`ReferenceTransport` — deterministic, in-process, takes every rank's buffer in one call
  (C++: csrc/comm/reference_transport.cpp).  The oracle for every distributed test on CPU.
* :class:`NcclTransport` — one process per GPU over ``torch.distributed`` (NCCL on NVLink/NVSwitch;
  gloo for CPU ranks).  This is the *baseline and bootstrap* transport; the product path for the hot
  collectives is the fused peer-memory kernels (parallel/dp.py, parallel/tp.py).  Launches are validated
  against the agreed plan (sequence, dtype, element count) and any error invalidates the context,
  as in crates/incin-backends/src/dist/nccl.rs:985-1014,1241-1280.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from .. import _native as nat
from ..core.dtype import DTypeId, from_torch
from .placement import Reduction
from .plan import CollectiveKind, PlanCursor, PlanError

_REF_DTYPE = {torch.float32: 0, torch.float64: 1, torch.float16: 2, torch.bfloat16: 3, torch.int64: 4,
              torch.uint32: 5, torch.uint8: 6}
_REF_OP = {Reduction.SUM: 0, Reduction.MEAN: 1, Reduction.MAX: 2, Reduction.MIN: 3, Reduction.PROD: 4}


class TransportError(RuntimeError):
    pass


class CollectiveBackend:
    world: int

    def all_reduce(self, bufs, op: Reduction = Reduction.SUM): raise NotImplementedError
    def all_gather(self, bufs): raise NotImplementedError
    def reduce_scatter(self, bufs, op: Reduction = Reduction.SUM): raise NotImplementedError
    def all_to_all(self, bufs): raise NotImplementedError
    def send_recv(self, bufs, src: int, dst: int): raise NotImplementedError


def _ptr_array(ts: Sequence[torch.Tensor]):
    arr = (C.c_void_p * len(ts))()
    for i, t in enumerate(ts):
        arr[i] = t.data_ptr()
    return arr


class ReferenceTransport(CollectiveBackend):
    """All ranks in one process: ``bufs[r]`` is rank r's contiguous CPU tensor; returns one output per rank."""

    def __init__(self, world: int):
        if world < 1:
            raise ValueError("world must be >= 1")
        self.world = world
        self._h = nat.host()
        for name in ("incin_ref_all_reduce", "incin_ref_all_gather", "incin_ref_reduce_scatter",
                     "incin_ref_all_to_all", "incin_ref_send_recv"):
            getattr(self._h, name).restype = C.c_int

    def _check(self, bufs):
        if len(bufs) != self.world:
            raise TransportError(f"expected {self.world} rank buffers, got {len(bufs)}")
        d, n = bufs[0].dtype, bufs[0].numel()
        if d not in _REF_DTYPE:
            raise TransportError(f"{d} cannot travel through a collective")
        for b in bufs:
            if b.dtype != d or b.numel() != n or b.is_cuda:
                raise TransportError("rank buffers must agree in dtype and size and live on the CPU")
        return [b.contiguous() for b in bufs], _REF_DTYPE[d], n

    def _rc(self, rc: int, what: str):
        if rc == 2:
            raise TransportError(f"{what}: integer overflow in reduction")
        if rc:
            raise TransportError(f"{what}: invalid argument (code {rc})")

    def all_reduce(self, bufs, op=Reduction.SUM):
        ins, dt, n = self._check(bufs)
        outs = [torch.empty_like(b) for b in ins]
        self._rc(self._h.incin_ref_all_reduce(_ptr_array(ins), _ptr_array(outs), self.world, C.c_int64(n), dt,
                                              _REF_OP[op]), "all_reduce")
        return outs

    def all_gather(self, bufs):
        ins, dt, n = self._check(bufs)
        outs = [torch.empty(n * self.world, dtype=b.dtype) for b in ins]
        self._rc(self._h.incin_ref_all_gather(_ptr_array(ins), _ptr_array(outs), self.world, C.c_int64(n), dt),
                 "all_gather")
        return outs

    def reduce_scatter(self, bufs, op=Reduction.SUM):
        ins, dt, n = self._check(bufs)
        if n % self.world:
            raise TransportError(f"{n} elements do not scatter over {self.world} ranks")
        outs = [torch.empty(n // self.world, dtype=b.dtype) for b in ins]
        self._rc(self._h.incin_ref_reduce_scatter(_ptr_array(ins), _ptr_array(outs), self.world, C.c_int64(n), dt,
                                                  _REF_OP[op]), "reduce_scatter")
        return outs

    def all_to_all(self, bufs):
        ins, dt, n = self._check(bufs)
        if n % self.world:
            raise TransportError(f"{n} elements do not split over {self.world} ranks")
        outs = [torch.empty_like(b) for b in ins]
        self._rc(self._h.incin_ref_all_to_all(_ptr_array(ins), _ptr_array(outs), self.world, C.c_int64(n), dt),
                 "all_to_all")
        return outs

    def send_recv(self, bufs, src, dst):
        ins, dt, n = self._check(bufs)
        outs = [b.clone() for b in ins]
        self._rc(self._h.incin_ref_send_recv(_ptr_array(ins), _ptr_array(outs), self.world, C.c_int64(n), dt, src,
                                             dst), "send_recv")
        return outs


class NcclTransport:
    """Per-rank transport over an initialised ``torch.distributed`` group (NCCL for CUDA, gloo for CPU)."""

    def __init__(self, group=None, *, context=None, agreed_plan=None):
        import torch.distributed as dist
        if not dist.is_initialized():
            raise TransportError("torch.distributed is not initialised")
        self.dist, self.group = dist, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.context = context
        self.cursor = PlanCursor(agreed_plan) if agreed_plan is not None else None

    @classmethod
    def connect_context(cls, context, plan, *, backend: str | None = None, device: torch.device | None = None,
                        timeout_s: float = 60.0) -> "NcclTransport":
        """Bring up the communicator from a rendezvous context, in the reference's order
        (crates/incin-backends/src/dist/nccl.rs:454-512 ``connect_context``, :1539-1587 ``exchange_bootstrap``):

        1. topology: every rank publishes where it runs (host, device kind, device identity) over the context's control
           channel; two ranks on one physical device, or ranks of different device kinds, are refused;
        2. preflight: the hash of ``plan`` must agree on every rank (``context.preflight``) BEFORE any communicator exists;
        3. bootstrap: rank 0 picks the address the library communicator will use and publishes it over the control
           channel (the role of the NCCL unique id); only then is the ``torch.distributed`` process group created.
        A failure in 1 or 2 invalidates the context and leaves ``torch.distributed`` untouched."""
        import datetime
        import json
        import os
        import socket
        import torch.distributed as dist
        from .context import ContextFailure
        context.ensure_active()
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        if device.type == "cuda":
            props = torch.cuda.get_device_properties(device)
            ident = str(getattr(props, "uuid", "")) or f"cuda:{device.index}"
        else:
            ident = f"cpu:{os.getpid()}"
        me = {"rank": context.rank, "host": socket.gethostname(), "kind": device.type, "device": ident}
        # (the control channel gathers equal-size blobs: identities and the address travel zero-padded)
        peers = [json.loads(b.rstrip(b"\0").decode()) for b in context.allgather_bytes(json.dumps(me).encode().ljust(512, b"\0"))]
        kinds = {p["kind"] for p in peers}
        seen: dict[tuple, int] = {}
        problem = None
        if len(kinds) != 1:
            problem = f"ranks run on different device kinds: {sorted(kinds)}"
        for p in peers:
            key = (p["host"], p["device"])
            if key in seen and p["kind"] == "cuda":
                problem = f"ranks {seen[key]} and {p['rank']} share device {p['device']} on {p['host']}"
            seen[key] = p["rank"]
        if problem:
            context.invalidate(ContextFailure.PLAN_MISMATCH)
            raise TransportError("topology rejected: " + problem)
        agreed = context.preflight(plan)              # raises PreflightError and invalidates the context on divergence
        if context.rank == 0:
            s = socket.socket()
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
            s.close()
            boot = f"tcp://127.0.0.1:{port}".encode()
        else:
            boot = b""
        boot = context.allgather_bytes(boot.ljust(64, b"\0"))[0].rstrip(b"\0").decode()
        if dist.is_initialized():
            raise TransportError("torch.distributed is already initialised: connect_context owns the communicator bootstrap")
        backend = backend or ("nccl" if device.type == "cuda" else "gloo")
        kw = {"device_id": device} if device.type == "cuda" else {}
        dist.init_process_group(backend, init_method=boot, rank=context.rank, world_size=context.world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
        tr = cls(None, context=context, agreed_plan=agreed)
        tr.topology = peers
        return tr

    def _guard(self, tag, kind: CollectiveKind, t: torch.Tensor):
        if self.context is not None:
            self.context.ensure_active()
        if not t.is_contiguous():
            raise TransportError("collective buffers must be contiguous")
        if self.cursor is not None:
            try:
                self.cursor.next(tag=tag, kind=kind, elements=t.numel(), dtype=from_torch(t.dtype))
            except PlanError:
                self._invalidate()
                raise

    def _invalidate(self):
        if self.context is not None:
            from .context import ContextFailure
            self.context.invalidate(ContextFailure.PLAN_MISMATCH)

    def _run(self, fn):
        try:
            return fn()
        except Exception:
            if self.context is not None:
                from .context import ContextFailure
                self.context.invalidate(ContextFailure.IO)
            raise

    def all_reduce(self, t, op=Reduction.SUM, tag=0):
        self._guard(tag, CollectiveKind.all_reduce(op), t)
        ops = {Reduction.SUM: self.dist.ReduceOp.SUM, Reduction.MAX: self.dist.ReduceOp.MAX,
               Reduction.MIN: self.dist.ReduceOp.MIN, Reduction.PROD: self.dist.ReduceOp.PRODUCT,
               Reduction.MEAN: self.dist.ReduceOp.SUM}
        self._run(lambda: self.dist.all_reduce(t, op=ops[op], group=self.group))
        if op is Reduction.MEAN:
            t.div_(self.world)
        return t

    def all_gather(self, t, tag=0):
        self._guard(tag, CollectiveKind.all_gather(), t)
        out = torch.empty(self.world * t.numel(), dtype=t.dtype, device=t.device)
        self._run(lambda: self.dist.all_gather_into_tensor(out, t.reshape(-1), group=self.group))
        return out

    def reduce_scatter(self, t, op=Reduction.SUM, tag=0):
        self._guard(tag, CollectiveKind.reduce_scatter(op), t)
        if t.numel() % self.world:
            raise TransportError(f"{t.numel()} elements do not scatter over {self.world} ranks")
        out = torch.empty(t.numel() // self.world, dtype=t.dtype, device=t.device)
        if t.is_cuda:
            self._run(lambda: self.dist.reduce_scatter_tensor(out, t.reshape(-1), group=self.group))
        else:  # gloo has no reduce_scatter: all-reduce then slice
            full = t.reshape(-1).clone()
            self._run(lambda: self.dist.all_reduce(full, group=self.group))
            out.copy_(full[self.rank * out.numel():(self.rank + 1) * out.numel()])
        if op is Reduction.MEAN:
            out.div_(self.world)
        return out

    def all_to_all(self, t, tag=0):
        self._guard(tag, CollectiveKind.all_to_all(), t)
        out = torch.empty_like(t)
        if t.is_cuda:
            self._run(lambda: self.dist.all_to_all_single(out.reshape(-1), t.reshape(-1), group=self.group))
        else:
            chunks = list(t.reshape(self.world, -1).unbind(0))
            outs = [torch.empty_like(c) for c in chunks]
            reqs = []
            for r in range(self.world):
                if r == self.rank:
                    outs[r].copy_(chunks[r])
                else:
                    reqs.append(self.dist.isend(chunks[r].contiguous(), r, group=self.group))
                    reqs.append(self.dist.irecv(outs[r], r, group=self.group))
            for q in reqs:
                q.wait()
            out.copy_(torch.stack(outs).reshape(t.shape))
        return out

    def send_recv(self, t, src, dst, tag=0):
        self._guard(tag, CollectiveKind.send_recv(src, dst), t)
        if self.rank == src:
            self._run(lambda: self.dist.send(t, dst, group=self.group))
        elif self.rank == dst:
            self._run(lambda: self.dist.recv(t, src, group=self.group))
        return t
