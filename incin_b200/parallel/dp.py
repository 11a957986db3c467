"""Data-parallel gradient reduction.

Product path (:class:`FusedReducer`): the flat fp32 gradient buffer and the flat bf16 parameter buffer
of every rank live in peer-mapped memory; per gradient bucket ONE kernel (``incin_dp_reduce_adamw``)
does reduce-scatter over P2P loads, AdamW on the owned shard, and all-gather of the new bf16 weights
over P2P stores.  With ``overlap=True`` buckets are launched on a side stream as soon as the backward
pass has finished every gradient they contain, with a small grid so the GEMMs keep the SMs.

Baseline path (:class:`NcclReducer`, not the product): ``all_reduce`` of the flat buffer through NCCL,
then the local flat AdamW kernel.

The reference's DP (crates/incin-core/src/dist/data_parallel.rs:136-245,
crates/incin-backends/src/dist/nccl.rs:606-632) reduces one parameter tensor per ncclAllReduce(Avg)
after backward, chained by ``depends_on``, two ranks only.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .. import _native as nat
from ..core.dtype import DTypeId
from ..ops.gemm import status_word
from .placement import Reduction
from .plan import CollectiveKind
from .symm import SymmetricBuffer

MAX_PEERS = 8
MAX_SLOTS = 64


class DpDesc(C.Structure):
    _fields_ = [("grads", C.c_void_p * MAX_PEERS), ("shadows", C.c_void_p * MAX_PEERS),
                ("pads", C.c_void_p * MAX_PEERS), ("master", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p),
                ("hyper", C.c_void_p), ("lo", C.c_longlong), ("hi", C.c_longlong), ("n_decay", C.c_longlong),
                ("world", C.c_int), ("rank", C.c_int), ("slot", C.c_int), ("ctas", C.c_int), ("status", C.c_void_p)]


nat.register_cuda_signatures({
    "incin_dp_reduce_adamw": (C.c_int, [C.POINTER(DpDesc), C.c_void_p]),
    "incin_dp_reduce_adamw_mc": (C.c_int, [C.POINTER(DpDesc), C.c_void_p, C.c_void_p, C.c_void_p]),
    "incin_dp_pad_bytes": (C.c_int, []),
})


class NcclReducer:
    """Baseline: NCCL all-reduce of the flat gradient buffer, then the local optimiser kernel."""

    kind = "nccl-allreduce+local-adamw (baseline)"

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group)

    def allocator(self, n, dtype, device):
        return torch.zeros(n, dtype=dtype, device=device)

    def attach(self, store, opt) -> None:
        self.store = store
        opt.grad_scale = 1.0 / self.world
        opt.reducer = self

    def begin_step(self) -> None:
        pass

    def finish_step(self, opt) -> None:
        dist.all_reduce(self.store.grad, group=self.group)
        opt.launch()


class FusedReducer:
    kind = "fused p2p reduce-scatter + adamw + all-gather (one kernel per bucket)"

    def __init__(self, device: torch.device, group=None, *, overlap: bool = True, bucket_elems: int = 16 << 20,
                 ctas_overlap: int = 24, ctas_tail: int = 64, session=None, ranks: list[int] | None = None, axis=None,
                 plan_ranks: list[int] | None = None, multimem: bool | None = None):
        """``session`` (a :class:`~incin_b200.parallel.session.CollectiveSession`) puts the reducer under the plan
        contract: ``attach`` builds the step's plan (one all-reduce(mean) per bucket, chained), agrees on its hash
        among ``ranks`` BEFORE any peer mapping is opened, moves the IPC handles over the session's control channel
        and checks every bucket launch against the plan cursor.  ``axis``: the mesh axis reduced over (default DATA);
        ``plan_ranks``: the ranks of that axis' group when the reduction spans more than one mesh axis (the plan is
        then agreed within the axis group, whose ranks the plan names, while buffers are shared among ``ranks``)."""
        self.device, self.group = device, group
        self.session, self.lane, self.axis = session, None, axis
        if session is not None and ranks is None and group is not None:
            ranks = dist.get_process_group_ranks(group)
        # NVSwitch multicast for the gradient and parameter buffers: in-switch reduction of the owned slice, one
        # replicated store of the new weights.  Default: on when the platform offers it and NVLS is not switched off.
        from .symm import MulticastBuffer
        self.multimem = MulticastBuffer.available() if multimem is None else bool(multimem)
        self.ranks = ranks
        self.plan_ranks = plan_ranks if plan_ranks is not None else ranks
        if session is not None and session.ctx is not None:
            job_ranks = ranks if ranks is not None else list(range(session.ctx.world))
            self.world, self.rank = len(job_ranks), job_ranks.index(session.ctx.rank)
        else:
            self.world = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
        if self.world > MAX_PEERS:
            raise ValueError(f"fused reducer supports up to {MAX_PEERS} ranks per node")
        self.overlap = overlap
        self.bucket_elems = bucket_elems
        self.ctas_overlap, self.ctas_tail = ctas_overlap, ctas_tail
        self._bufs: list[SymmetricBuffer] = []
        self.comm_stream = None

    def describe(self) -> str:
        """What this reducer does, for benchmark records (valid once the buffers have been allocated)."""
        mc_g = getattr(getattr(self, "grad_buf", None), "mc_ptr", 0)
        mc_s = getattr(getattr(self, "shadow_buf", None), "mc_ptr", 0)
        staged = getattr(self, "grad_stage", None) is not None
        how = (("in-switch multimem.ld_reduce of the owned gradient slice" + (" from a multicast-bound copy of the gradients" if staged else "")
                if (mc_g or staged) else "P2P loads of the owned gradient slice") + " + " +
               ("one multimem.st of the new weights through NVSwitch" if mc_s else "P2P stores of the new weights"))
        when = "overlapped with backward" if self.overlap else "after backward"
        return f"fused reduce-scatter + AdamW + all-gather, one kernel per bucket ({how}), {when}"

    # ParamStore calls this for the bf16 shadow and the fp32 gradient buffer
    def allocator(self, n: int, dtype: torch.dtype, device) -> torch.Tensor:
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        import os
        # Which buffers are bound to the multicast object.  Measured on 2 B200s inside the GPT-2-small step (one call):
        # nothing bound 11.04 ms, parameters only 10.99 ms, gradients only 11.72 ms, both 11.81 ms: the backward
        # kernels' fp32 accumulation into multicast-bound memory (split-K reduce-adds, norm and bias gradients) runs
        # markedly slower than into ordinary device memory, which costs far more than the in-switch reduction of
        # 1/world of the gradients saves.  So only the parameter buffer is bound by default (one multimem.st instead
        # of world - 1 peer stores per 16 bytes); INCIN_MULTIMEM_BUFFERS=grad,shadow binds both.  "stage" keeps the
        # gradients in ordinary memory and copies each bucket into a multicast-bound buffer right before its reduction
        # (one extra local pass over the gradients buys the in-switch reduction: world - 1 times fewer inbound bytes).
        which = os.environ.get("INCIN_MULTIMEM_BUFFERS", "shadow")
        if self.multimem and (("grad" in which) if dtype == torch.float32 else ("shadow" in which)):
            from .symm import MulticastBuffer
            try:
                buf = MulticastBuffer(nbytes, torch.device(device))
            except Exception:      # no symmetric-memory allocator on this platform: plain peer-mapped buffers
                self.multimem = False
                buf = SymmetricBuffer(nbytes, torch.device(device))
        else:
            buf = SymmetricBuffer(nbytes, torch.device(device))
        self._bufs.append(buf)
        return buf.typed(dtype, n)

    def attach(self, store, opt) -> None:
        from ..optim.flat import AdamW
        if not isinstance(opt, AdamW):
            raise TypeError("the fused reducer implements AdamW")
        self.store, self.opt = store, opt
        opt.reducer = self
        shadow_buf = next(b for b in self._bufs if b.ptr == store.shadow.data_ptr())
        grad_buf = next(b for b in self._bufs if b.ptr == store.grad.data_ptr())
        # buckets: contiguous ranges of the flat buffer, cut at parameter boundaries
        self.buckets = bucket_ranges(store.entries, store.numel, self.bucket_elems if self.overlap else 0)
        if len(self.buckets) > MAX_SLOTS:
            raise ValueError("too many gradient buckets")
        if self.session is not None:
            # the plan first: a rank whose buckets differ (other model, other bucket size) is rejected here, before
            # any of its memory is mapped into a peer
            self.lane = self.session.agree(reducer_plan(self.session.mesh, self.session.rank, self.buckets, self.axis),
                                           self.plan_ranks, self.group if self.plan_ranks is self.ranks else None)
        self.pad = SymmetricBuffer(nat.cuda().incin_dp_pad_bytes(), self.device)
        for b in (shadow_buf, grad_buf, self.pad):
            b.exchange(self.group, session=self.session, ranks=self.ranks)
        self.shadow_buf, self.grad_buf = shadow_buf, grad_buf
        self.grad_stage = None
        import os
        if self.multimem and "stage" in os.environ.get("INCIN_MULTIMEM_BUFFERS", "shadow") and not getattr(grad_buf, "mc_ptr", 0):
            from .symm import MulticastBuffer
            self.grad_stage = MulticastBuffer(store.grad.numel() * 4, self.device).exchange(self.group, session=self.session)
            self._stage_view = self.grad_stage.typed(torch.float32, store.grad.numel())
        self._descs = [self._make_desc(i, lo, hi) for i, (lo, hi) in enumerate(self.buckets)]
        # readiness bookkeeping: a bucket is ready when every parameter overlapping it is complete
        self._entry_buckets: dict[int, list[int]] = {}
        self._bucket_need = [0] * len(self.buckets)
        for name, p, off, numel in store.entries:
            hit = [i for i, (lo, hi) in enumerate(self.buckets) if off < hi and off + numel > lo]
            self._entry_buckets[id(p)] = hit
            for i in hit:
                self._bucket_need[i] += 1
            if self.overlap:
                p._grad_ready = self._on_ready
        if self.overlap:
            self.comm_stream = torch.cuda.Stream(device=self.device)
        if self.session is not None and self.session.ctx is not None:
            self.session.barrier(self.ranks)
        else:
            dist.barrier(group=self.group)

    def _make_desc(self, slot: int, lo: int, hi: int) -> DpDesc:
        d = DpDesc()
        for r in range(self.world):
            d.grads[r] = self.grad_buf.ptrs[r]
            d.shadows[r] = self.shadow_buf.ptrs[r]
            d.pads[r] = self.pad.ptrs[r]
        d.master, d.m, d.v = self.store.master.data_ptr(), self.opt.m.data_ptr(), self.opt.v.data_ptr()
        d.hyper = self.opt.hyper.data_ptr()
        d.lo, d.hi, d.n_decay = lo, hi, self.store.n_decay
        d.world, d.rank, d.slot = self.world, self.rank, slot
        d.ctas = self.ctas_overlap if self.overlap else self.ctas_tail
        d.status = status_word(self.device).data_ptr()
        return d

    def begin_step(self) -> None:
        if self.lane is not None:
            self.lane.begin_step()
        self._uses_left = {id(p): getattr(p, "_grad_uses", 1) for _, p, _, _ in self.store.entries}
        self._need_left = list(self._bucket_need)
        self._launched = [False] * len(self.buckets)
        self._next = 0

    def _launch(self, i: int, stream: torch.cuda.Stream) -> None:
        if self.lane is not None:    # fail-stop state, then: is bucket i the next collective of the agreed plan?
            lo, hi = self.buckets[i]
            self.lane.launch(tag=i, kind=CollectiveKind.all_reduce(Reduction.MEAN), elements=hi - lo, dtype=DTypeId.F32)
        if self.multimem:
            mc_g = getattr(self.grad_buf, "mc_ptr", None)
            if self.grad_stage is not None:
                lo, hi = self.buckets[i]
                with torch.cuda.stream(stream):
                    self._stage_view[lo:hi].copy_(self.store.grad[lo:hi])
                mc_g = self.grad_stage.mc_ptr
            nat.check(nat.cuda().incin_dp_reduce_adamw_mc(C.byref(self._descs[i]), mc_g,
                                                          getattr(self.shadow_buf, "mc_ptr", None), stream.cuda_stream),
                      "dp_reduce_adamw_mc")
        else:
            nat.check(nat.cuda().incin_dp_reduce_adamw(C.byref(self._descs[i]), stream.cuda_stream), "dp_reduce_adamw")
        self._launched[i] = True

    def _on_ready(self, p) -> None:
        key = id(p)
        self._uses_left[key] -= 1
        if self._uses_left[key] != 0:
            return
        for i in self._entry_buckets[key]:
            self._need_left[i] -= 1
        # buckets start in plan order (the order every rank agreed on): the first not yet started one, once complete
        while self._next < len(self.buckets) and self._need_left[self._next] == 0:
            cur = torch.cuda.current_stream()
            self.comm_stream.wait_stream(cur)
            self._launch(self._next, self.comm_stream)
            self._next += 1

    def finish_step(self, opt) -> None:
        cur = torch.cuda.current_stream()
        if self.overlap:
            rest = [i for i, done in enumerate(self._launched) if not done]
            if rest:
                self.comm_stream.wait_stream(cur)
                for i in rest:
                    self._launch(i, self.comm_stream)
            cur.wait_stream(self.comm_stream)
        else:
            self._launch(0, cur)


def bucket_ranges(entries, numel: int, bucket_elems: int) -> list[tuple[int, int]]:
    """Contiguous ranges of the flat buffer cut at parameter boundaries, at least ``bucket_elems`` long each (0 = one
    bucket for everything)."""
    if bucket_elems <= 0:
        return [(0, numel)]
    bounds = [0]
    for name, p, off, n in entries:
        if off - bounds[-1] >= bucket_elems:
            bounds.append(off)
    bounds.append(numel)
    return [(bounds[i], bounds[i + 1]) for i in range(len(bounds) - 1) if bounds[i + 1] > bounds[i]]


def reducer_plan(mesh, rank: int, buckets, axis=None):
    """The gradient reduction of one step as a plan: one all-reduce(mean) of fp32 elements per bucket, in launch order,
    each depending on the one before (crates/incin-core/src/dist/data_parallel.rs:136-245 plans one per parameter)."""
    from .mesh import Axis
    from .strategies import DataParallelPlanBuilder
    b = DataParallelPlanBuilder(mesh, rank, axis or Axis.DATA)
    for i, (lo, hi) in enumerate(buckets):
        b.push(i, hi - lo, DTypeId.F32)
    return b.finish()


def make_reducer(kind: str, device: torch.device, group=None, session=None):
    """Returns ``(reducer, allocator, description)`` for ``bench.py`` / the Trainer."""
    if kind in ("fused", "fused-overlap"):
        import os
        r = FusedReducer(device, group, overlap=True, ctas_overlap=int(os.environ.get("INCIN_DP_OVERLAP_CTAS", "8")),
                         bucket_elems=int(os.environ.get("INCIN_DP_BUCKET_ELEMS", str(16 << 20))), session=session)
        return r, r.allocator, r.kind + " overlapped with backward"
    if kind in ("auto", "fused-tail"):
        r = FusedReducer(device, group, overlap=False, session=session)
        return r, r.allocator, r.kind + " after backward"
    r = NcclReducer(group)
    return r, r.allocator, r.kind
