"""Tensor parallelism with sequence-sharded activations, lowered onto two fused kernels.

Between layers an activation ``[M, C]`` (M = all tokens of the step) is ``Sharded(0)`` over the tensor-parallel
group: every rank holds ``M / tp`` rows.

* column-parallel linear (QKV, gate/up; weight ``Sharded(0)`` over outputs):  ``Sharded(0) -> Replicated`` input
  transition fused into the GEMM — copy CTAs of the same launch pull the peers' row shards into local memory by
  bulk copies while the remaining CTAs run tcgen05 tiles on the rows that have arrived
  (``incin_gemm_bf16`` with ``gather``);
* row-parallel linear (attention output, FFN down; weight ``Sharded(1)`` over inputs): the product is
  ``Partial(Sum)`` and goes ``-> Sharded(0)``: the GEMM epilogue stores each 128-row tile as bf16 into this rank's
  slot of the OWNER's buffer over NVLink peer stores (``scatter``), then the owner sums the slots (+ residual).

The backward of each is the other one (all-gather <-> reduce-scatter are adjoint), so the same two kernels serve
both passes.  Buffers that peers read or write live in peer-mapped memory and alternate between two parities;
one barrier kernel (``incin_peer_barrier``) per fused op orders "my shard is written" / "your slots are complete"
against the peers' streams.  No NCCL call is on this path.

Reference: crates/incin-core/src/dist/tensor_parallel.rs (ColumnOutputGather / RowOutputSum) executed as
ncclAllGather / ncclAllReduce plus separate SGEMMs and reshapes (crates/incin-backends/src/dist/nccl.rs:642-791,
1187-1229), two ranks only.
"""
from __future__ import annotations

import os

import ctypes as C

import torch
import torch.distributed as dist

from .. import _native as nat
from ..core.dtype import DTypeId
from ..ops import gemm as G
from ..ops import kernels as K
from ..ops.functional import _ready, main_grad
from ..ops.gemm import status_word
from .placement import (Partial, Placement, PlacementError, PlacementTransition, Reduction, Replicated, Sharded,
                        validate_transition)
from .plan import CollectiveKind
from .strategies import TensorParallelCollective, tp_tag
from .symm import SymmetricBuffer

nat.register_cuda_signatures({
    "incin_peer_barrier": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "incin_barrier_pad_bytes": (C.c_int, []),
    "incin_peer_sum_ranges": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
})


class TensorParallel:
    """Per-process context of one tensor-parallel group (all ranks of ``group`` on one NVSwitch node)."""

    def __init__(self, device: torch.device, group=None, *, max_rows_per_rank: int, max_cols: int, copy_ctas: int = 0,
                 mode: str = "fused", session=None, plan=None, ranks: list[int] | None = None):
        """``mode="nccl"`` is the baseline arm (not the product): the same layers with NCCL all-gather /
        reduce-scatter as separate launches around the local GEMM.

        ``session`` (a :class:`~incin_b200.parallel.session.CollectiveSession`) with ``plan`` (the step's collectives in
        launch order, e.g. ``models.llama_tp.tensor_parallel_plan``) puts the group under the plan contract: the plan
        hash is agreed among ``ranks`` (the job ranks of this group) FIRST — a divergent rank is rejected before any
        peer-mapped buffer exists — the IPC handles then travel over the session's control channel, and every fused
        launch that is given a tag is checked against the plan cursor."""
        assert mode in ("fused", "nccl")
        self.mode = mode
        self.device, self.group = device, group
        self.session, self.lane = session, None
        if session is not None and ranks is None and group is not None:
            ranks = dist.get_process_group_ranks(group)
        self.ranks = ranks
        if session is not None and plan is not None:
            self.lane = session.agree(plan, ranks, group)       # raises PreflightError before anything is opened
        if session is not None and session.ctx is not None:
            job_ranks = ranks if ranks is not None else list(range(session.ctx.world))
            self.world, self.rank = len(job_ranks), job_ranks.index(session.ctx.rank)
        else:
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("a tensor-parallel group spans at most the 8 GPUs of one node")
        if max_rows_per_rank % 128:
            raise ValueError("rows per rank must be a multiple of 128 (one GEMM tile never straddles two owners)")
        self.rows, self.cols = max_rows_per_rank, max_cols
        self.copy_ctas = copy_ctas          # 0 = choose per call from the copy volume and the GEMM size
        self._tuned: dict[tuple, int] = {}  # (op, rows per rank, K, N) -> copy CTAs committed by tune_copy_ctas
        # INCIN_TP_AUTOTUNE=1: a shape seen for the first time outside a graph capture is tuned on the spot (every rank
        # of the group reaches the same op in the same order, so the measurement is collective by construction)
        self.autotune = os.environ.get("INCIN_TP_AUTOTUNE") == "1"
        self._tuning = False
        shard_bytes = max_rows_per_rank * max_cols * 2
        ex = dict(session=session, ranks=ranks)
        self.shard = [SymmetricBuffer(shard_bytes, device).exchange(group, **ex) for _ in range(2)]
        self.slots = [SymmetricBuffer(self.world * shard_bytes, device).exchange(group, **ex) for _ in range(2)]
        self.pad = SymmetricBuffer(nat.cuda().incin_barrier_pad_bytes(), device).exchange(group, **ex)
        self._pad_ptrs = torch.tensor(self.pad.ptrs, dtype=torch.int64, device=device)
        self._shard_parity = self._slot_parity = 0
        self._barrier_slot = 0
        if session is not None and session.ctx is not None:
            session.barrier(ranks)
        else:
            dist.barrier(group=group)

    def begin_step(self) -> None:
        """Rewind the plan cursor: the plan describes one training step."""
        if self.lane is not None:
            self.lane.begin_step()

    def _planned(self, tag, kind, elements: int) -> None:
        if self.lane is not None and tag is not None:
            self.lane.launch(tag=tag, kind=kind, elements=elements, dtype=DTypeId.BF16)

    # ------------------------------------------------------------------------------------------------ primitives
    # What one copy CTA of a fused launch sustains over NVLink while the rest of the GPU computes.  A copy-only kernel
    # reaches 26-37 GB/s per CTA; inside the fused launches the best CTA counts of a tp = 4 sweep (12 / 20 / 32 / 44
    # copy CTAs: all-gather 0.352 / 0.256 / 0.218 / 0.227 ms at shard width 384, 0.366 / 0.264 / 0.237 / 0.245 ms at
    # 1408) correspond to about 18 GB/s for the pulling all-gather; the pushing reduce-scatter, whose GEMM is the
    # heavier one at the same shard width, does best with fewer (0.228 / 0.230 / 0.235 ms with 20 / 32 / 44 at 1408).
    COPY_CTA_GBS = 18.0
    COPY_CTA_GBS_PUSH = 24.0
    LINK_GBS = 650.0
    GEMM_TFLOPS = 1200.0

    def tune_copy_ctas(self, op: str, x: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False,
                       candidates=(12, 20, 32, 44), samples: int = 3):
        """Measure the copy-CTA count of one fused op for one shape under the collective tuning contract
        (:mod:`incin_b200.tuning.collective`): every rank of the group times the same candidates in the same order,
        the sample reports are exchanged, a candidate's score is the median over samples of the MAX over ranks, every
        rank votes, and the winner is committed only if the votes agree.  Later calls of ``gather_gemm`` /
        ``gemm_scatter`` with this shape use the committed count.  ``op``: ``"gather"`` (x = this rank's shard) or
        ``"scatter"`` (x = the full rows).  Collective: every rank of the group must call it with the same arguments."""
        import json
        from ..tuning import collective as CT
        assert self.mode == "fused" and op in ("gather", "scatter")
        run = (lambda: self.gather_gemm(x, w, b_mn=b_mn)) if op == "gather" else (lambda: self.gemm_scatter(x, w, b_mn=b_mn))
        N = w.shape[1] if b_mn else w.shape[0]
        key = (op, x.shape[0] if op == "gather" else x.shape[0] // self.world, x.shape[1], N)
        saved, reports = self.copy_ctas, []
        self._tuning = True
        try:
            for c in candidates:
                self.copy_ctas = int(c)
                run()                                                # warm-up (and buffer parities advance in lockstep)
                times = []
                for _ in range(samples):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    run()
                    e1.record()
                    e1.synchronize()
                    times.append(int(e0.elapsed_time(e1) * 1e6))
                cand = CT.CollectiveCandidate(CT.CollectiveAlgorithm.ONE_SHOT_P2P, channels=int(c))
                reports.append(CT.SampleReport(self.rank, cand.token(), tuple(times)))
        finally:
            self.copy_ctas = saved
            self._tuning = False
        mine = json.dumps([(r.rank, r.candidate, r.samples_ns) for r in reports])
        everyone = self._exchange(mine)
        all_reports = [CT.SampleReport(rk, cd, tuple(sm)) for blob in everyone for rk, cd, sm in json.loads(blob)]
        vote = CT.local_vote(self.rank, all_reports)
        votes = [CT.CommitVote(*json.loads(v)) for v in self._exchange(json.dumps([vote.rank, vote.candidate]))]
        committed = CT.commit(self.world, all_reports, votes)       # raises TuningDisagreement unless unanimous
        by_token = {CT.CollectiveCandidate(CT.CollectiveAlgorithm.ONE_SHOT_P2P, channels=int(c)).token(): int(c) for c in candidates}
        self._tuned[key] = by_token[committed.candidate]
        return committed

    def _maybe_tune(self, op: str, x, w, b_mn: bool, key) -> None:
        if self.autotune and not self._tuning and not self.copy_ctas and key not in self._tuned and \
                not torch.cuda.is_current_stream_capturing():
            self.tune_copy_ctas(op, x.detach(), w.detach(), b_mn=b_mn)

    def _exchange(self, text: str) -> list[str]:
        """One string per rank of the group, over the session's control channel when there is one."""
        if self.session is not None and self.session.ctx is not None:
            if len(text.encode()) > 4096:     # the control channel gathers equal-size blobs
                raise ValueError("tuning report too large for one control message: fewer candidates or samples")
            blobs = self.session.allgather(text.encode().ljust(4096, b"\0"), self.ranks)
            return [b.rstrip(b"\0").decode() for b in blobs]
        out = [None] * self.world
        dist.all_gather_object(out, text, group=self.group)
        return out

    def _copy_ctas(self, copy_bytes: float, link_bytes: float, flops: float, push: bool = False, key=None) -> int:
        """Who moves the data of a fused launch.  By default the number of CTAs of the launch that copy instead of
        computing: the count that minimises ``max(copy time, link time, GEMM time on the remaining SMs)``.  Negative
        (``INCIN_TP_COPY=warps``): one extra warp in every compute CTA moves the data and no SM is taken from the
        tensor-core work; the value is minus the number of operand stages of shared memory that become the copy ring.
        Measured between two B200s the copy warps lose: a bulk store to a peer that waits for link credits holds up
        the operand loads of its own SM behind it (GEMM -> reduce-scatter 0.53 ms against 0.17 ms with copy CTAs),
        so dedicated CTAs, which keep that back-pressure on SMs that do nothing else, stay the default."""
        if self.copy_ctas:
            return self.copy_ctas
        if key is not None and key in self._tuned:
            return self._tuned[key]
        if os.environ.get("INCIN_TP_COPY", "ctas") == "warps":
            return -max(1, int(os.environ.get("INCIN_TP_COPY_STAGES", "2")))   # operand stages that become the copy ring
        best, best_t = 8, float("inf")
        for c in range(4, 73, 4):
            t = max(copy_bytes / (c * (self.COPY_CTA_GBS_PUSH if push else self.COPY_CTA_GBS) * 1e9), link_bytes / (self.LINK_GBS * 1e9),
                    flops / (self.GEMM_TFLOPS * 1e12 * (148 - c) / 148))
            if t < best_t * 0.97:      # prefer fewer copy CTAs unless more of them buy at least 3 %
                best, best_t = c, t
        return best

    def barrier(self) -> None:
        """Cross-GPU barrier as one tiny kernel on the current stream (bounded waits, status word on timeout)."""
        nat.check(nat.cuda().incin_peer_barrier(self._pad_ptrs.data_ptr(), self.world, self.rank, 0,
                                               status_word(self.device).data_ptr(), nat.stream_ptr()), "peer_barrier")

    def gather_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False, out: torch.Tensor | None = None,
                    ldc: int | None = None, c_offset: int = 0, tag: int | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """``(all_gather(x_shard) @ W^T, gathered)``: x_shard ``[Ml, Kd]`` bf16, W ``[N, Kd]`` (or ``[Kd, N]`` with
        ``b_mn``).  Returns the product ``[tp*Ml, N]`` and the gathered input (kept for the weight gradient)."""
        Ml, Kd = x_shard.shape
        self._planned(tag, CollectiveKind.all_gather(), Ml * Kd)      # Sharded(0) -> Replicated: Ml x Kd elements in
        if self.mode == "nccl":
            M = Ml * self.world
            N = w.shape[1] if b_mn else w.shape[0]
            gathered = torch.empty(M, Kd, dtype=torch.bfloat16, device=self.device)
            dist.all_gather_into_tensor(gathered, x_shard.contiguous(), group=self.group)
            if out is None:
                out, ldc = torch.empty(M, N, dtype=torch.bfloat16, device=self.device), N
            G.gemm(gathered, w, out, M=M, N=N, K=Kd, lda=Kd, ldb=(N if b_mn else Kd), ldc=ldc, b_mn=b_mn,
                   c_offset=c_offset)
            return out, gathered
        if Ml % 128 or Ml > self.rows or Kd > self.cols or Kd % 8:
            raise ValueError(f"shard [{Ml}, {Kd}] does not fit the tensor-parallel buffers [{self.rows}, {self.cols}]")
        self._maybe_tune("gather", x_shard, w, b_mn, ("gather", Ml, Kd, w.shape[1] if b_mn else w.shape[0]))
        p = self._shard_parity
        self._shard_parity ^= 1
        buf = self.shard[p]
        buf.typed(torch.bfloat16, Ml * Kd).view(Ml, Kd).copy_(x_shard)
        self.barrier()   # every peer's shard of this parity is written; every peer is done with this parity's last use
        M = Ml * self.world
        N = w.shape[1] if b_mn else w.shape[0]
        gathered = torch.empty(M, Kd, dtype=torch.bfloat16, device=self.device)
        # this rank's own rows go into place with one local copy; the fused launch moves only the peers' shards
        gathered[self.rank * Ml:(self.rank + 1) * Ml].copy_(x_shard)
        src = list(buf.ptrs)
        src[self.rank] = 0
        flags = torch.zeros(M // 128, dtype=torch.int32, device=self.device)
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=self.device)
            ldc = N
        G.gemm(gathered, w, out, M=M, N=N, K=Kd, lda=Kd, ldb=(N if b_mn else Kd), ldc=ldc, b_mn=b_mn, c_offset=c_offset,
               gather={"world": self.world, "rank": self.rank, "rows_per_rank": Ml, "src": src, "flags": flags,
                       "copy_ctas": self._copy_ctas((self.world - 1) * Ml * Kd * 2, (self.world - 1) * Ml * Kd * 2,
                                                    2.0 * M * N * Kd, key=("gather", Ml, Kd, N))})
        return out, gathered

    def gemm_scatter(self, a: torch.Tensor, w: torch.Tensor, *, b_mn: bool = False,
                     residual: torch.Tensor | None = None, tag: int | None = None) -> torch.Tensor:
        """``reduce_scatter(a @ W^T) (+ residual)``: a ``[M, Kd]`` (full rows, local K shard), W ``[N, Kd]`` (or
        ``[Kd, N]`` with ``b_mn``) -> ``[M / tp, N]`` rows owned by this rank."""
        M, Kd = a.shape
        N = w.shape[1] if b_mn else w.shape[0]
        Ml = M // self.world
        self._planned(tag, CollectiveKind.reduce_scatter(Reduction.SUM), M * N)   # Partial(Sum) -> Sharded(0): M x N in
        if self.mode == "nccl":
            full = torch.empty(M, N, dtype=torch.bfloat16, device=self.device)
            G.gemm(a, w, full, M=M, N=N, K=Kd, lda=Kd, ldb=(N if b_mn else Kd), ldc=N, b_mn=b_mn)
            out = torch.empty(Ml, N, dtype=torch.bfloat16, device=self.device)
            dist.reduce_scatter_tensor(out, full, group=self.group)
            return out if residual is None else out + residual
        if M % self.world or Ml % 128 or Ml > self.rows or N > self.cols or N % 8:
            raise ValueError(f"product [{M}, {N}] does not fit the tensor-parallel buffers")
        self._maybe_tune("scatter", a, w, b_mn, ("scatter", Ml, Kd, N))
        p = self._slot_parity
        self._slot_parity ^= 1
        buf = self.slots[p]
        # tiles owned by peers are staged locally and pushed by copy CTAs of the same launch (large bulk transfers
        # over NVLink instead of one small store per thread); this rank's own tiles go straight into its slot
        stage = torch.empty(M, N, dtype=torch.bfloat16, device=self.device)
        ready = torch.zeros(M // 128, dtype=torch.int32, device=self.device)
        remote = (self.world - 1) * Ml * N * 2
        G.gemm(a, w, stage, M=M, N=N, K=Kd, lda=Kd, ldb=(N if b_mn else Kd), ldc=N, b_mn=b_mn,
               scatter={"world": self.world, "rank": self.rank, "rows_per_rank": Ml, "dst": buf.ptrs,
                        "slot_stride": Ml * N, "ready": ready,
                        "copy_ctas": self._copy_ctas(remote, remote, 2.0 * M * N * Kd, push=True,
                                                     key=("scatter", Ml, Kd, N))})
        self.barrier()   # every peer's tiles for my rows have landed in my slot buffer
        out = torch.empty(Ml, N, dtype=torch.bfloat16, device=self.device)
        nat.check(nat.cuda().incin_slot_reduce(buf.ptr, Ml * N, self.world, nat.ptr(residual), out.data_ptr(), Ml, N, N,
                                              nat.stream_ptr()), "slot_reduce")
        return out


# ---------------------------------------------------------------------------------------------------- autograd
def _tags(tp_id: int | None, forward: TensorParallelCollective, backward: TensorParallelCollective):
    """Plan tags of one parallel linear: its forward collective and the adjoint its backward pass runs."""
    if tp_id is None:
        return None, None
    return tp_tag(2 * tp_id, forward), tp_tag(2 * tp_id + 1, backward)


class _ColumnParallel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, tp: TensorParallel, tp_id, *weights):
        x_shard = x_shard.contiguous()
        n_total = sum(w.shape[0] for w in weights)
        M = x_shard.shape[0] * tp.world
        out = torch.empty(M, n_total, dtype=torch.bfloat16, device=x_shard.device)
        tag_f, ctx.tag_b = _tags(tp_id, TensorParallelCollective.COLUMN_OUTPUT_GATHER, TensorParallelCollective.ROW_OUTPUT_SCATTER)
        _, gathered = tp.gather_gemm(x_shard, weights[0], out=out, ldc=n_total, c_offset=0, tag=tag_f)
        off = weights[0].shape[0]
        for w in weights[1:]:      # further weights reuse the gathered rows: plain local GEMMs
            G.gemm(gathered, w, out, M=M, N=w.shape[0], K=w.shape[1], lda=w.shape[1], ldb=w.shape[1], ldc=n_total,
                   c_offset=off)
            off += w.shape[0]
        ctx.save_for_backward(gathered, *weights)
        ctx.tp = tp
        return out

    @staticmethod
    def backward(ctx, dy):
        gathered, *weights = ctx.saved_tensors
        tp, dy = ctx.tp, dy.contiguous()
        M, n_total = dy.shape
        Kd = gathered.shape[1]
        # weight gradients from the gathered input
        off = 0
        for w in weights:
            n = w.shape[0]
            if w.requires_grad:
                G.gemm(dy, gathered, main_grad(w), M=n, N=Kd, K=M, lda=n_total, ldb=Kd, ldc=Kd, a_mn=True, b_mn=True,
                       accumulate=True, splits=G.auto_splits(n, Kd, M), a_offset=off)
            off += n
        # dx = dy @ [W0; W1; ...]: partial over the output shards -> reduce-scatter over rows
        if len(weights) == 1:
            dx = tp.gemm_scatter(dy, weights[0], b_mn=True, tag=ctx.tag_b)
        else:
            wcat = torch.cat(list(weights), dim=0)
            dx = tp.gemm_scatter(dy, wcat, b_mn=True, tag=ctx.tag_b)
        for w in weights:      # after the last enqueued reader of the weights (a ready callback may start their update)
            if w.requires_grad:
                _ready(w)
        return (dx, None, None) + (None,) * len(weights)


class _RowParallel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, tp: TensorParallel, tp_id, w, residual_shard):
        a = a.contiguous()
        ctx.save_for_backward(a, w)
        ctx.tp, ctx.has_res = tp, residual_shard is not None
        tag_f, ctx.tag_b = _tags(tp_id, TensorParallelCollective.ROW_OUTPUT_SCATTER, TensorParallelCollective.COLUMN_OUTPUT_GATHER)
        return tp.gemm_scatter(a, w, residual=residual_shard.contiguous() if residual_shard is not None else None, tag=tag_f)

    @staticmethod
    def backward(ctx, dy_shard):
        a, w = ctx.saved_tensors
        tp, dy_shard = ctx.tp, dy_shard.contiguous()
        # da = all_gather(dy) @ W   (W is [N, Kd]: read MN-major);  dW += all_gather(dy)^T @ a
        da, dy_full = tp.gather_gemm(dy_shard, w, b_mn=True, tag=ctx.tag_b)
        if w.requires_grad:
            M, N = dy_full.shape
            Kd = a.shape[1]
            G.gemm(dy_full, a, main_grad(w), M=N, N=Kd, K=M, lda=N, ldb=Kd, ldc=Kd, a_mn=True, b_mn=True,
                   accumulate=True, splits=G.auto_splits(N, Kd, M))
            _ready(w)
        return da, None, None, None, (dy_shard if ctx.has_res else None)


def parallel_linear(x, tp: TensorParallel, weights, *, src: Placement, dst: Placement, tp_id: int | None = None,
                    residual_shard=None):
    """A linear layer over the tensor-parallel group, LOWERED FROM THE PLACEMENTS of its activation: the transition
    ``src -> dst`` that the layer has to realise decides the fused kernel, as the reference lowers its
    ``TensorParallelCollective`` descriptors (crates/incin-backends/src/dist/nccl.rs:741-791):

    * input ``Sharded(0)`` (token rows), needed ``Replicated``  -> all-gather -> GEMM (column-parallel weights);
    * product ``Partial(Sum)``, wanted ``Sharded(0)``           -> GEMM -> reduce-scatter (row-parallel weight).

    Anything else has no fused kernel and is refused with the reason.  ``tp_id`` names the layer in the step's plan."""
    tr = validate_transition(src, dst)
    weights = tuple(weights) if isinstance(weights, (tuple, list)) else (weights,)
    if tr is PlacementTransition.ALL_GATHER:
        if src.tensor_axis != 0 or residual_shard is not None:
            raise PlacementError("the fused all-gather -> GEMM gathers token rows (Sharded(0)) and takes no residual")
        return _ColumnParallel.apply(x, tp, tp_id, *weights)
    if tr is PlacementTransition.REDUCE_SCATTER:
        if dst.tensor_axis != 0 or src.reduction is not Reduction.SUM or len(weights) != 1:
            raise PlacementError("the fused GEMM -> reduce-scatter sums partial products into token-row shards (one weight)")
        return _RowParallel.apply(x, tp, tp_id, weights[0], residual_shard)
    raise PlacementError(f"no fused tensor-parallel kernel realises {src.token()} -> {dst.token()} ({tr.value})")


def column_parallel_linear(x_shard, tp: TensorParallel, *weights, tp_id: int | None = None):
    """``all_gather(x_shard) @ cat(weights)^T`` -> ``[M, sum(out_i)]`` (columns of this rank's weight shards):
    the ``Sharded(0) -> Replicated`` lowering of :func:`parallel_linear`."""
    return parallel_linear(x_shard, tp, weights, src=Sharded(0), dst=Replicated(), tp_id=tp_id)


def row_parallel_linear(a, tp: TensorParallel, w, residual_shard=None, tp_id: int | None = None):
    """``reduce_scatter(a @ w^T) + residual_shard`` -> ``[M / tp, N]``: the ``Partial(Sum) -> Sharded(0)`` lowering."""
    return parallel_linear(a, tp, (w,), src=Partial(Reduction.SUM), dst=Sharded(0), tp_id=tp_id, residual_shard=residual_shard)


class PeerRangeSum:
    """In-place all-reduce(sum) of fp32 element ranges of a peer-mapped buffer over a sub-group of ranks.  All
    device-side tables are built once, so ``run()`` only enqueues kernels (capturable in a CUDA graph)."""

    def __init__(self, bufs: SymmetricBuffer, ranges: list[tuple[int, int]], group_ranks: list[int], my_rank: int,
                 tp: TensorParallel, device):
        order = sorted(group_ranks)
        self.tp, self.n_peers, self.n_ranges = tp, len(order), len(ranges)
        self.bases_all = torch.tensor([bufs.ptrs[r] for r in order], dtype=torch.int64, device=device)
        self.base_self = torch.tensor([bufs.ptrs[my_rank]], dtype=torch.int64, device=device)
        self.ranges = torch.tensor(ranges, dtype=torch.int64, device=device).reshape(-1)
        self.scratch = torch.empty(sum(k for _, k in ranges), dtype=torch.float32, device=device)

    def run(self) -> None:
        lib = nat.cuda()
        self.tp.barrier()    # every peer's gradients are final
        nat.check(lib.incin_peer_sum_ranges(self.bases_all.data_ptr(), self.n_peers, self.ranges.data_ptr(),
                                            self.n_ranges, self.scratch.data_ptr(), 0, nat.stream_ptr()), "peer_sum")
        self.tp.barrier()    # every peer has finished reading before anyone overwrites
        nat.check(lib.incin_peer_sum_ranges(self.base_self.data_ptr(), 1, self.ranges.data_ptr(), self.n_ranges,
                                            self.scratch.data_ptr(), 1, nat.stream_ptr()), "peer_sum")
