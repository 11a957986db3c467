"""Plan builders for data, tensor and pipeline parallelism.

Counterparts: crates/incin-core/src/dist/data_parallel.rs (one ``AllReduce(Mean)``
``Partial<Mean> -> Replicated`` per gradient, chained by ``depends_on``), dist/tensor_parallel.rs
(ColumnOutputGather{axis} / RowOutputSum / AttentionHeadGather{axis}; tag ``(id << 2) | code``) and
dist/pipeline.rs (GPipe and 1F1B transfer orders, tag ``(boundary << 33) | (microbatch << 1) | dir``,
clock timeline with bubble and live-activation evidence).

Differences that follow from the fused kernels of this build: the DP builder plans one collective per
gradient *bucket* (the unit ``incin_dp_reduce_adamw`` works on), and the TP builder can emit the
reduce-scatter form of the row-parallel output (legal in the reference's rule table but never emitted
by its builders) because the fused GEMM -> reduce-scatter kernel produces exactly that placement.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass

from ..core.dtype import DTypeId
from .mesh import Axis, DeviceMesh
from .placement import Partial, PipelineStage, Reduction, Replicated, Sharded
from .plan import CollectiveKind, CollectivePlan, CollectivePlanBuilder, PlanError


# --------------------------------------------------------------------------------------------- data parallel
class DataParallelPlanBuilder:
    """``push(gradient_id, elements, dtype)`` per bucket, in the order the backward pass completes them."""

    def __init__(self, mesh: DeviceMesh, rank: int = 0, axis: Axis = Axis.DATA):
        """``axis``: the mesh axis the gradients are averaged over (DATA; TENSOR for the replicated parameters of a
        tensor-parallel model, whose gradients are partial over the token shards of the tensor-parallel group)."""
        self._b = CollectivePlanBuilder(mesh, rank)
        self._last: int | None = None
        self.axis = axis

    def push(self, gradient_id: int, elements: int, dtype: DTypeId = DTypeId.F32) -> int:
        seq = self._b.push(gradient_id, self.axis, CollectiveKind.all_reduce(Reduction.MEAN), elements, dtype,
                           Partial(Reduction.MEAN, self.axis), Replicated(), depends_on=self._last)
        self._last = seq
        return seq

    def finish(self) -> CollectivePlan:
        return self._b.finish()


# --------------------------------------------------------------------------------------------- tensor parallel
class TensorParallelCollective(enum.Enum):
    COLUMN_OUTPUT_GATHER = 0   # Sharded{axis} -> Replicated (all-gather)
    ROW_OUTPUT_SUM = 1         # Partial<Sum>  -> Replicated (all-reduce)
    ATTENTION_HEAD_GATHER = 2  # Sharded{head axis} -> Replicated
    ROW_OUTPUT_SCATTER = 3     # Partial<Sum>  -> Sharded{axis} (reduce-scatter; fused GEMM epilogue)


def tp_tag(tp_id: int, collective: TensorParallelCollective) -> int:
    return (tp_id << 2) | collective.value


class TensorParallelPlanBuilder:
    def __init__(self, mesh: DeviceMesh, rank: int = 0):
        self._b = CollectivePlanBuilder(mesh, rank)
        self.mesh = mesh

    def _local(self, global_shape, axis) -> int:
        n = self.mesh.spec.tp
        if global_shape[axis] % n:
            raise PlanError(f"extent {global_shape[axis]} of axis {axis} does not divide over tp={n}")
        e = 1
        for i, d in enumerate(global_shape):
            e *= d // n if i == axis else d
        return e

    def push_column(self, tp_id: int, global_shape, axis: int, dtype=DTypeId.BF16) -> int:
        return self._b.push(tp_tag(tp_id, TensorParallelCollective.COLUMN_OUTPUT_GATHER), Axis.TENSOR,
                            CollectiveKind.all_gather(), self._local(global_shape, axis), dtype, Sharded(axis),
                            Replicated())

    def push_attention(self, tp_id: int, global_shape, head_axis: int, dtype=DTypeId.BF16) -> int:
        return self._b.push(tp_tag(tp_id, TensorParallelCollective.ATTENTION_HEAD_GATHER), Axis.TENSOR,
                            CollectiveKind.all_gather(), self._local(global_shape, head_axis), dtype,
                            Sharded(head_axis), Replicated())

    def push_row(self, tp_id: int, global_shape, dtype=DTypeId.BF16) -> int:
        e = 1
        for d in global_shape:
            e *= d
        return self._b.push(tp_tag(tp_id, TensorParallelCollective.ROW_OUTPUT_SUM), Axis.TENSOR,
                            CollectiveKind.all_reduce(Reduction.SUM), e, dtype, Partial(Reduction.SUM), Replicated())

    def push_row_scatter(self, tp_id: int, global_shape, axis: int, dtype=DTypeId.BF16) -> int:
        e = 1
        for d in global_shape:
            e *= d
        return self._b.push(tp_tag(tp_id, TensorParallelCollective.ROW_OUTPUT_SCATTER), Axis.TENSOR,
                            CollectiveKind.reduce_scatter(Reduction.SUM), e, dtype, Partial(Reduction.SUM),
                            Sharded(axis))

    def finish(self) -> CollectivePlan:
        return self._b.finish()


# --------------------------------------------------------------------------------------------- pipeline
class PipelineSchedule(enum.Enum):
    GPIPE = "gpipe"
    ONE_F_ONE_B = "1f1b"


class ActivationCheckpoint(enum.Enum):
    KEEP = "keep"
    RECOMPUTE = "recompute"


class PipelineTransfer(enum.Enum):
    FORWARD_ACTIVATION = 0
    BACKWARD_GRADIENT = 1


def pp_tag(boundary: int, microbatch: int, transfer: PipelineTransfer) -> int:
    return (boundary << 33) | (microbatch << 1) | transfer.value


def transfer_order(schedule: PipelineSchedule, microbatches: int) -> list[tuple[PipelineTransfer, int]]:
    F, B = PipelineTransfer.FORWARD_ACTIVATION, PipelineTransfer.BACKWARD_GRADIENT
    if schedule is PipelineSchedule.GPIPE:
        return [(F, m) for m in range(microbatches)] + [(B, m) for m in reversed(range(microbatches))]
    order = [(F, 0)]
    for m in range(1, microbatches):
        order += [(F, m), (B, m - 1)]
    order.append((B, microbatches - 1))
    return order


@dataclass(frozen=True)
class PipelineTimeline:
    clocks: tuple[tuple[str | None, ...], ...]   # clocks[t][stage] = "F3" / "B1" / None (bubble)
    bubble_slots: int
    peak_live_activations: tuple[int, ...]       # per stage

    @property
    def bubble_fraction(self) -> float:
        total = len(self.clocks) * len(self.clocks[0]) if self.clocks else 1
        return self.bubble_slots / total


def build_timeline(schedule: PipelineSchedule, stages: int, microbatches: int,
                   checkpoint: ActivationCheckpoint = ActivationCheckpoint.KEEP) -> PipelineTimeline:
    """Greedy clocked simulation: forward of microbatch m on stage s needs F(m, s-1); backward needs
    B(m, s+1) (and F(m, s)).  1F1B prefers a ready backward over a forward once a stage holds
    ``stages - s`` microbatches in flight; GPipe runs every forward first."""
    done_f = [[-1] * stages for _ in range(microbatches)]
    done_b = [[-1] * stages for _ in range(microbatches)]
    next_f, next_b = [0] * stages, [0] * stages
    live, peak = [0] * stages, [0] * stages
    clocks, t, bubbles = [], 0, 0
    b_order = (list(reversed(range(microbatches))) if schedule is PipelineSchedule.GPIPE else list(range(microbatches)))
    while any(nb < microbatches for nb in next_b):
        row = []
        for s in range(stages):
            act = None
            can_b = False
            if next_b[s] < microbatches:
                m = b_order[next_b[s]]
                dep = done_b[m][s + 1] if s + 1 < stages else done_f[m][s]
                can_b = 0 <= dep < t and 0 <= done_f[m][s] < t
            can_f = False
            if next_f[s] < microbatches:
                mf = next_f[s]
                can_f = s == 0 or 0 <= done_f[mf][s - 1] < t
            prefer_b = can_b and (schedule is PipelineSchedule.ONE_F_ONE_B
                                  or schedule is PipelineSchedule.GPIPE and next_f[s] >= microbatches)
            if prefer_b:
                m = b_order[next_b[s]]
                done_b[m][s] = t
                next_b[s] += 1
                live[s] -= 1
                act = f"B{m}"
            elif can_f and (schedule is PipelineSchedule.GPIPE or live[s] < stages - s):
                m = next_f[s]
                done_f[m][s] = t
                next_f[s] += 1
                live[s] += 1
                peak[s] = max(peak[s], live[s])
                act = f"F{m}"
            else:
                bubbles += 1
            row.append(act)
        clocks.append(tuple(row))
        t += 1
        if t > 8 * (microbatches + stages) * 2:
            raise PlanError("pipeline schedule did not converge")
    if checkpoint is ActivationCheckpoint.RECOMPUTE:
        peak = [1 if p else 0 for p in peak]   # only stage inputs are kept; the rest is recomputed
    return PipelineTimeline(tuple(clocks), bubbles, tuple(peak))


class PipelinePlanBuilder:
    """Activation / gradient transfers across every stage boundary, in schedule order."""

    def __init__(self, mesh: DeviceMesh, rank: int = 0):
        self.mesh, self.rank = mesh, rank

    def build(self, schedule: PipelineSchedule, microbatches: int, activation_elements: int,
              dtype: DTypeId = DTypeId.BF16,
              checkpoint: ActivationCheckpoint = ActivationCheckpoint.KEEP) -> tuple[CollectivePlan, PipelineTimeline]:
        if microbatches < 1:
            raise PlanError("at least one microbatch")
        stages = self.mesh.spec.pp
        if stages < 2:
            raise PlanError("a pipeline needs at least two stages")
        b = CollectivePlanBuilder(self.mesh, self.rank)
        group = self.mesh.group_of(self.rank, Axis.PIPELINE)
        last = None
        for transfer, m in transfer_order(schedule, microbatches):
            for boundary in range(stages - 1):
                lo, hi = group.ranks[boundary], group.ranks[boundary + 1]
                src, dst = (lo, hi) if transfer is PipelineTransfer.FORWARD_ACTIVATION else (hi, lo)
                s_stage = boundary if transfer is PipelineTransfer.FORWARD_ACTIVATION else boundary + 1
                d_stage = boundary + 1 if transfer is PipelineTransfer.FORWARD_ACTIVATION else boundary
                last = b.push_send_recv_tagged(pp_tag(boundary, m, transfer), src, dst, activation_elements, dtype,
                                               PipelineStage(s_stage), PipelineStage(d_stage), depends_on=last)
        return b.finish(), build_timeline(schedule, stages, microbatches, checkpoint)
