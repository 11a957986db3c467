"""Collective vocabulary, descriptors, plans with a stable hash, and the cross-rank preflight.

Counterpart of crates/incin-core/src/dist/collective.rs (CollectiveKind + adjoint, CollectiveDType,
GroupId, StreamId) and dist/plan.rs (CollectiveDescriptor :74-88, CollectivePlanBuilder :210-458, stable
FNV-1a plan hash over "incin.collective.plan.v2" :843-866, PlanSummary, preflight -> AgreedPlan
:590-651).  A plan is the ordered list of collectives a step will issue; every rank builds it
independently, the hashes are compared BEFORE any communicator or peer mapping is created, and a
divergent rank is rejected on the host instead of deadlocking a collective on the device.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field

from ..core.dtype import DTypeId, size_bytes
from .mesh import Axis, CollectiveGroup, DeviceMesh, Digest
from .placement import Placement, PlacementError, PlacementTransition, Reduction, validate_transition


class CollectiveOp(enum.Enum):
    ALL_REDUCE = "all_reduce"
    ALL_GATHER = "all_gather"
    REDUCE_SCATTER = "reduce_scatter"
    ALL_TO_ALL = "all_to_all"
    SEND_RECV = "send_recv"


@dataclass(frozen=True)
class CollectiveKind:
    op: CollectiveOp
    reduction: Reduction | None = None
    src: int | None = None
    dst: int | None = None

    @staticmethod
    def all_reduce(r: Reduction = Reduction.SUM) -> "CollectiveKind":
        return CollectiveKind(CollectiveOp.ALL_REDUCE, r)

    @staticmethod
    def all_gather() -> "CollectiveKind":
        return CollectiveKind(CollectiveOp.ALL_GATHER)

    @staticmethod
    def reduce_scatter(r: Reduction = Reduction.SUM) -> "CollectiveKind":
        return CollectiveKind(CollectiveOp.REDUCE_SCATTER, r)

    @staticmethod
    def all_to_all() -> "CollectiveKind":
        return CollectiveKind(CollectiveOp.ALL_TO_ALL)

    @staticmethod
    def send_recv(src: int, dst: int) -> "CollectiveKind":
        return CollectiveKind(CollectiveOp.SEND_RECV, None, src, dst)

    def adjoint(self) -> "CollectiveKind":
        """The collective the backward pass issues for this forward collective."""
        if self.op is CollectiveOp.ALL_GATHER:
            return CollectiveKind.reduce_scatter(Reduction.SUM)
        if self.op is CollectiveOp.REDUCE_SCATTER:
            return CollectiveKind.all_gather()
        if self.op is CollectiveOp.SEND_RECV:
            return CollectiveKind.send_recv(self.dst, self.src)
        return self  # all-reduce(sum) and all-to-all are self-adjoint

    def token(self) -> str:
        t = self.op.value
        if self.reduction is not None:
            t += ":" + self.reduction.value
        if self.op is CollectiveOp.SEND_RECV:
            t += f":{self.src}>{self.dst}"
        return t


COLLECTIVE_DTYPES = (DTypeId.F32, DTypeId.F64, DTypeId.F16, DTypeId.BF16, DTypeId.I64, DTypeId.U32, DTypeId.U8)


class PlanError(ValueError):
    pass


@dataclass(frozen=True)
class CollectiveDescriptor:
    tag: int
    group: CollectiveGroup
    kind: CollectiveKind
    input_elements: int
    output_elements: int
    dtype: DTypeId
    source: Placement
    destination: Placement
    sequence: int
    stream: int = 0
    depends_on: int | None = None

    @property
    def input_bytes(self) -> int:
        return size_bytes(self.dtype, self.input_elements)

    @property
    def output_bytes(self) -> int:
        return size_bytes(self.dtype, self.output_elements)


@dataclass(frozen=True)
class PlanSummary:
    collectives: int
    bytes_in: int
    bytes_out: int
    by_kind: dict


@dataclass(frozen=True)
class CollectivePlan:
    mesh_id: int
    descriptors: tuple[CollectiveDescriptor, ...]
    hash: int

    def summary(self) -> PlanSummary:
        by: dict[str, int] = {}
        for d in self.descriptors:
            by[d.kind.op.value] = by.get(d.kind.op.value, 0) + 1
        return PlanSummary(len(self.descriptors), sum(d.input_bytes for d in self.descriptors),
                           sum(d.output_bytes for d in self.descriptors), by)


def plan_hash(mesh_id: int, descriptors) -> int:
    dg = Digest().bytes(b"incin.collective.plan.v2").number(mesh_id).number(len(descriptors))
    for d in descriptors:
        dg.number(d.tag).text(d.group.token()).number(len(d.group.ranks)).text(d.kind.token())
        dg.number(d.input_elements).number(d.output_elements).number(d.input_bytes).number(d.output_bytes)
        dg.text(d.dtype.value).text(d.source.token()).text(d.destination.token())
        dg.number(d.sequence).number(d.stream).number((1 << 64) - 1 if d.depends_on is None else d.depends_on)
    return dg.finish()


_EXPECTED = {PlacementTransition.ALL_GATHER: CollectiveOp.ALL_GATHER,
             PlacementTransition.ALL_REDUCE: CollectiveOp.ALL_REDUCE,
             PlacementTransition.REDUCE_SCATTER: CollectiveOp.REDUCE_SCATTER}


class CollectivePlanBuilder:
    def __init__(self, mesh: DeviceMesh, rank: int = 0):
        self.mesh, self.rank = mesh, rank
        self._descs: list[CollectiveDescriptor] = []
        self._tags: set[int] = set()

    def push(self, tag: int, axis: Axis, kind: CollectiveKind, elements: int, dtype: DTypeId, source: Placement,
             destination: Placement, *, stream: int = 0, depends_on: int | None = None) -> int:
        """Append one collective; returns its sequence number (usable as ``depends_on`` of a later one)."""
        if tag in self._tags:
            raise PlanError(f"duplicate collective tag {tag}")
        if dtype not in COLLECTIVE_DTYPES:
            raise PlanError(f"{dtype.value} cannot travel through a collective")
        if elements <= 0:
            raise PlanError("a collective moves at least one element")
        group = self.mesh.group_of(self.rank, axis)
        n = len(group.ranks)
        if kind.op is not CollectiveOp.ALL_TO_ALL and kind.op is not CollectiveOp.SEND_RECV:
            try:
                tr = validate_transition(source, destination)
            except PlacementError as e:
                raise PlanError(str(e)) from None
            if _EXPECTED.get(tr) is not kind.op:
                raise PlanError(f"{kind.op.value} does not realise {source.token()} -> {destination.token()}")
        if kind.reduction is not None and dtype in (DTypeId.U8,) and kind.reduction is Reduction.MEAN:
            raise PlanError("mean is not defined for u8")
        if kind.op is CollectiveOp.ALL_GATHER:
            out = elements * n
        elif kind.op is CollectiveOp.REDUCE_SCATTER:
            if elements % n:
                raise PlanError(f"{elements} elements do not scatter evenly over {n} ranks")
            out = elements // n
        elif kind.op is CollectiveOp.ALL_TO_ALL:
            if elements % n:
                raise PlanError(f"{elements} elements do not split evenly over {n} ranks")
            out = elements
        else:
            out = elements
        if depends_on is not None and not 0 <= depends_on < len(self._descs):
            raise PlanError("depends_on must name an earlier collective of this plan")
        seq = len(self._descs)
        self._descs.append(CollectiveDescriptor(tag, group, kind, elements, out, dtype, source, destination, seq,
                                                stream, depends_on))
        self._tags.add(tag)
        return seq

    def push_send_recv_tagged(self, tag: int, src: int, dst: int, elements: int, dtype: DTypeId,
                              source: Placement, destination: Placement, *, depends_on: int | None = None) -> int:
        group = self.mesh.group_of(self.rank, Axis.PIPELINE)
        if src == dst or src not in group.ranks or dst not in group.ranks:
            raise PlanError(f"send/recv {src}->{dst} is not between two ranks of the pipeline group")
        return self.push(tag, Axis.PIPELINE, CollectiveKind.send_recv(src, dst), elements, dtype, source, destination,
                         depends_on=depends_on)

    def finish(self) -> CollectivePlan:
        ds = tuple(self._descs)
        return CollectivePlan(self.mesh.mesh_id, ds, plan_hash(self.mesh.mesh_id, ds))


@dataclass(frozen=True)
class AgreedPlan:
    plan: CollectivePlan
    world: int


class PreflightError(RuntimeError):
    pass


def preflight(world: int, reports: list[tuple[int, int, int]], local: CollectivePlan) -> AgreedPlan:
    """``reports[r] = (mesh_id, plan_hash, count)`` gathered from every rank (rendezvous all-gather).
    Any disagreement is rejected here, before a communicator or peer mapping exists."""
    if len(reports) != world:
        raise PreflightError(f"expected {world} plan reports, got {len(reports)}")
    mine = (local.mesh_id, local.hash, len(local.descriptors))
    for r, rep in enumerate(reports):
        if rep[0] != mine[0]:
            raise PreflightError(f"rank {r} bound a different mesh ({rep[0]:#x} vs {mine[0]:#x})")
        if rep[2] != mine[2]:
            raise PreflightError(f"rank {r} plans {rep[2]} collectives, this rank {mine[2]}")
        if rep[1] != mine[1]:
            raise PreflightError(f"rank {r} built a divergent plan ({rep[1]:#x} vs {mine[1]:#x})")
    return AgreedPlan(local, world)


class PlanCursor:
    """Launch-time contract (crates/incin-backends/src/dist/nccl.rs:1241-1280): collectives are issued in
    plan order and must match the planned dtype / element counts; any violation is fail-stop."""

    def __init__(self, agreed: AgreedPlan):
        self.agreed, self.cursor = agreed, 0

    def next(self, *, tag: int, kind: CollectiveKind, elements: int, dtype: DTypeId) -> CollectiveDescriptor:
        ds = self.agreed.plan.descriptors
        if self.cursor >= len(ds):
            raise PlanError("more collectives issued than planned")
        d = ds[self.cursor]
        if d.tag != tag or d.kind != kind or d.input_elements != elements or d.dtype is not dtype:
            raise PlanError(f"launch #{self.cursor} ({kind.token()}, tag {tag}, {elements} x {dtype.value}) "
                            f"does not match the plan ({d.kind.token()}, tag {d.tag}, {d.input_elements} x {d.dtype.value})")
        self.cursor += 1
        return d

    def reset(self) -> None:
        self.cursor = 0
