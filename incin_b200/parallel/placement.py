"""Placements of a tensor on a mesh and the table of legal transitions between them.

Counterpart of crates/incin-core/src/dist/placement.rs (Local / Replicated / Sharded<Mesh, Axis> /
Partial<Mesh, R> / PipelineStage<Mesh, I>) and dist/rule.rs (LegalTransition: Identity, LocalShard,
AllGather, AllReduce, ReduceScatter; ShardDivisible; ElementwisePlacement; ReduceShardedAxis).
The reference proves these at compile time; here ``validate_transition`` / ``validate_shard`` raise
:class:`PlacementError` before any plan is built, so an illegal redistribution never reaches a transport.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass

from .mesh import Axis, MeshSpec


class PlacementKind(enum.Enum):
    LOCAL = "local"
    REPLICATED = "replicated"
    SHARDED = "sharded"
    PARTIAL = "partial"
    PIPELINE_STAGE = "pipeline_stage"


class Reduction(enum.Enum):
    SUM = "sum"
    MEAN = "mean"
    MAX = "max"
    MIN = "min"
    PROD = "prod"


@dataclass(frozen=True)
class Placement:
    kind: PlacementKind
    mesh_axis: Axis | None = None      # which mesh axis the tensor is sharded / partial over
    tensor_axis: int | None = None     # Sharded: which tensor dimension is split
    reduction: Reduction | None = None # Partial: how the per-rank values combine
    stage: int | None = None           # PipelineStage: owning stage

    def token(self) -> str:
        parts = [self.kind.value]
        if self.mesh_axis is not None:
            parts.append(self.mesh_axis.value)
        if self.tensor_axis is not None:
            parts.append(f"dim{self.tensor_axis}")
        if self.reduction is not None:
            parts.append(self.reduction.value)
        if self.stage is not None:
            parts.append(f"stage{self.stage}")
        return ":".join(parts)


Local = Placement(PlacementKind.LOCAL)


def Replicated() -> Placement:
    return Placement(PlacementKind.REPLICATED)


def Sharded(tensor_axis: int, mesh_axis: Axis = Axis.TENSOR) -> Placement:
    if tensor_axis < 0:
        raise ValueError("tensor axis must be >= 0")
    return Placement(PlacementKind.SHARDED, mesh_axis, tensor_axis)


def Partial(reduction: Reduction = Reduction.SUM, mesh_axis: Axis = Axis.TENSOR) -> Placement:
    return Placement(PlacementKind.PARTIAL, mesh_axis, None, reduction)


def PipelineStage(stage: int) -> Placement:
    return Placement(PlacementKind.PIPELINE_STAGE, Axis.PIPELINE, None, None, stage)


class PlacementTransition(enum.Enum):
    IDENTITY = "identity"
    LOCAL_SHARD = "local_shard"        # Replicated -> Sharded: slice locally, no communication
    ALL_GATHER = "all_gather"          # Sharded -> Replicated
    ALL_REDUCE = "all_reduce"          # Partial -> Replicated
    REDUCE_SCATTER = "reduce_scatter"  # Partial -> Sharded


class PlacementError(ValueError):
    pass


def validate_transition(src: Placement, dst: Placement) -> PlacementTransition:
    k, K = src.kind, PlacementKind
    if src == dst:
        return PlacementTransition.IDENTITY
    if k is K.REPLICATED and dst.kind is K.SHARDED:
        return PlacementTransition.LOCAL_SHARD
    if k is K.SHARDED and dst.kind is K.REPLICATED:
        return PlacementTransition.ALL_GATHER
    if k is K.PARTIAL and dst.kind is K.REPLICATED:
        return PlacementTransition.ALL_REDUCE
    if k is K.PARTIAL and dst.kind is K.SHARDED:
        if src.mesh_axis is not dst.mesh_axis:
            raise PlacementError("reduce-scatter must stay on the mesh axis the partial values live on")
        return PlacementTransition.REDUCE_SCATTER
    raise PlacementError(f"no legal transition {src.token()} -> {dst.token()}")


def validate_shard(global_shape: tuple[int, ...], placement: Placement, mesh: MeshSpec) -> tuple[int, ...]:
    """Rank-local shape of a tensor with this placement; sharded extents must divide evenly (ShardDivisible)."""
    if placement.kind is not PlacementKind.SHARDED:
        return tuple(global_shape)
    ax = placement.tensor_axis
    if ax >= len(global_shape):
        raise PlacementError(f"tensor axis {ax} out of range for rank {len(global_shape)}")
    n = mesh.extent(placement.mesh_axis)
    if global_shape[ax] % n:
        raise PlacementError(f"extent {global_shape[ax]} of axis {ax} is not divisible by {n} ranks")
    out = list(global_shape)
    out[ax] //= n
    return tuple(out)


def elementwise_placement(a: Placement, b: Placement) -> Placement:
    """Placement of ``a (op) b`` for an elementwise op (ElementwisePlacement): operands must agree, and
    Partial values only combine under addition-like ops, which the caller asserts by passing Partial twice."""
    if a == b:
        return a
    if a.kind is PlacementKind.REPLICATED and b.kind is PlacementKind.SHARDED:
        return b   # the replicated operand is sliced locally
    if b.kind is PlacementKind.REPLICATED and a.kind is PlacementKind.SHARDED:
        return a
    raise PlacementError(f"elementwise operands placed {a.token()} and {b.token()} do not combine")


def reduce_sharded_axis(p: Placement, reduced_axis: int, reduction: Reduction) -> Placement:
    """Reducing over the axis a tensor is sharded on yields a Partial value (ReduceShardedAxis)."""
    if p.kind is PlacementKind.SHARDED and p.tensor_axis == reduced_axis:
        return Partial(reduction, p.mesh_axis)
    if p.kind is PlacementKind.SHARDED and p.tensor_axis > reduced_axis:
        return Sharded(p.tensor_axis - 1, p.mesh_axis)
    return p


def matmul_placement(a: Placement, b: Placement) -> Placement:
    """Placement of ``x @ w`` for the tensor-parallel Linear patterns:
    column parallel  x Replicated, w Sharded(out) -> y Sharded(last);
    row parallel     x Sharded(last), w Sharded(in) -> y Partial(Sum)."""
    K = PlacementKind
    if a.kind is K.REPLICATED and b.kind is K.REPLICATED:
        return Replicated()
    if a.kind is K.REPLICATED and b.kind is K.SHARDED and b.tensor_axis == 1:
        return Sharded(1, b.mesh_axis)
    if a.kind is K.SHARDED and b.kind is K.SHARDED and b.tensor_axis == 0 and a.mesh_axis is b.mesh_axis:
        return Partial(Reduction.SUM, a.mesh_axis)
    raise PlacementError(f"matmul of {a.token()} and {b.token()} has no distributed rule")


LegalTransition = PlacementTransition      # the reference's name (crates/incin-core/src/dist/placement.rs)
