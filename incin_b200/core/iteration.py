"""Iteration plans for pointwise kernels: how a launch walks its operands.

Counterpart of crates/incin-backends/src/iteration.rs (``IterationPlan`` / ``UnaryIterationPlan`` / ``OperandLayout``,
broadcast-stride normalisation, the ``max_physical_index`` bounds proof and the ``LayoutClass`` classification that
selects a kernel specialisation).  The plan is computed once on the host from tensor metadata; the fused pointwise
kernels (:mod:`incin_b200.codegen`) and the strided copy receive the collapsed geometry, so the device code never
sees more dimensions or indirection than the data needs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

from .spec import LayoutClass, TensorMeta


class IterationError(ValueError):
    pass


@dataclass(frozen=True)
class OperandLayout:
    strides: tuple[int, ...]      # in elements, aligned to the plan's (collapsed) shape; 0 = broadcast
    offset: int
    layout: LayoutClass

    def max_physical_index(self, shape: Sequence[int]) -> int:
        """Largest element index the walk touches: the bounds proof the launcher checks against the allocation."""
        return self.offset + sum((d - 1) * s for d, s in zip(shape, self.strides) if d > 0)


@dataclass(frozen=True)
class IterationPlan:
    shape: tuple[int, ...]                  # collapsed iteration space
    operands: tuple[OperandLayout, ...]     # inputs first, output last
    numel: int

    @property
    def layout(self) -> LayoutClass:
        """The specialisation one kernel serves every operand with."""
        kinds = {o.layout for o in self.operands}
        if kinds <= {LayoutClass.CONTIGUOUS}:
            return LayoutClass.CONTIGUOUS
        if kinds <= {LayoutClass.CONTIGUOUS, LayoutClass.SCALAR}:
            return LayoutClass.SCALAR
        if LayoutClass.STRIDED in kinds:
            return LayoutClass.STRIDED
        return LayoutClass.BROADCAST


def _broadcast_strides(meta: TensorMeta, shape: Sequence[int]) -> list[int]:
    """Right-align ``meta`` to ``shape``; size-1 and missing axes get stride 0."""
    pad = len(shape) - len(meta.shape)
    if pad < 0:
        raise IterationError(f"operand of rank {len(meta.shape)} cannot broadcast to rank {len(shape)}")
    out = [0] * pad
    for d, s, target in zip(meta.shape, meta.strides, shape[pad:]):
        if d == target:
            out.append(s if d != 1 else 0)
        elif d == 1:
            out.append(0)
        else:
            raise IterationError(f"axis of extent {d} cannot broadcast to {target}")
    return out


def _classify(shape: Sequence[int], strides: Sequence[int]) -> LayoutClass:
    if all(d == 1 or s == 0 for d, s in zip(shape, strides)):
        return LayoutClass.SCALAR
    expect = 1
    dense = True
    for d, s in zip(reversed(shape), reversed(strides)):
        if d != 1 and s != expect:
            dense = False
        expect *= d
    if dense:
        return LayoutClass.CONTIGUOUS
    return LayoutClass.BROADCAST if any(s == 0 and d != 1 for d, s in zip(shape, strides)) else LayoutClass.STRIDED


def plan(inputs: Sequence[TensorMeta], output: TensorMeta) -> IterationPlan:
    """Normalise strides to the output shape, drop size-1 axes and merge axes that are contiguous in EVERY operand."""
    shape = list(output.shape)
    all_strides = [_broadcast_strides(m, shape) for m in inputs] + [list(output.strides)]
    # drop extent-1 axes
    keep = [i for i, d in enumerate(shape) if d != 1] or ([len(shape) - 1] if shape else [])
    shape = [shape[i] for i in keep]
    all_strides = [[st[i] for i in keep] for st in all_strides]
    # merge axis i into i+1 when stride[i] == stride[i+1] * shape[i+1] for every operand
    i = len(shape) - 2
    while i >= 0:
        if all(st[i] == st[i + 1] * shape[i + 1] for st in all_strides):
            shape[i + 1] *= shape[i]
            del shape[i]
            for st in all_strides:
                del st[i]
        i -= 1
    metas = list(inputs) + [output]
    operands = tuple(OperandLayout(tuple(st), m.offset, _classify(shape, st)) for st, m in zip(all_strides, metas))
    numel = 1
    for d in shape:
        numel *= d
    if any(s == 0 for s in all_strides[-1]) and numel > 1:
        raise IterationError("the output of a pointwise op cannot be a broadcast view")
    return IterationPlan(tuple(shape), operands, numel)


@dataclass(frozen=True)
class UnaryIterationPlan(IterationPlan):
    """The plan of a one-input elementwise op (what :func:`unary_plan` returns)."""

    @property
    def input(self) -> "OperandLayout":
        return self.operands[0]


def unary_plan(x: TensorMeta, out: TensorMeta) -> IterationPlan:
    if tuple(x.shape) != tuple(out.shape):
        raise IterationError("a unary op keeps the shape")
    p = plan([x], out)
    return UnaryIterationPlan(p.shape, p.operands, p.numel)


def check_bounds(p: IterationPlan, allocation_elems: Sequence[int]) -> None:
    """Raise unless every operand's walk stays inside its allocation (lengths in elements, inputs first)."""
    for o, n in zip(p.operands, allocation_elems):
        if p.numel and o.max_physical_index(p.shape) >= n:
            raise IterationError(f"walk reaches element {o.max_physical_index(p.shape)} of an allocation of {n}")
