"""Shapes: static, dynamic and named dimensions, broadcast / reshape rules, and ``idx`` slicing.

The reference proves shapes at compile time with typenum (``s![2,3]``, ``s![dyn,784]``, ``dim!(Batch)``,
``idx![0..5, .., 15..30]``; crates/incin-core/src/shapes/*.rs).  Python has no compile time, so the same
rules are checked eagerly when a :class:`Shape` is bound to a tensor or combined with another shape, and
failures raise :class:`ShapeError` naming the operation, exactly like ``ShapeError``/``OperationKind``
there (shapes/error.rs).  A named dimension (``dim("Batch")``) is a runtime-sized axis whose *identity*
is checked: two tensors that share ``Batch`` must agree on its extent, and a ``Batch`` axis never unifies
with a ``Seq`` axis even when the extents match.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Iterable, Sequence

MAX_RANK = 8


class OperationKind(enum.Enum):
    BROADCAST = "broadcast"
    MATMUL = "matmul"
    RESHAPE = "reshape"
    SLICE = "slice"
    CONCAT = "concat"
    STACK = "stack"
    BIND = "bind"
    CONV = "conv"
    POOL = "pool"
    REDUCE = "reduce"


class ShapeError(ValueError):
    def __init__(self, op: OperationKind, message: str):
        super().__init__(f"{op.value}: {message}")
        self.op = op


@dataclass(frozen=True)
class Dim:
    """A dimension with a fixed extent."""
    size: int

    def __post_init__(self):
        if self.size < 0:
            raise ValueError("negative dimension")

    def resolve(self, actual: int, env: dict) -> int:
        if actual != self.size:
            raise ShapeError(OperationKind.BIND, f"expected extent {self.size}, got {actual}")
        return actual

    def __str__(self) -> str:
        return str(self.size)


@dataclass(frozen=True)
class DynDim:
    """An anonymous runtime-sized dimension (``dyn``)."""

    def resolve(self, actual: int, env: dict) -> int:
        return actual

    def __str__(self) -> str:
        return "dyn"


@dataclass(frozen=True)
class NamedDim:
    """A runtime-sized dimension with an identity (``dim("Batch")``)."""
    name: str

    def resolve(self, actual: int, env: dict) -> int:
        seen = env.setdefault(self.name, actual)
        if seen != actual:
            raise ShapeError(OperationKind.BIND, f"axis {self.name} bound to {seen} and {actual}")
        return actual

    def __str__(self) -> str:
        return self.name


def dim(*names: str):
    """``Batch, Seq = dim("Batch", "Seq")`` — named runtime-sized axes."""
    out = tuple(NamedDim(n) for n in names)
    return out[0] if len(out) == 1 else out


DYN = DynDim()


class Shape:
    """An ordered list of dimensions; ``s(2, 3)``, ``s("dyn", 784)``, ``s(Batch, Seq, 768)``."""

    def __init__(self, dims: Iterable):
        ds = []
        for d in dims:
            if isinstance(d, (Dim, DynDim, NamedDim)):
                ds.append(d)
            elif isinstance(d, int):
                ds.append(Dim(d))
            elif d in ("dyn", None, -1):
                ds.append(DYN)
            elif isinstance(d, str):
                ds.append(NamedDim(d))
            else:
                raise TypeError(f"not a dimension: {d!r}")
        if len(ds) > MAX_RANK:
            raise ShapeError(OperationKind.BIND, f"rank {len(ds)} exceeds MAX_RANK={MAX_RANK}")
        self.dims = tuple(ds)

    @property
    def rank(self) -> int:
        return len(self.dims)

    @property
    def is_static(self) -> bool:
        return all(isinstance(d, Dim) for d in self.dims)

    def numel(self) -> int:
        if not self.is_static:
            raise ShapeError(OperationKind.BIND, "numel of a shape with runtime dimensions")
        n = 1
        for d in self.dims:
            n *= d.size
        return n

    def bind(self, actual: Sequence[int], env: dict | None = None) -> tuple[int, ...]:
        """Check a concrete size tuple against this shape; named axes are unified through ``env``."""
        env = {} if env is None else env
        if len(actual) != self.rank:
            raise ShapeError(OperationKind.BIND, f"expected rank {self.rank} ({self}), got {tuple(actual)}")
        return tuple(d.resolve(int(a), env) for d, a in zip(self.dims, actual))

    def check(self, tensor, env: dict | None = None):
        self.bind(tuple(tensor.shape), env)
        return tensor

    def __iter__(self):
        return iter(self.dims)

    def __eq__(self, other) -> bool:
        return isinstance(other, Shape) and self.dims == other.dims

    def __hash__(self) -> int:
        return hash(self.dims)

    def __repr__(self) -> str:
        return "s[" + ", ".join(map(str, self.dims)) + "]"


def s(*dims) -> Shape:
    return Shape(dims)


def _unify(a, b, op: OperationKind):
    """Broadcast-unify two dimensions."""
    if isinstance(a, Dim) and isinstance(b, Dim):
        if a.size == b.size or b.size == 1:
            return a
        if a.size == 1:
            return b
        raise ShapeError(op, f"extents {a.size} and {b.size} do not broadcast")
    if isinstance(a, NamedDim) and isinstance(b, NamedDim):
        if a.name != b.name:
            raise ShapeError(op, f"named axes {a.name} and {b.name} never unify")
        return a
    if isinstance(a, Dim) and a.size == 1:
        return b
    if isinstance(b, Dim) and b.size == 1:
        return a
    if isinstance(a, NamedDim) or isinstance(b, NamedDim):
        named, other = (a, b) if isinstance(a, NamedDim) else (b, a)
        if isinstance(other, DynDim):
            return named
        raise ShapeError(op, f"named axis {named.name} cannot unify with fixed extent {other}")
    return a if isinstance(a, Dim) else b  # dyn with dyn / dyn with fixed: checked at bind time


def broadcast_shapes(a: Shape | Sequence[int], b: Shape | Sequence[int]) -> Shape:
    """NumPy-style right-aligned broadcasting over symbolic shapes (shapes/broadcast.rs)."""
    a = a if isinstance(a, Shape) else Shape(a)
    b = b if isinstance(b, Shape) else Shape(b)
    out = []
    for i in range(1, max(a.rank, b.rank) + 1):
        da = a.dims[-i] if i <= a.rank else Dim(1)
        db = b.dims[-i] if i <= b.rank else Dim(1)
        out.append(_unify(da, db, OperationKind.BROADCAST))
    return Shape(reversed(out))


def matmul_shape(a: Shape | Sequence[int], b: Shape | Sequence[int]) -> Shape:
    a = a if isinstance(a, Shape) else Shape(a)
    b = b if isinstance(b, Shape) else Shape(b)
    if a.rank < 2 or b.rank < 2:
        raise ShapeError(OperationKind.MATMUL, "operands need rank >= 2")
    ka, kb = a.dims[-1], b.dims[-2]
    if isinstance(ka, Dim) and isinstance(kb, Dim) and ka.size != kb.size:
        raise ShapeError(OperationKind.MATMUL, f"inner extents {ka.size} and {kb.size} differ")
    if isinstance(ka, NamedDim) and isinstance(kb, NamedDim) and ka.name != kb.name:
        raise ShapeError(OperationKind.MATMUL, f"inner axes {ka.name} and {kb.name} differ")
    batch = broadcast_shapes(Shape(a.dims[:-2]), Shape(b.dims[:-2])) if (a.rank > 2 or b.rank > 2) else Shape(())
    return Shape(batch.dims + (a.dims[-2], b.dims[-1]))


def reshape_infer(numel: int, target: Sequence[int]) -> tuple[int, ...]:
    """Resolve one ``-1`` (InferDim) in a reshape target (shapes/reshape.rs)."""
    unknown = [i for i, d in enumerate(target) if d == -1]
    if len(unknown) > 1:
        raise ShapeError(OperationKind.RESHAPE, "at most one dimension can be inferred")
    known = 1
    for d in target:
        if d != -1:
            if d < 0:
                raise ShapeError(OperationKind.RESHAPE, f"invalid extent {d}")
            known *= d
    if unknown:
        if known == 0 or numel % known:
            raise ShapeError(OperationKind.RESHAPE, f"cannot infer a dimension: {numel} is not divisible by {known}")
        out = list(target)
        out[unknown[0]] = numel // known
        return tuple(out)
    if known != numel:
        raise ShapeError(OperationKind.RESHAPE, f"{numel} elements cannot be viewed as {tuple(target)}")
    return tuple(target)


def conv2d_out(h: int, w: int, kernel, stride=(1, 1), padding=(0, 0), dilation=(1, 1)) -> tuple[int, int]:
    """Spatial output size of a convolution / pooling window (shapes/spatial.rs)."""
    out = []
    for n, k, st, p, d in zip((h, w), kernel, stride, padding, dilation):
        eff = d * (k - 1) + 1
        if n + 2 * p < eff:
            raise ShapeError(OperationKind.CONV, f"window {eff} larger than padded input {n + 2 * p}")
        out.append((n + 2 * p - eff) // st + 1)
    return out[0], out[1]


class _Idx:
    """``idx[0:5, ..., 15:30]`` — validated slicing; ``-1`` as a whole-axis marker is written ``:``."""

    def __getitem__(self, item):
        items = item if isinstance(item, tuple) else (item,)
        items = tuple(i.to_python() if hasattr(i, "to_python") else i for i in items)      # Slice objects
        if sum(1 for i in items if i is Ellipsis) > 1:
            raise ShapeError(OperationKind.SLICE, "only one ellipsis is allowed")
        return IndexSpec(items)


@dataclass(frozen=True)
class IndexSpec:
    items: tuple

    def apply(self, tensor):
        """Slice with bounds checking (Python would silently clamp an out-of-range slice)."""
        shape = tuple(tensor.shape)
        n_explicit = sum(1 for i in self.items if i is not Ellipsis)
        if n_explicit > len(shape):
            raise ShapeError(OperationKind.SLICE, f"{n_explicit} indices for rank {len(shape)}")
        axis = 0
        for it in self.items:
            if it is Ellipsis:
                axis = len(shape) - (n_explicit - sum(1 for j in self.items[: self.items.index(it)] if j is not Ellipsis))
                continue
            ext = shape[axis]
            if isinstance(it, slice):
                start = 0 if it.start is None else it.start
                stop = ext if it.stop is None else it.stop
                if start < 0 or stop > ext or start > stop:
                    raise ShapeError(OperationKind.SLICE, f"range {start}..{stop} out of bounds for axis {axis} ({ext})")
            elif isinstance(it, int):
                if not -ext <= it < ext:
                    raise ShapeError(OperationKind.SLICE, f"index {it} out of bounds for axis {axis} ({ext})")
            axis += 1
        return tensor[self.items]

    def out_shape(self, shape: Sequence[int]) -> tuple[int, ...]:
        import torch
        return tuple(self.apply(torch.empty(tuple(shape), device="meta")).shape)


idx = _Idx()


# ---- the reference's typed index / shape-rule vocabulary as run-time objects (shapes/idx.rs, broadcast.rs, reshape.rs)
@dataclass(frozen=True)
class Slice:
    """``start..end`` (optionally stepped) along one axis; ``idx[...]`` accepts it next to Python slices."""
    start: int | None = None
    end: int | None = None
    step: int = 1

    def to_python(self):
        return slice(self.start, self.end, self.step if self.step != 1 else None)


class _InferDim:
    """The ``-1`` of a reshape target: the extent that the element count determines."""

    def __index__(self):
        return -1

    def __repr__(self):
        return "InferDim"


InferDim = _InferDim()
EllipsisDim = Ellipsis      # the reference's ``Ellipsis`` index: every axis not named otherwise


@dataclass(frozen=True)
class BroadcastShape:
    """Two operand shapes and the shape their elementwise result has (ShapeError when they do not broadcast)."""
    lhs: tuple
    rhs: tuple

    @property
    def result(self) -> Shape:
        return broadcast_shapes(self.lhs, self.rhs)


@dataclass(frozen=True)
class ReshapeShape:
    """A source shape viewed as ``target`` (one extent may be ``InferDim`` / ``-1``)."""
    source: tuple
    target: tuple

    @property
    def result(self) -> tuple[int, ...]:
        numel = 1
        for d in self.source:
            numel *= int(d)
        return reshape_infer(numel, [int(d.__index__()) if hasattr(d, "__index__") else int(d) for d in self.target])

