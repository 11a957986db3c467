"""Readable shape errors.

Counterpart of crates/incin-diagnostics (a humaniser that turns the compiler's type-level shape errors into
sentences, with one parser per operation) and of the editor/LSP glue that shows them inline.  Shapes are run-time
values here, so the same job is done on exceptions: :func:`explain` recognises the mismatch messages of PyTorch and
of this package's own ops and says which operand, which axis, and what would fix it; :func:`humanize` is a context
manager / decorator that re-raises with the explanation attached.
"""
from __future__ import annotations

import contextlib
import re
from dataclasses import dataclass


@dataclass
class Diagnosis:
    op: str
    summary: str
    hint: str

    def __str__(self) -> str:
        return f"[{self.op}] {self.summary}\n  hint: {self.hint}"


_MATMUL = re.compile(r"mat1 and mat2 shapes cannot be multiplied \((\d+)x(\d+) and (\d+)x(\d+)\)")
_BROADCAST = re.compile(r"The size of tensor a \((\d+)\) must match the size of tensor b \((\d+)\) at non-singleton dimension (\d+)")
_RESHAPE = re.compile(r"shape '\[([-\d, ]+)\]' is invalid for input of size (\d+)")
_CAT = re.compile(r"Sizes of tensors must match except in dimension (\d+)\. Expected size (\d+) but got size (\d+) for tensor number (\d+)")
_CONV = re.compile(r"expected input\[([\d, ]+)\] to have (\d+) channels, but got (\d+) channels")
_TP = re.compile(r"shard \[(\d+), (\d+)\] does not fit the tensor-parallel buffers \[(\d+), (\d+)\]")
_TMA = re.compile(r"misaligned operand")
_INDEX = re.compile(r"index (-?\d+) is out of bounds for dimension (\d+) with size (\d+)")
_STACK = re.compile(r"stack expects each tensor to be equal size, but got \[([\d, ]*)\] at entry (\d+) and \[([\d, ]*)\] at entry (\d+)")
_DIM_RANGE = re.compile(r"Dimension out of range \(expected to be in range of \[(-?\d+), (-?\d+)\], but got (-?\d+)\)")
_NARROW = re.compile(r"start \((-?\d+)\) \+ length \((-?\d+)\) exceeds dimension size \((\d+)\)")
_POOL = re.compile(r"Given input size: \(([\dx]+)\)\. Calculated output size: \(([\dx]+)\)\. Output size is too small")
_KERNEL = re.compile(r"Calculated padded input size per channel: \(([\d x]+)\)\. Kernel size: \(([\d x]+)\)\. Kernel size can't be greater")

# one sentence per operation family: what the shapes have to satisfy
RULES = {
    "matmul": "[M, K] times [K, N] gives [M, N]: the inner extents K must be equal (leading batch axes broadcast).",
    "broadcast": "Aligned from the last axis, two extents must be equal or one of them must be 1.",
    "reshape": "The number of elements (product of the extents) must be the same before and after; one axis may be -1.",
    "concat": "Every axis except the concatenation axis must have the same extent in all inputs.",
    "stack": "All inputs of a stack must have exactly the same shape; the new axis has one entry per input.",
    "conv2d": "Input is [N, C, H, W], weight [O, C / groups, kH, kW]: C must agree and the padded H, W must cover the kernel.",
    "pool2d": "The (padded) spatial extents H, W must be at least the kernel extents, or the output would be empty.",
    "index": "Indices count from 0; -k addresses the k-th entry from the end; both must stay inside the axis.",
    "slice": "start + length of a slice must not exceed the extent of the axis it is taken from.",
    "axis": "An axis argument of a rank-r tensor must lie in [-r, r - 1] (transpose, reductions, flatten, softmax ...).",
    "tensor-parallel": "Rows per rank are a multiple of 128 and fit max_rows_per_rank; sharded widths fit max_cols.",
    "gemm": "TMA moves 16-byte units: bf16 row strides and offsets are multiples of 8 elements (4 for fp32).",
}


def explain(message: str) -> Diagnosis | None:
    m = _MATMUL.search(message)
    if m:
        a0, a1, b0, b1 = map(int, m.groups())
        hint = (f"the right operand looks transposed: use its transpose ({b1}x{b0})" if a1 == b1 else
                f"inner dimensions must agree: {a1} (left columns) vs {b0} (right rows)")
        return Diagnosis("matmul", f"cannot multiply [{a0}, {a1}] by [{b0}, {b1}]: {a1} != {b0}", hint)
    m = _BROADCAST.search(message)
    if m:
        a, b, dim = map(int, m.groups())
        return Diagnosis("broadcast", f"axis {dim} has extent {a} on the left and {b} on the right; neither is 1",
                         "extents must be equal or 1 to broadcast: reshape / unsqueeze the smaller operand, or reduce the larger")
    m = _RESHAPE.search(message)
    if m:
        dims = [int(x) for x in m.group(1).split(",")]
        n = int(m.group(2))
        known = 1
        for d in dims:
            if d != -1:
                known *= d
        if -1 in dims:
            hint = f"{n} elements are not divisible by the known extents ({known})"
        else:
            hint = f"the target holds {known} elements, the input {n}; use -1 for one axis to have it inferred"
        return Diagnosis("reshape", f"cannot view {n} elements as {dims}", hint)
    m = _CAT.search(message)
    if m:
        dim, want, got, idx = map(int, m.groups())
        return Diagnosis("concat", f"tensor #{idx} has extent {got} where the others have {want}",
                         f"all axes except the concatenation axis {dim} must match")
    m = _CONV.search(message)
    if m:
        return Diagnosis("conv2d", f"input has {m.group(3)} channels, the weight expects {m.group(2)}",
                         "input layout is [N, C, H, W]; check in_channels of the layer (or a missing permute from NHWC)")
    m = _TP.search(message)
    if m:
        r, c, R, C = map(int, m.groups())
        return Diagnosis("tensor-parallel", f"a [{r}, {c}] shard was given to buffers sized [{R}, {C}]",
                         "construct TensorParallel with max_rows_per_rank >= tokens / tp and max_cols >= the widest sharded activation; "
                         "rows per rank must be a multiple of 128")
    if _TMA.search(message):
        return Diagnosis("gemm", "an operand is not 16-byte aligned",
                         "bf16 row strides and offsets must be multiples of 8 elements (TMA moves 16-byte units): pad the inner dimension")
    m = _INDEX.search(message)
    if m:
        i, dim, size = map(int, m.groups())
        return Diagnosis("index", f"index {i} on axis {dim} of extent {size}", f"valid indices are {-size}..{size - 1}")
    m = _STACK.search(message)
    if m:
        a, ia, b, ib = m.group(1), int(m.group(2)), m.group(3), int(m.group(4))
        return Diagnosis("stack", f"input #{ia} is [{a}] but input #{ib} is [{b}]",
                         "stack needs identical shapes; to join along an existing axis use concat instead")
    m = _DIM_RANGE.search(message)
    if m:
        lo, hi, got = map(int, m.groups())
        return Diagnosis("axis", f"axis {got} was given to a rank-{hi + 1} tensor",
                         f"valid axes are {lo}..{hi}; a missing batch axis (unsqueeze) is the usual cause")
    m = _NARROW.search(message)
    if m:
        start, length, size = map(int, m.groups())
        return Diagnosis("slice", f"[{start}, {start + length}) reaches past the axis of extent {size}",
                         f"the longest slice starting at {start} has length {max(size - start, 0)}")
    m = _POOL.search(message)
    if m:
        return Diagnosis("pool2d", f"an input of {m.group(1)} would give an output of {m.group(2)}",
                         "the window is larger than the (padded) input: lower kernel_size / stride or add padding")
    m = _KERNEL.search(message)
    if m:
        return Diagnosis("conv2d", f"the kernel ({m.group(2).strip()}) does not fit the padded input ({m.group(1).strip()})",
                         "raise padding, shrink the kernel, or check that H and W were not swapped with the channel axis")
    return None


def translate(message: str, *, with_rule: bool = False) -> str:
    """The text the ``translate`` command prints for a pasted error message: the message itself, the diagnosis
    underneath when one of the parsers recognises it, and (``with_rule``) the rule of that operation family."""
    d = explain(message)
    if d is None:
        return message.rstrip()
    out = [message.rstrip(), str(d)]
    if with_rule and d.op in RULES:
        out.append(f"  rule: {RULES[d.op]}")
    return "\n".join(out)


@contextlib.contextmanager
def humanize():
    """``with humanize(): ...`` re-raises shape errors with a plain-language explanation appended."""
    try:
        yield
    except (RuntimeError, ValueError, IndexError) as e:
        d = explain(str(e))
        if d is None:
            raise
        raise type(e)(f"{e}\n{d}") from e
