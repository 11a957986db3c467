"""Run-time counterparts of the reference's proc-macro surface (crates/incin-macros/src/lib.rs:88-341).

The reference does these at compile time in Rust; Python has no compile step, so each is a decorator or a function
that validates when it is applied and fails with the same kind of message:

* :func:`module` — ``#[module]`` (lib.rs:195, module.rs:255-300): turns an annotated class into a module with
  ``parameters()``, the trailing-dot ``state_dict_incin()``, ``named_layers()``, ``train_mode()``, ``to_device()`` and
  ``compute_stats()``.
* :func:`import_model` / :func:`model` — ``model!`` / ``import_model!`` (lib.rs:222-227): a typed module built from
  the tensor table of a ``.safetensors`` or ``.onnx`` file.
* :func:`einsum` — ``einsum!`` (lib.rs:319, einsum.rs): subscript validation, then the contraction.
* :func:`distributed_main` — ``#[distributed_main]`` (distributed_main.rs:5-45): ``--rank`` / ``--world-size``
  parsing and "any failure ends the rank with exit status 1".
* :func:`rank_sweep` / :func:`max_rank` — ``rank_sweep!`` / ``max_rank!`` (lib.rs:227-267): one call per rank up to
  the single rank ceiling.
* :func:`parallel` — ``parallel!`` (parallel_block.rs:33-53): a scoping block that pins a mesh for its body.
* :func:`placement` / :func:`axes` — ``placement!`` / ``axes!``: parsed from the same surface syntax.
"""
from __future__ import annotations

import contextlib
import functools
import inspect
import os
import re
import sys
from pathlib import Path
from typing import Callable, get_type_hints

import torch

from .core.shapes import MAX_RANK


# --------------------------------------------------------------------------------------------------- einsum
class EinsumError(ValueError):
    pass


def validate_einsum(subscript: str, n_operands: int) -> tuple[list[str], str]:
    """The reference's rules (einsum.rs): exactly one ``->``, one comma-separated group per operand, only ``a``-``z``
    as index labels, every output index present on the input side, no index repeated in the output."""
    parts = subscript.split("->")
    if len(parts) != 2:
        raise EinsumError("einsum subscript must contain exactly one '->' separator (e.g. \"ij,jk->ik\")")
    groups, out = parts[0].split(","), parts[1]
    if len(groups) != n_operands:
        raise EinsumError(f"einsum subscript has {len(groups)} input group(s) but {n_operands} operand(s) were provided")
    for ch in subscript:
        if ch in "->,":
            continue
        if not ("a" <= ch <= "z"):
            raise EinsumError(f"einsum subscript character '{ch}' is not a lowercase ASCII letter; only 'a'-'z' are "
                              "allowed as index labels")
    seen = set("".join(groups))
    for ch in out:
        if ch not in seen:
            raise EinsumError(f"einsum output index '{ch}' does not appear in any input subscript")
    if len(set(out)) != len(out):
        raise EinsumError("einsum output subscript repeats an index")
    return groups, out


def einsum(subscript: str, *operands: torch.Tensor) -> torch.Tensor:
    """Validate ``subscript`` against the operands (count, ranks, equal extents of equal labels), then contract.
    Two-operand contractions over bf16 CUDA tensors that are one (batched) matrix product go through the tcgen05 GEMM;
    everything else is evaluated by PyTorch."""
    groups, out = validate_einsum(subscript, len(operands))
    extent: dict[str, int] = {}
    for g, t in zip(groups, operands):
        if len(g) != t.dim():
            raise EinsumError(f"einsum group '{g}' has {len(g)} indices but its operand has rank {t.dim()}")
        for ch, d in zip(g, t.shape):
            if extent.setdefault(ch, int(d)) != int(d):
                raise EinsumError(f"einsum index '{ch}' has extents {extent[ch]} and {int(d)}")
    if len(operands) == 2:
        y = _einsum_as_matmul(groups, out, operands[0], operands[1])
        if y is not None:
            return y
    return torch.einsum(subscript, *operands)


def _einsum_as_matmul(groups, out, a, b):
    """``[batch..] m k , [batch..] k n -> [batch..] m n`` patterns (any order of the groups' letters)."""
    ga, gb = groups
    if len(set(ga)) != len(ga) or len(set(gb)) != len(gb):
        return None
    batch = [c for c in ga if c in gb and c in out]
    contr = [c for c in ga if c in gb and c not in out]
    m = [c for c in ga if c not in gb]
    n = [c for c in gb if c not in ga]
    if not contr or any(c not in out for c in m + n) or set(out) != set(batch + m + n):
        return None
    from .tensor import bmm
    ext = {c: s for g, t in ((ga, a), (gb, b)) for c, s in zip(g, t.shape)}
    size = lambda cs: int(torch.tensor([ext[c] for c in cs]).prod()) if cs else 1   # noqa: E731
    pa = a.permute([ga.index(c) for c in batch + m + contr]).reshape(size(batch), size(m), size(contr))
    pb = b.permute([gb.index(c) for c in batch + contr + n]).reshape(size(batch), size(contr), size(n))
    y = bmm(pa, pb).reshape([ext[c] for c in batch + m + n])
    cur = batch + m + n
    return y.permute([cur.index(c) for c in out])


# --------------------------------------------------------------------------------------------------- distributed_main
def parse_rank_args(argv: list[str]) -> tuple[int, int]:
    """``--rank R`` / ``--world-size W`` anywhere in ``argv`` (unparsable values fall back to 0 / 1, as the reference
    does); the ``INCIN_RANK`` / ``INCIN_WORLD_SIZE`` environment gives the defaults."""
    def _int(text, default):
        try:
            return int(text)
        except (TypeError, ValueError):
            return default
    rank = _int(os.environ.get("INCIN_RANK"), 0)
    world = _int(os.environ.get("INCIN_WORLD_SIZE"), 1)
    for i, a in enumerate(argv):
        if a == "--rank" and i + 1 < len(argv):
            rank = _int(argv[i + 1], 0)
        elif a == "--world-size" and i + 1 < len(argv):
            world = _int(argv[i + 1], 1)
    return rank, world


def distributed_main(fn: Callable | None = None, *, exit_fn: Callable[[int], None] = sys.exit):
    """Decorator for a rank's entry point.  The wrapped function may take ``(rank, world_size)``, ``(rank,)`` or
    nothing.  Whatever it raises is reported as ``[distributed_main] Rank r / w failed`` on stderr and the process
    exits with status 1, so a launcher (and the other ranks' rendezvous timeouts) see a plain failure."""
    def deco(f):
        @functools.wraps(f)
        def wrapper(*args, **kw):
            rank, world = parse_rank_args(sys.argv)
            n = len([p for p in inspect.signature(f).parameters.values()
                     if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD) and p.default is p.empty])
            call = (rank, world)[:max(0, min(2, n - len(args)))]
            try:
                return f(*args, *call, **kw)
            except SystemExit:
                raise
            except BaseException as e:   # noqa: BLE001 - a rank must never leave with a traceback and status 0
                print(f"[distributed_main] Rank {rank} / {world} failed or panicked: {type(e).__name__}: {e}", file=sys.stderr)
                exit_fn(1)
        return wrapper
    return deco(fn) if fn is not None else deco


# --------------------------------------------------------------------------------------------------- rank_sweep
def max_rank() -> int:
    """The single rank ceiling every shape rule is generated up to."""
    return MAX_RANK


_LETTERS = "ABCDEFGHIJKLMNOPQRSTUVWXYZ"


def _sweep_args(form: str, rank: int):
    if form == "names":
        return tuple(f"D{i}" for i in range(rank))
    if form == "names_from1":
        return tuple(f"D{i + 1}" for i in range(rank))
    if form == "ranked_pairs":
        return (rank, *((f"D{i}", i) for i in range(rank)))
    if form == "letters":
        return tuple(_LETTERS[:rank])
    if form == "letters_from_b":
        return tuple(_LETTERS[1:rank + 1])
    if form == "conv1d":
        return (rank + 1, *((f"B{i}", i) for i in range(rank)))
    if form == "conv2d":
        return (rank + 1, rank + 2, *((f"B{i}", i) for i in range(rank)))
    raise ValueError(f"unknown rank_sweep form '{form}'")


def rank_sweep(form: str, fn: Callable, *, min: int = 1, max: int | None = None) -> list:   # noqa: A002
    """Call ``fn(*arguments_for_rank)`` once per rank in ``min..=max`` (default ``1..=MAX_RANK``) and return the
    results.  ``max`` above the ceiling is rejected rather than honoured: no rule sets its own ceiling."""
    hi = MAX_RANK if max is None else max
    if hi > MAX_RANK:
        raise ValueError(f"rank_sweep max = {hi} exceeds MAX_RANK = {MAX_RANK}")
    if min < 0 or min > hi:
        raise ValueError(f"rank_sweep range {min}..={hi} is empty")
    return [fn(*_sweep_args(form, r)) for r in range(min, hi + 1)]


# --------------------------------------------------------------------------------------------------- parallel / placement / axes
_mesh_stack: list = []


@contextlib.contextmanager
def parallel(mesh=None):
    """``with parallel(mesh): ...`` — the body runs with ``mesh`` as the current mesh (:func:`current_mesh`)."""
    _mesh_stack.append(mesh)
    try:
        yield mesh
    finally:
        _mesh_stack.pop()


def current_mesh():
    return _mesh_stack[-1] if _mesh_stack else None


def placement(text: str, mesh=None):
    """``placement("Sharded(0) on M")``, ``"Replicated on M"``, ``"Partial(Sum) on M"``, ``"PipelineStage(1) on M"``,
    ``"Local"``: the reference's ``placement![...]`` syntax.  ``mesh`` (or the current ``parallel`` mesh) resolves the
    name after ``on``; a placement other than ``Local`` without a mesh is an error."""
    from .parallel.placement import (Partial, PipelineStage, Placement, PlacementKind, Reduction, Replicated, Sharded)
    m = re.fullmatch(r"\s*(\w+)\s*(?:\(\s*(\w+)\s*\))?\s*(?:on\s+(\w+))?\s*", text)
    if not m:
        raise ValueError(f"cannot parse placement '{text}'")
    kind, arg, on = m.groups()
    if kind == "Local":
        if arg or on:
            raise ValueError("Local takes no argument and no mesh")
        return Placement(PlacementKind.LOCAL)
    if on is None:
        raise ValueError(f"placement '{kind}' needs 'on <Mesh>'")
    mesh = mesh if mesh is not None else current_mesh()
    if kind == "Replicated":
        return Replicated()
    if kind == "Sharded":
        return Sharded(int(arg))
    if kind == "Partial":
        return Partial(Reduction((arg or "sum").lower()))
    if kind == "PipelineStage":
        return PipelineStage(int(arg))
    raise ValueError(f"unknown placement kind '{kind}'")


def axes(*names: str):
    """``axes("Batch", "Channels", "Height", "Width")``: a tuple of named axes (``core.shapes.dim`` tags)."""
    from .core.shapes import dim
    if len(set(names)) != len(names):
        raise ValueError("axis names must be distinct")
    return tuple(dim(n) for n in names)


# --------------------------------------------------------------------------------------------------- #[module]
def module(cls=None):
    """Class decorator: every annotated field whose value is a ``torch.nn.Module`` or a tensor parameter becomes a
    registered child, in declaration order; the class gains the derived surface of the reference's ``#[module]``."""
    def deco(c):
        hints = list(getattr(c, "__annotations__", {}))
        user_init = c.__dict__.get("__init__")
        forward = c.__dict__.get("forward")

        def __init__(self, *args, **kw):
            torch.nn.Module.__init__(self)
            if user_init is not None:
                user_init(self, *args, **kw)
            else:
                if len(args) > len(hints):
                    raise TypeError(f"{c.__name__} takes {len(hints)} fields")
                vals = dict(zip(hints, args))
                vals.update(kw)
                missing = [h for h in hints if h not in vals]
                if missing:
                    raise TypeError(f"{c.__name__} is missing fields {missing}")
                for h in hints:
                    setattr(self, h, vals[h])

        def named_layers(self):
            return [(n, m) for n, m in self.named_children()]

        def state_dict_incin(self):
            from .io.checkpoint import state_dict
            return state_dict(self)

        def train_mode(self, on: bool = True):
            return self.train(on)

        def to_device(self, device):
            return self.to(device)

        def compute_stats(self):
            from .nn.layers import ComputeStats
            return ComputeStats.of(self)

        ns = {k: v for k, v in c.__dict__.items() if k not in ("__dict__", "__weakref__", "__init__")}
        ns.update(__init__=__init__, named_layers=named_layers, state_dict_incin=state_dict_incin, train_mode=train_mode,
                  to_device=to_device, compute_stats=compute_stats, __module_fields__=tuple(hints))
        if forward is None:
            def _forward(self, x):
                for n in hints:
                    v = getattr(self, n)
                    if isinstance(v, torch.nn.Module):
                        x = v(x)
                return x
            ns["forward"] = _forward
        return type(c.__name__, (torch.nn.Module,), ns)
    return deco(cls) if cls is not None else deco


# --------------------------------------------------------------------------------------------------- model! / import_model!
def _tensor_table(path: Path) -> dict[str, tuple[tuple[int, ...], torch.Tensor | None]]:
    if path.suffix == ".safetensors":
        from .io.safetensors import load_safetensors
        return {k: (tuple(v.shape), v) for k, v in load_safetensors(path).items()}
    if path.suffix == ".onnx":
        from .io.onnx import import_model as read_onnx
        return {k: (tuple(v.shape), v) for k, v in read_onnx(path).initializers.items()}
    raise ValueError(f"import_model reads .safetensors and .onnx files, not '{path.suffix}'")


def import_model(path, name: str = "ImportedModel"):
    """Build a module class from a model file and return an instance with the file's weights.

    The tensor table is grouped by prefix: ``<p>.weight`` of rank 2 (+ optional ``<p>.bias``) becomes a ``Linear`` of
    that shape, rank-1 ``weight`` + ``bias`` a ``LayerNorm``, rank-1 ``weight`` alone an ``RMSNorm``, a lone rank-2
    ``<p>.embedding`` / ``wte`` / ``wpe`` table an ``Embedding``; anything else is kept as a plain parameter.  Field
    names are the prefixes with dots replaced by underscores; ``layers()`` lists (field, kind, shape) in file order."""
    from . import nn
    path = Path(path)
    table = _tensor_table(path)
    groups: dict[str, dict[str, tuple]] = {}
    for key, (shape, t) in table.items():
        k = key[:-1] if key.endswith(".") else key
        prefix, _, leaf = k.rpartition(".")
        groups.setdefault(prefix, {})[leaf] = (shape, t)
    fields: list[tuple[str, str, tuple, torch.nn.Module | torch.nn.Parameter]] = []
    for prefix, leaves in groups.items():
        field = re.sub(r"\W", "_", prefix) or "root"
        if field[0].isdigit():
            field = "l" + field
        w = leaves.get("weight")
        if w is not None and len(w[0]) == 2 and set(leaves) <= {"weight", "bias"}:
            out_f, in_f = w[0]
            if "bias" not in leaves and ("emb" in prefix or prefix.split(".")[-1] in ("wte", "wpe")):
                layer = nn.Embedding(out_f, in_f)
                kind = "Embedding"
            else:
                layer = nn.Linear(in_f, out_f, bias="bias" in leaves)
                kind = "Linear"
        elif w is not None and len(w[0]) == 1 and set(leaves) <= {"weight", "bias"}:
            layer = nn.LayerNorm(w[0][0]) if "bias" in leaves else nn.RMSNorm(w[0][0])
            kind = "LayerNorm" if "bias" in leaves else "RMSNorm"
        else:
            for leaf, (shape, t) in leaves.items():
                p = torch.nn.Parameter(t.clone().float() if t is not None and t.is_floating_point()
                                       else torch.zeros(shape), requires_grad=t is None or t.is_floating_point())
                fields.append((f"{field}_{leaf}" if prefix else leaf, "Param", shape, p))
            continue
        with torch.no_grad():
            for leaf, (shape, t) in leaves.items():
                if t is not None:
                    getattr(layer, leaf).copy_(t.to(getattr(layer, leaf).dtype))
        fields.append((field, kind, w[0], layer))

    class _Imported(torch.nn.Module):
        def __init__(self):
            super().__init__()
            for f, _, _, obj in fields:
                if isinstance(obj, torch.nn.Parameter):
                    self.register_parameter(f, obj)
                else:
                    self.add_module(f, obj)

        @staticmethod
        def layers():
            return [(f, kind, shape) for f, kind, shape, _ in fields]

    _Imported.__name__ = _Imported.__qualname__ = name
    return _Imported()


model = import_model
