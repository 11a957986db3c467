"""Graph IR, op tracing and the compiled-graph layer.

Counterparts: crates/incin-core/src/graph.rs (``Graph`` / ``OpType``), tensor/tracing.rs (``TracingBackend``
records every op into a process-wide graph; ``extract_graph`` / ``tracing_graph_snapshot``) and
crates/incin-core/src/compiled (``CapturedGraph::capture``, ``FusionPass``, ``ShapeBucket``, ``CompiledPlan`` +
``ShapeGuard``, ``AllocationPlanner`` / ``LivenessMap`` / ``MemoryPlan``, ``CompiledArtifact`` with an Adler-32
header, ``ReproducibilityManifest``).

Tracing here hooks PyTorch's dispatcher (``TorchDispatchMode``) instead of wrapping a backend type, so any model
code is traceable unchanged.  The fusion pass groups maximal chains of pointwise ops (the reference fuses adjacent
pairs) and lowers each chain to one kernel of :mod:`incin_b200.codegen`.  The execution-side counterpart of a
compiled plan is the CUDA-graph capture in :class:`incin_b200.engine.TrainStep`; ``CompiledPlan`` carries the shape
guard that decides whether a captured graph may be replayed for a new input.
"""
from __future__ import annotations

import hashlib
import json
import struct
import zlib
from dataclasses import asdict, dataclass, field

import torch
from torch.utils._python_dispatch import TorchDispatchMode

POINTWISE = {"add", "sub", "mul", "div", "relu", "gelu", "silu", "sigmoid", "tanh", "exp", "log", "sqrt", "neg", "abs",
             "rsqrt", "clamp", "pow", "maximum", "minimum", "where", "mish", "elu", "softplus", "sign", "reciprocal"}


@dataclass
class Node:
    id: int
    op: str
    inputs: list[int]
    shape: tuple[int, ...]
    dtype: str
    attrs: dict = field(default_factory=dict)


class Graph:
    def __init__(self):
        self.nodes: list[Node] = []
        self.inputs: list[int] = []
        self.outputs: list[int] = []

    def add(self, op: str, inputs, shape, dtype: str, **attrs) -> int:
        nid = len(self.nodes)
        self.nodes.append(Node(nid, op, list(inputs), tuple(shape), dtype, attrs))
        return nid

    def to_list(self) -> list[dict]:
        return [asdict(n) for n in self.nodes]

    def digest(self) -> str:
        return hashlib.sha256(json.dumps(self.to_list(), sort_keys=True, default=str).encode()).hexdigest()

    def consumers(self) -> dict[int, list[int]]:
        out: dict[int, list[int]] = {n.id: [] for n in self.nodes}
        for n in self.nodes:
            for i in n.inputs:
                out[i].append(n.id)
        return out


class _Tracer(TorchDispatchMode):
    def __init__(self, graph: Graph):
        super().__init__()
        self.g = graph
        self.ids: dict[int, int] = {}

    def _id(self, t: torch.Tensor) -> int:
        key = id(t)
        if key not in self.ids:
            self.ids[key] = self.g.add("input", [], t.shape, str(t.dtype).replace("torch.", ""))
            self.g.inputs.append(self.ids[key])
        return self.ids[key]

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        out = func(*args, **(kwargs or {}))
        name = func.__name__.split(".")[0].rstrip("_")
        ins = [self._id(a) for a in args if isinstance(a, torch.Tensor)]
        for a in args:
            if isinstance(a, (list, tuple)):
                ins += [self._id(x) for x in a if isinstance(x, torch.Tensor)]
        outs = out if isinstance(out, (list, tuple)) else [out]
        for o in outs:
            if isinstance(o, torch.Tensor):
                self.ids[id(o)] = self.g.add(name, ins, o.shape, str(o.dtype).replace("torch.", ""),
                                             scalars=[a for a in args if isinstance(a, (int, float)) and not isinstance(a, bool)])
        self._keep = getattr(self, "_keep", []) + [o for o in outs if isinstance(o, torch.Tensor)]  # ids stay unique
        return out


_TRACING_GRAPH: Graph | None = None


def trace(fn, *args) -> Graph:
    """Run ``fn(*args)`` once and record every dispatched op (``CapturedGraph::capture``)."""
    global _TRACING_GRAPH
    g = Graph()
    tr = _Tracer(g)
    for a in args:
        if isinstance(a, torch.Tensor):
            tr._id(a)
    with tr:
        out = fn(*args)
    outs = out if isinstance(out, (list, tuple)) else [out]
    g.outputs = [tr.ids[id(o)] for o in outs if isinstance(o, torch.Tensor) and id(o) in tr.ids]
    _TRACING_GRAPH = g
    return g


def tracing_graph_snapshot() -> Graph | None:
    return _TRACING_GRAPH


# ------------------------------------------------------------------------------------------------ fusion
@dataclass
class FusionGroup:
    nodes: list[int]


def fusion_pass(g: Graph) -> list[FusionGroup]:
    """Maximal chains of pointwise nodes where each intermediate has exactly one consumer and the same shape."""
    cons = g.consumers()
    grouped: set[int] = set()
    groups = []
    for n in g.nodes:
        if n.op not in POINTWISE or n.id in grouped:
            continue
        chain = [n.id]
        cur = n
        while True:
            nxt = cons[cur.id]
            if len(nxt) != 1:
                break
            c = g.nodes[nxt[0]]
            if c.op not in POINTWISE or c.shape != cur.shape or c.id in grouped:
                break
            chain.append(c.id)
            cur = c
        if len(chain) > 1:
            groups.append(FusionGroup(chain))
            grouped.update(chain)
    return groups


def constant_fold(g: Graph, constants: set[int] = frozenset()) -> list[int]:
    """Nodes that depend only on ``constants`` (graph inputs that are weights): candidates for evaluation at
    compile time.  (``ConstantFolder`` in the reference is a pass-through stub; this one does the analysis and leaves
    the evaluation to the caller, which owns the tensors.)"""
    dynamic = set(g.inputs) - set(constants)
    for n in g.nodes:
        if any(i in dynamic for i in n.inputs):
            dynamic.add(n.id)
    return [n.id for n in g.nodes if n.op != "input" and n.id not in dynamic]


def weight_prepack_plan(g: Graph, weight_inputs: set[int]) -> dict[int, str]:
    """Which weight operands a compiled plan would re-lay-out once ahead of time: the second operand of every matrix
    product fed directly by a weight.  The tcgen05 GEMM reads K-major and MN-major operands alike, so the plan is
    "none" for every weight; the pass exists so that a back end with a layout preference has a place to say so."""
    plan = {}
    for n in g.nodes:
        if n.op in ("mm", "matmul", "addmm", "linear", "bmm") and n.inputs and n.inputs[-1] in weight_inputs:
            plan[n.inputs[-1]] = "none (either major is read in place)"
    return plan


_UNARY = {"relu": "relu", "gelu": "gelu", "silu": "swish", "sigmoid": "sigmoid", "tanh": "tanh", "exp": "exp", "log": "log",
          "sqrt": "sqrt", "rsqrt": "rsqrt", "neg": "neg", "abs": "abs", "mish": "mish", "elu": "elu",
          "softplus": "softplus", "sign": "sign", "reciprocal": "recip"}
_BINARY = {"add": "add", "sub": "sub", "mul": "mul", "div": "div", "maximum": "max", "minimum": "min", "pow": "pow"}


def lower_group(g: Graph, group: FusionGroup):
    """One fusion group -> ``(PointwiseExpr, external input node ids)``: the expression of the group's last node
    over the tensors that enter the group from outside.  ``codegen.compile_pointwise`` turns it into one kernel."""
    from .codegen.pointwise import Arg, Binary, Const, Unary
    inside = set(group.nodes)
    ext: list[int] = []
    memo: dict[int, object] = {}

    def expr(nid: int):
        if nid not in inside:
            if nid not in ext:
                ext.append(nid)
            return Arg(ext.index(nid))
        if nid in memo:
            return memo[nid]
        n = g.nodes[nid]
        ops = [expr(i) for i in n.inputs] + [Const(float(s)) for s in n.attrs.get("scalars", [])]
        if n.op in _UNARY and len(ops) == 1:
            e = Unary(_UNARY[n.op], ops[0])
        elif n.op in _BINARY and len(ops) == 2:
            e = Binary(_BINARY[n.op], ops[0], ops[1])
        else:
            raise ValueError(f"cannot lower {n.op} with {len(ops)} operands")
        memo[nid] = e
        return e

    return expr(group.nodes[-1]), ext


# ------------------------------------------------------------------------------------------------ row chains
ROW_OPS = {"_softmax": "softmax", "softmax": "softmax", "_log_softmax": "log_softmax", "log_softmax": "log_softmax"}


@dataclass
class RowFusionGroup:
    """A last-axis softmax / log-softmax with the pointwise nodes that feed it and follow it."""
    pre: list[int]        # pointwise nodes before the row op (may be empty), topological order
    row: int              # the row op's node id
    post: list[int]       # pointwise nodes after it (may be empty)

    @property
    def nodes(self) -> list[int]:
        return self.pre + [self.row] + self.post


def row_fusion_pass(g: Graph) -> list[RowFusionGroup]:
    """Around every last-axis softmax: the pointwise nodes whose only consumer lies inside the group (walking up from
    the row op), and the single-consumer pointwise chain that follows it.  Every member has the row tensor's shape;
    tensors entering from outside may also be ``[C]`` vectors (lowered to per-column operands)."""
    cons = g.consumers()
    out, taken = [], set()
    for n in g.nodes:
        kind = ROW_OPS.get(n.op)
        if kind is None or not n.inputs or not n.shape:
            continue
        dim = (n.attrs.get("scalars") or [-1])[0]
        if int(dim) not in (-1, len(n.shape) - 1):
            continue
        pre: list[int] = []
        frontier = [n.inputs[0]]
        while frontier:
            nid = frontier.pop()
            m = g.nodes[nid]
            if m.op not in POINTWISE or m.shape != n.shape or nid in taken or nid in pre:
                continue
            if nid in g.outputs or any(c != n.id and c not in pre for c in cons[nid]):
                continue                      # somebody outside the group needs this value: it stays materialised
            pre.append(nid)
            frontier.extend(m.inputs)
        post, cur = [], n
        while len(cons[cur.id]) == 1 and cur.id not in g.outputs:
            c = g.nodes[cons[cur.id][0]]
            if c.op not in POINTWISE or c.shape != n.shape or c.id in taken:
                break
            post.append(c.id)
            cur = c
        if pre or post:
            grp = RowFusionGroup(sorted(pre), n.id, post)
            taken.update(grp.nodes)
            out.append(grp)
    return out


def lower_row_group(g: Graph, group: RowFusionGroup):
    """-> ``(kind, pre expression, post expression, row-tensor node ids, column-vector node ids)`` for
    :func:`incin_b200.codegen.fused_rows` (``Arg(i)`` = i-th row tensor, ``Col(i)`` = i-th vector)."""
    from .codegen.pointwise import Arg, Binary, Const, Unary
    from .codegen.rows import Col, Norm
    row = g.nodes[group.row]
    C = row.shape[-1]
    rows_ext: list[int] = []
    cols_ext: list[int] = []

    def leaf(nid: int):
        shape = tuple(g.nodes[nid].shape)
        if shape == tuple(row.shape):
            if nid not in rows_ext:
                rows_ext.append(nid)
            return Arg(rows_ext.index(nid))
        if shape == (C,):
            if nid not in cols_ext:
                cols_ext.append(nid)
            return Col(cols_ext.index(nid))
        raise ValueError(f"operand %{nid} of shape {shape} is neither a row tensor {tuple(row.shape)} nor a [{C}] vector")

    def build(nid: int, inside: set[int], norm_of: int | None):
        if nid == norm_of:
            return Norm()
        if nid not in inside:
            return leaf(nid)
        n = g.nodes[nid]
        ops = [build(i, inside, norm_of) for i in n.inputs] + [Const(float(s)) for s in n.attrs.get("scalars", [])]
        if n.op in _UNARY and len(ops) == 1:
            return Unary(_UNARY[n.op], ops[0])
        if n.op in _BINARY and len(ops) == 2:
            return Binary(_BINARY[n.op], ops[0], ops[1])
        raise ValueError(f"cannot lower {n.op} with {len(ops)} operands")

    pre = build(row.inputs[0], set(group.pre), None)
    post = build(group.post[-1], set(group.post), group.row) if group.post else None
    if not rows_ext:
        raise ValueError("the chain reads no row tensor")
    return ROW_OPS[row.op], pre, post, rows_ext, cols_ext


# ------------------------------------------------------------------------------------------------ memory planning
@dataclass
class MemoryPlan:
    offsets: dict[int, int]
    peak_bytes: int
    naive_bytes: int


_ESZ = {"float32": 4, "bfloat16": 2, "float16": 2, "int64": 8, "int32": 4, "uint8": 1, "bool": 1, "float64": 8}


@dataclass
class SavedTensorSet:
    """Values that forward ops stash for their backward recipes (crates/incin-core/src/compiled/alloc.rs:129-160): the
    memory plan keeps them alive to the end of the backward pass instead of to their last forward use."""
    values: set = field(default_factory=set)

    def save(self, value_id: int) -> None:
        self.values.add(value_id)

    def __contains__(self, value_id: int) -> bool:
        return value_id in self.values

    def __len__(self) -> int:
        return len(self.values)


# what each op's backward reads: "in" = its inputs, "out" = its own output, "in0" = the first input only
_SAVES = {"mm": "in", "bmm": "in", "addmm": "in", "linear": "in", "matmul": "in", "mul": "in", "div": "in", "pow": "in",
          "maximum": "in", "minimum": "in", "where": "in", "relu": "out", "sigmoid": "out", "tanh": "out", "exp": "out",
          "sqrt": "out", "rsqrt": "out", "_softmax": "out", "softmax": "out", "_log_softmax": "out",
          "log_softmax": "out", "gelu": "in", "silu": "in", "log": "in", "abs": "in", "reciprocal": "out", "mish": "in",
          "elu": "in", "softplus": "in", "native_layer_norm": "in", "layer_norm": "in", "convolution": "in",
          "max_pool2d_with_indices": "in", "embedding": "in0", "nll_loss_forward": "in"}


def saved_for_backward(g: Graph) -> SavedTensorSet:
    """The values a backward pass over ``g`` will read again, by the rule table above (ops it does not know keep
    their inputs: the safe side for a memory plan)."""
    saved = SavedTensorSet()
    for n in g.nodes:
        if n.op == "input":
            continue
        rule = _SAVES.get(n.op, "in" if n.op not in ("add", "sub", "neg", "sum", "mean", "view", "reshape", "t",
                                                     "transpose", "permute", "expand", "clone", "detach") else None)
        if rule == "out":
            saved.save(n.id)
        elif rule == "in":
            for i in n.inputs:
                saved.save(i)
        elif rule == "in0" and n.inputs:
            saved.save(n.inputs[0])
    return saved


def liveness(g: Graph, saved: SavedTensorSet | None = None, backward_end: int | None = None) -> dict[int, tuple[int, int]]:
    """node id -> (first, last) position it is alive; graph outputs live to the end.  With ``saved`` the saved values
    stay alive until ``backward_end`` (default: the end of the graph), as ``extend_for_saved_tensors`` does."""
    last = {n.id: n.id for n in g.nodes}
    for n in g.nodes:
        for i in n.inputs:
            last[i] = max(last[i], n.id)
    for o in g.outputs:
        last[o] = len(g.nodes)
    if saved is not None:
        end = len(g.nodes) if backward_end is None else backward_end
        for v in saved.values:
            if v in last and last[v] < end:
                last[v] = end
    return {n.id: (n.id, last[n.id]) for n in g.nodes}


def _plan_memory_native(g: Graph, live, size) -> "MemoryPlan | None":
    """The same greedy first fit in native code (csrc/runtime/memplan.cpp); ``None`` when the host library is absent,
    in which case the Python loop below runs.  ``INCIN_NATIVE_MEMPLAN=0`` forces the Python path."""
    import os
    if os.environ.get("INCIN_NATIVE_MEMPLAN", "1") == "0":
        return None
    try:
        from .runtime import first_fit_arena
        nodes = list(g.nodes)
        offs, peak = first_fit_arena([size[n.id] for n in nodes], [live[n.id][0] for n in nodes],
                                     [live[n.id][1] for n in nodes], [n.op == "input" for n in nodes])
    except (OSError, RuntimeError, AttributeError):
        return None
    offsets = {n.id: o for n, o in zip(nodes, offs) if n.op != "input"}
    return MemoryPlan(offsets, peak, sum(size[n.id] for n in nodes if n.op != "input"))


def plan_memory(g: Graph, align: int = 256, saved: SavedTensorSet | None = None) -> MemoryPlan:
    """Greedy first-fit reuse of a single arena by liveness (``AllocationPlanner``); ``saved`` keeps the values a
    backward pass needs alive to the end."""
    live = liveness(g, saved)
    size = {}
    for n in g.nodes:
        numel = 1
        for d in n.shape:
            numel *= d
        size[n.id] = (numel * _ESZ.get(n.dtype, 4) + align - 1) // align * align
    planned = _plan_memory_native(g, live, size)
    if planned is not None:
        return planned
    placed: list[tuple[int, int, int, int]] = []   # (offset, size, first, last)
    offsets, peak = {}, 0
    for n in g.nodes:
        if n.op == "input":
            continue
        f, l = live[n.id]
        busy = sorted((o, s) for o, s, pf, pl in placed if not (pl < f or pf > l))
        off = 0
        for o, s in busy:
            if off + size[n.id] <= o:
                break
            off = max(off, o + s)
        offsets[n.id] = off
        placed.append((off, size[n.id], f, l))
        peak = max(peak, off + size[n.id])
    return MemoryPlan(offsets, peak, sum(size[n.id] for n in g.nodes if n.op != "input"))


# ------------------------------------------------------------------------------------------------ bounded plan tuning
@dataclass
class PlanTuningReport:
    baseline_latency_us: float
    tuned_latency_us: float
    speedup_ratio: float
    iterations_evaluated: int
    is_bounded: bool
    best: str = "baseline"
    met_target: bool = False


class BoundedPlanTuner:
    """Scores a bounded number of execution variants of a traced graph and reports the best one against the unfused
    single-launch-per-node baseline (crates/incin-core/src/compiled/tuning.rs:24-64, where the sweep is simulated).
    Here the variants are real plan choices (no fusion, pointwise chains fused, row chains fused as well, and arena
    alignments for the memory plan) and the score is an analytical latency: every launch costs ``launch_us`` and every
    materialised tensor is written once and read once per consumer at ``gbs``; a fused group launches once and
    materialises only its last value."""

    def __init__(self, max_iterations: int = 8, min_speedup_target: float = 1.0, launch_us: float = 3.0, gbs: float = 6500.0):
        if max_iterations < 1:
            raise ValueError("max_iterations must be >= 1")
        self.max_iterations, self.min_speedup_target = max_iterations, min_speedup_target
        self.launch_us, self.gbs = launch_us, gbs

    def _latency(self, g: Graph, groups: list[list[int]]) -> float:
        cons = g.consumers()
        member = {}
        for k, grp in enumerate(groups):
            for nid in grp:
                member[nid] = k
        launches = sum(1 for n in g.nodes if n.op != "input" and n.id not in member) + len(groups)
        traffic = 0
        for n in g.nodes:
            numel = 1
            for d in n.shape:
                numel *= d
            nbytes = numel * _ESZ.get(n.dtype, 4)
            k = member.get(n.id)
            internal = k is not None and n.id != groups[k][-1] and all(member.get(c) == k for c in cons[n.id])
            if internal:
                continue                                  # lives in registers inside the fused kernel
            readers = len({member.get(c, ("n", c)) for c in cons[n.id]})   # a fused group reads an operand once
            traffic += nbytes * ((0 if n.op == "input" else 1) + readers)
        return launches * self.launch_us + traffic / (self.gbs * 1e3)

    def tune_plan(self, g: Graph) -> PlanTuningReport:
        variants = [("baseline", [])]
        pw = [grp.nodes for grp in fusion_pass(g)]
        if pw:
            variants.append(("pointwise chains fused", pw))
        rows = row_fusion_pass(g)
        if rows:
            taken = {nid for r in rows for nid in r.nodes}
            variants.append(("pointwise and row chains fused", [r.nodes for r in rows] + [grp for grp in pw if not taken & set(grp)]))
        baseline = self._latency(g, [])
        best_name, best = "baseline", baseline
        it = 0
        for name, groups in variants[: self.max_iterations]:
            it += 1
            t = self._latency(g, groups)
            if t < best:
                best_name, best = name, t
        speed = baseline / best if best > 0 else 1.0
        return PlanTuningReport(baseline, best, speed, it, it <= self.max_iterations, best_name, speed >= self.min_speedup_target)


# ------------------------------------------------------------------------------------------------ plans / artifacts
def shape_bucket(n: int, base: int = 64) -> int:
    """Round a dynamic extent up to its bucket (powers of two times ``base``) so nearby shapes share a plan."""
    b = base
    while b < n:
        b *= 2
    return b


@dataclass
class ShapeGuard:
    shapes: tuple[tuple[int, ...], ...]
    dtypes: tuple[str, ...]

    def admits(self, *tensors: torch.Tensor) -> bool:
        return (tuple(tuple(t.shape) for t in tensors) == self.shapes and
                tuple(str(t.dtype).replace("torch.", "") for t in tensors) == self.dtypes)


@dataclass
class CompiledPlan:
    graph_digest: str
    guard: ShapeGuard
    fusion_groups: list[list[int]]
    memory: MemoryPlan

    @staticmethod
    def build(fn, *args) -> "CompiledPlan":
        g = trace(fn, *args)
        ts = [a for a in args if isinstance(a, torch.Tensor)]
        guard = ShapeGuard(tuple(tuple(t.shape) for t in ts), tuple(str(t.dtype).replace("torch.", "") for t in ts))
        return CompiledPlan(g.digest(), guard, [fg.nodes for fg in fusion_pass(g)], plan_memory(g))


MAGIC = b"INCINCG1"


def write_artifact(path, plan: CompiledPlan, manifest: dict | None = None) -> None:
    """``magic | adler32(payload) | length | payload(json)``: a torn or edited file fails the checksum on load."""
    payload = json.dumps({"plan": {"graph_digest": plan.graph_digest, "guard": asdict(plan.guard),
                                   "fusion_groups": plan.fusion_groups, "memory": asdict(plan.memory)},
                          "manifest": manifest or reproducibility_manifest()}).encode()
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<IQ", zlib.adler32(payload), len(payload)) + payload)


def read_artifact(path) -> dict:
    raw = open(path, "rb").read()
    if raw[:8] != MAGIC:
        raise ValueError("not a compiled-graph artifact")
    chk, n = struct.unpack_from("<IQ", raw, 8)
    payload = raw[20:20 + n]
    if len(payload) != n or zlib.adler32(payload) != chk:
        raise ValueError("compiled-graph artifact failed its checksum")
    return json.loads(payload)


def reproducibility_manifest() -> dict:
    from . import __version__
    from .core.policy import current_policy
    return {"incin_b200": __version__, "torch": torch.__version__, "cuda": str(torch.version.cuda),
            "policy": current_policy().cache_key(), "arch": "sm_100a"}
