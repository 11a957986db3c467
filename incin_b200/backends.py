"""Backends, the run-time (``Dyn``) dispatcher, the shape-only fake and the conformance suite.

Counterparts: the backend trait family and ``DummyBackend`` (crates/incin-core/src/tensor/backend.rs:66-985), the
``Dyn``-device dispatcher (crates/incin-backends/src/dispatch.rs:9-66, 1196-1217: ``DispatchStorage{Cpu, Wgpu, Cuda,
Unavailable}`` and a per-op ``match device.kind()``) and the capability-driven conformance suite that external
backends are held to (crates/incin-backends/src/external/conformance.rs:1-80: skip what a subject does not claim,
compare the rest with ``Tolerance{EXACT, F32_ACCUMULATED, F32_WIDE}``).

A backend here is a table ``op name -> callable`` over torch tensors plus its capability registry:

* :class:`CpuBackend`    the oracle and default: PyTorch CPU math in fp32 plus the C++ oracle library;
* :class:`CudaBackend`   the hand-written sm_100a kernels (every entry raises if the library is missing: no fallback);
* :class:`DummyBackend`  computes shapes and dtypes only (meta tensors): planners and tests use it to walk a model
                         without memory or a device;
* :class:`DispatchBackend` picks per call from the device of the first tensor argument and refuses devices that have
                         no backend in this process ("unavailable"), which is what a ``Dyn`` device means.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Callable

import torch

from .core.device import DeviceKind
from .core.dtype import DTypeId, from_torch
from .core.spec import REGISTRIES, CapabilityQuery, SupportLevel
from .ops import functional as F
from .ops import tensor_ops as T


class BackendUnavailable(RuntimeError):
    pass


_FUSABLE = (torch.float32, torch.bfloat16, torch.float16)
_UNARY_ALIASES = {"silu": "swish", "reciprocal": "recip"}


def _binary(name: str, torch_fn: Callable) -> Callable:
    """Elementwise binary op: on CUDA it is one kernel of the pointwise fuser (NVRTC, sm_100a; broadcasting through the
    strided layout), on the CPU the PyTorch op."""
    def run(a, b):
        if isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor) and a.is_cuda and b.is_cuda and \
                a.dtype == b.dtype and a.dtype in _FUSABLE:
            from .codegen import Arg, Binary, fused
            return fused(Binary(name, Arg(0), Arg(1)), a, b)
        return torch_fn(a, b)
    return run


def _unary(x, name: str):
    from .codegen.pointwise import UNARY
    op = _UNARY_ALIASES.get(name, name)
    if x.is_cuda and x.dtype in _FUSABLE and op in UNARY:
        from .codegen import Arg, Unary, fused
        return fused(Unary(op, Arg(0)), x)
    return F.activation(x, name) if name in ("gelu", "silu") else getattr(torch, name)(x)


def _ops() -> dict[str, Callable]:
    """The op surface shared by the real backends (functional front end: CUDA kernels or their CPU twins)."""
    return {
        "matmul": lambda a, b: F.linear(a, b.t().contiguous()) if a.is_cuda else a @ b,
        "addmm": lambda x, w, b: F.linear(x, w, b),
        "add": _binary("add", torch.add), "sub": _binary("sub", torch.sub), "mul": _binary("mul", torch.mul),
        "div": _binary("div", torch.div), "maximum": _binary("max", torch.maximum), "minimum": _binary("min", torch.minimum),
        "unary": _unary,
        "softmax": lambda x, dim=-1: T.softmax(x, dim),
        "conv1d": T.conv1d, "conv2d": T.conv2d, "conv_transpose2d": T.conv_transpose2d,
        "adaptive_avg_pool2d": T.adaptive_avg_pool2d,
        "layer_norm": F.layer_norm, "rms_norm": F.rms_norm, "embedding": F.embedding,
        "cross_entropy": lambda logits, target: F.cross_entropy(logits, target, logits.shape[-1]),
        "sdpa": lambda qkv, heads: F.causal_attention(qkv, heads),
        "sum": lambda x, dim=None: T.reduce(x, "sum", dim), "mean": lambda x, dim=None: T.reduce(x, "mean", dim),
        "max": lambda x, dim=None: T.reduce(x, "max", dim), "min": lambda x, dim=None: T.reduce(x, "min", dim),
        "argmax": lambda x, dim=None: T.reduce(x, "argmax", dim), "cumsum": T.cumsum,
        "max_pool2d": T.max_pool2d, "avg_pool2d": T.avg_pool2d, "batch_norm": T.batch_norm,
        "concat": T.concat, "gather": T.gather_last, "index_select": T.index_select,
        "transpose": lambda x, a, b: x.transpose(a, b), "reshape": lambda x, shape: x.reshape(shape),
        "rope": F.rope, "swiglu": F.swiglu,
    }


class Backend:
    kind: DeviceKind
    name: str

    def __init__(self):
        self.ops = _ops()
        self.registry = REGISTRIES[self.kind]

    def supports(self, op: str, dtype: DTypeId) -> SupportLevel:
        return self.registry.query(CapabilityQuery(op, dtype, self.kind)).level

    def device(self) -> torch.device:
        raise NotImplementedError

    def run(self, op: str, *args, **kw):
        if op not in self.ops:
            raise KeyError(f"{self.name} backend has no op {op!r}")
        return self.ops[op](*args, **kw)


class CpuBackend(Backend):
    kind, name = DeviceKind.CPU, "cpu"

    def device(self):
        return torch.device("cpu")


class CudaBackend(Backend):
    kind, name = DeviceKind.CUDA, "cuda"

    def __init__(self, index: int = 0):
        if not torch.cuda.is_available():
            raise BackendUnavailable("no CUDA device is visible to this process")
        from . import _native
        _native.cuda()      # fail loudly here, not at the first op, if the kernel library cannot be loaded
        super().__init__()
        self.index = index

    def device(self):
        return torch.device("cuda", self.index)


class NumpyBackend(Backend):
    """An EXTERNAL library held to the same contract: the op table mapped onto NumPy, with a capability table of its
    own (fp32 only, a subset of the ops).  This is the role of the reference's Candle adapter
    (crates/incin-backends/src/external/: a third-party tensor library behind the backend traits, admitted through the
    conformance suite): what it does not claim is skipped, what it claims must match the fp32 CPU reference."""
    kind, name = DeviceKind.CPU, "numpy"

    def __init__(self):
        import numpy as np
        from .core.spec import CapabilityRegistry, CapabilityRule
        f32 = (DTypeId.F32,)
        claimed = ("matmul", "addmm", "add", "sub", "mul", "div", "unary", "softmax", "layer_norm", "rms_norm", "sum",
                   "mean", "max", "min", "argmax", "cumsum", "concat", "transpose", "index_select", "embedding")
        self.registry = CapabilityRegistry(DeviceKind.CPU, [CapabilityRule(op, f32, SupportLevel.NATIVE, "numpy") for op in claimed])
        n = lambda t: t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else t
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)) if isinstance(a, np.ndarray) else torch.as_tensor(a)

        def softmax(x, dim=-1):
            e = np.exp(x - x.max(axis=dim, keepdims=True))
            return e / e.sum(axis=dim, keepdims=True)

        def layer_norm(x, g, b=None, eps=1e-5):
            mu, var = x.mean(-1, keepdims=True), x.var(-1, keepdims=True)
            y = (x - mu) / np.sqrt(var + eps) * g
            return y if b is None else y + b

        erf = np.vectorize(__import__("math").erf, otypes=[np.float32])
        unary = {"relu": lambda x: np.maximum(x, 0), "exp": np.exp, "log": np.log, "tanh": np.tanh, "sqrt": np.sqrt,
                 "abs": np.abs, "neg": np.negative, "sigmoid": lambda x: 1 / (1 + np.exp(-x)),
                 "gelu": lambda x: 0.5 * x * (1 + erf(x * 0.70710678)), "silu": lambda x: x / (1 + np.exp(-x))}
        table = {
            "matmul": lambda a, b: a @ b, "addmm": lambda x, w, b: x @ w.T + b,
            "add": np.add, "sub": np.subtract, "mul": np.multiply, "div": np.divide,
            "unary": lambda x, name: unary[name](x), "softmax": softmax, "layer_norm": layer_norm,
            "rms_norm": lambda x, g, eps=1e-5: x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * g,
            "sum": lambda x, dim=None: x.sum(axis=dim), "mean": lambda x, dim=None: x.mean(axis=dim),
            "max": lambda x, dim=None: x.max(axis=dim), "min": lambda x, dim=None: x.min(axis=dim),
            "argmax": lambda x, dim=None: x.argmax(axis=dim), "cumsum": lambda x, dim: np.cumsum(x, axis=dim),
            "concat": lambda ts, dim=0: np.concatenate(ts, axis=dim), "transpose": lambda x, a, b: np.swapaxes(x, a, b),
            "index_select": lambda x, dim, idx: np.take(x, idx, axis=dim),
            "embedding": lambda idx, w, pos=None: w[idx] if pos is None else w[idx] + pos[: idx.shape[-1]],
        }
        self.ops = {name: (lambda *a, _f=fn, **kw: t(_f(*[[n(u) for u in v] if isinstance(v, (list, tuple)) and v and
                                                           isinstance(v[0], torch.Tensor) else n(v) for v in a], **kw)))
                    for name, fn in table.items()}

    def device(self):
        return torch.device("cpu")


class DummyBackend(Backend):
    """Shape-only execution on meta tensors: no storage, no kernels."""
    kind, name = DeviceKind.CPU, "dummy"

    def device(self):
        return torch.device("meta")

    def run(self, op: str, *args, **kw):
        args = [a.to("meta") if isinstance(a, torch.Tensor) else a for a in args]
        table = {"matmul": lambda a, b: a @ b, "addmm": lambda x, w, b: torch.nn.functional.linear(x, w, b),
                 "layer_norm": lambda x, g, b=None, eps=1e-5: torch.nn.functional.layer_norm(x, x.shape[-1:], g, b, eps),
                 "rms_norm": lambda x, g, eps=1e-5: x, "concat": lambda ts, dim=0: torch.cat(ts, dim),
                 "sum": lambda x, dim=None: x.sum() if dim is None else x.sum(dim),
                 "mean": lambda x, dim=None: x.mean() if dim is None else x.mean(dim),
                 "max_pool2d": lambda x, k, s=None, p=0: torch.nn.functional.max_pool2d(x, k, s, p)}
        fn = table.get(op)
        if fn is None:
            raise KeyError(f"dummy backend has no shape rule for {op!r}")
        return fn(*args, **kw)


class DispatchBackend:
    """``Dyn`` device: the backend is chosen per call from where the data lives."""

    def __init__(self):
        self._backends: dict[DeviceKind, Backend] = {DeviceKind.CPU: CpuBackend()}
        try:
            self._backends[DeviceKind.CUDA] = CudaBackend()
        except Exception as e:          # stays unavailable; asking for it says why
            self._unavailable = {DeviceKind.CUDA: str(e)}
        else:
            self._unavailable = {}

    def backend_for(self, t: torch.Tensor) -> Backend:
        kind = DeviceKind.CUDA if t.is_cuda else DeviceKind.CPU
        if t.device.type not in ("cpu", "cuda"):
            raise BackendUnavailable(f"no backend for device type {t.device.type!r}")
        b = self._backends.get(kind)
        if b is None:
            raise BackendUnavailable(f"{kind.value} backend unavailable: {self._unavailable.get(kind, 'not built')}")
        return b

    def run(self, op: str, *args, **kw):
        first = next((a for a in args if isinstance(a, torch.Tensor)), None)
        if first is None and args and isinstance(args[0], (list, tuple)):
            first = args[0][0]
        if first is None:
            raise ValueError("dispatch needs at least one tensor argument")
        return self.backend_for(first).run(op, *args, **kw)


# ---------------------------------------------------------------------------------------------------- conformance
class Tolerance(enum.Enum):
    EXACT = (0.0, 0.0)
    F32_ACCUMULATED = (1e-5, 1e-5)
    F32_WIDE = (1e-3, 1e-3)
    BF16 = (3e-2, 3e-2)

    @property
    def rtol(self):
        return self.value[0]

    @property
    def atol(self):
        return self.value[1]


@dataclass
class Case:
    op: str
    dtype: DTypeId
    make: Callable[[torch.device, torch.dtype], tuple]
    tolerance: Tolerance
    reference: Callable | None = None       # fp32 CPU reference; default: the CPU backend's own op


@dataclass
class CaseResult:
    op: str
    dtype: str
    status: str          # passed | failed | skipped
    detail: str = ""


def _cases() -> list[Case]:
    g = lambda *shape: torch.randn(*shape, generator=torch.Generator().manual_seed(sum(shape)))
    mk = lambda *tensors: (lambda dev, dt: tuple(t.to(dev, dt) if t.is_floating_point() else t.to(dev) for t in tensors))
    out = []
    for dt, tol in ((DTypeId.F32, Tolerance.F32_WIDE), (DTypeId.BF16, Tolerance.BF16)):
        out += [
            Case("matmul", dt, mk(g(128, 64), g(64, 96)), tol, lambda a, b: a @ b),
            Case("addmm", dt, mk(g(128, 64), g(96, 64), g(96)), tol, lambda x, w, b: x @ w.t() + b),
            Case("layer_norm", dt, mk(g(64, 128), torch.ones(128), torch.zeros(128)), tol,
                 lambda x, w, b: torch.nn.functional.layer_norm(x, (128,), w, b)),
            Case("rms_norm", dt, mk(g(64, 128), torch.ones(128)), tol,
                 lambda x, w: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w),
            Case("sum", dt, mk(g(33, 257)), tol, lambda x: x.sum()),
            Case("max", dt, mk(g(33, 257)), Tolerance.EXACT if dt is DTypeId.F32 else tol, lambda x: x.max()),
            Case("cumsum", dt, lambda dev, d, x=g(8, 300): (x.to(dev, d), 1), tol, lambda x, dim: torch.cumsum(x, dim)),
            Case("max_pool2d", dt, lambda dev, d, x=g(2, 3, 16, 16): (x.to(dev, d), 2), Tolerance.EXACT if dt is DTypeId.F32 else tol,
                 lambda x, k: torch.nn.functional.max_pool2d(x, k)),
            Case("concat", dt, lambda dev, d, a=g(4, 8), b=g(4, 3): ([a.to(dev, d), b.to(dev, d)], 1), Tolerance.EXACT,
                 lambda ts, dim: torch.cat(ts, dim)),
            Case("add", dt, mk(g(32, 48), g(32, 48)), tol, torch.add),
            Case("sub", dt, mk(g(32, 48), g(1, 48)), tol, torch.sub),                      # broadcast over rows
            Case("mul", dt, mk(g(32, 48), g(32, 1)), tol, torch.mul),                      # broadcast over columns
            Case("div", dt, lambda dev, d, a=g(32, 48), b=g(32, 48).abs() + 0.5: (a.to(dev, d), b.to(dev, d)), tol, torch.div),
            Case("unary", dt, lambda dev, d, x=g(40, 72): (x.to(dev, d), "gelu"), tol, lambda x, n: torch.nn.functional.gelu(x)),
            Case("unary", dt, lambda dev, d, x=g(40, 72): (x.to(dev, d), "tanh"), tol, lambda x, n: torch.tanh(x)),
            Case("unary", dt, lambda dev, d, x=g(40, 72) * 0.5: (x.to(dev, d), "exp"), tol, lambda x, n: torch.exp(x)),
            Case("softmax", dt, lambda dev, d, x=g(24, 200): (x.to(dev, d), -1), tol, lambda x, dim: torch.softmax(x, dim)),
            Case("mean", dt, lambda dev, d, x=g(17, 130): (x.to(dev, d), 1), tol, lambda x, dim: x.mean(dim)),
            Case("min", dt, mk(g(33, 257)), Tolerance.EXACT if dt is DTypeId.F32 else tol, lambda x: x.min()),
            Case("argmax", dt, lambda dev, d, x=g(9, 120): (x.to(dev, d), 1), Tolerance.EXACT, lambda x, dim: x.argmax(dim)),
            Case("avg_pool2d", dt, lambda dev, d, x=g(2, 3, 16, 16): (x.to(dev, d), 2), tol,
                 lambda x, k: torch.nn.functional.avg_pool2d(x, k)),
            Case("adaptive_avg_pool2d", dt, lambda dev, d, x=g(2, 3, 15, 10): (x.to(dev, d), (4, 3)), tol,
                 lambda x, o: torch.nn.functional.adaptive_avg_pool2d(x, o)),
            Case("conv2d", dt, mk(g(2, 8, 12, 12), g(16, 8, 3, 3) * 0.2, g(16)), tol,
                 lambda x, w, b: torch.nn.functional.conv2d(x, w, b)),
            Case("conv1d", dt, mk(g(2, 8, 40), g(16, 8, 3) * 0.2, g(16)), tol, lambda x, w, b: torch.nn.functional.conv1d(x, w, b)),
            Case("conv_transpose2d", dt, mk(g(2, 8, 6, 6), g(8, 16, 3, 3) * 0.2, g(16)), tol,
                 lambda x, w, b: torch.nn.functional.conv_transpose2d(x, w, b)),
            Case("transpose", dt, lambda dev, d, x=g(6, 10): (x.to(dev, d), 0, 1), Tolerance.EXACT, lambda x, a, b: x.transpose(a, b)),
            Case("index_select", dt, lambda dev, d, x=g(12, 16): (x.to(dev, d), 0, torch.tensor([3, 0, 11, 3]).to(dev)),
                 Tolerance.EXACT, lambda x, dim, idx: x.index_select(dim, idx)),
            Case("embedding", dt, lambda dev, d, w=g(50, 32): (torch.tensor([[1, 4, 49], [0, 0, 7]]).to(dev), w.to(dev, d)),
                 Tolerance.EXACT if dt is DTypeId.F32 else tol, lambda idx, w: w[idx]),
        ]
    return out


def run_conformance(subject: Backend, device: torch.device | None = None) -> list[CaseResult]:
    """Hold ``subject`` to the fp32 CPU reference on every case whose (op, dtype) it claims; skip the rest."""
    from .core.dtype import to_torch
    device = device or subject.device()
    results = []
    for c in _cases():
        if not subject.supports(c.op, c.dtype).is_supported:
            results.append(CaseResult(c.op, c.dtype.value, "skipped", "not claimed by the subject's capability table"))
            continue
        try:
            args = c.make(device, to_torch(c.dtype))
            got = subject.run(c.op, *args)
            # the reference sees the same (rounded) inputs, in fp32
            up = lambda a: a.float() if isinstance(a, torch.Tensor) and a.is_floating_point() else a
            ref_args = [[up(t) for t in a] if isinstance(a, list) else up(a) for a in c.make(torch.device("cpu"), to_torch(c.dtype))]
            want = c.reference(*ref_args)
            torch.testing.assert_close(got.detach().float().cpu(), want.float(), rtol=c.tolerance.rtol,
                                       atol=c.tolerance.atol * max(1.0, float(want.abs().max())))
            results.append(CaseResult(c.op, c.dtype.value, "passed"))
        except AssertionError as e:
            results.append(CaseResult(c.op, c.dtype.value, "failed", str(e).splitlines()[0][:200]))
        except Exception as e:
            results.append(CaseResult(c.op, c.dtype.value, "failed", f"{type(e).__name__}: {e}"[:200]))
    return results
