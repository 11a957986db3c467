"""Row-chain fuser: pointwise prologue -> row normalisation (softmax / layer norm / rms norm) -> pointwise epilogue,
rendered as ONE sm_100a kernel.

The reference's renderer specialises its normalisation templates per dtype and fuses neighbouring pointwise pairs only
(crates/incin-backends/src/kernel.rs:1233-1389, crates/incin-core/src/compiled/: ``FusionPass``); chains such as
``softmax(x * scale + mask)``, ``layer_norm(x + residual) * g + b`` or ``gelu(rms_norm(x) * g)`` cost it one launch and
one round trip through memory per op.  Here the whole chain is one kernel:

* ``pre``   a :class:`PointwiseExpr` over ``Arg(i)`` (row tensors ``[rows, C]``), ``Col(i)`` (vectors ``[C]``, one
            value per column) and ``Scalar(i)``: the value that is normalised;
* ``kind``  ``softmax`` | ``log_softmax`` | ``layer_norm`` | ``rms_norm`` over the last axis;
* ``post``  a :class:`PointwiseExpr` in which ``Norm()`` stands for the normalised value (default: just that).

One warp owns a row; the prologue is re-evaluated in each of the two or three passes over the row instead of being
stored (inputs of a row stay in L1 / L2 between the passes), 16-bit types compute in fp32.
"""
from __future__ import annotations

import collections
import ctypes
import hashlib
from dataclasses import dataclass

from .pointwise import BINARY, CTYPES, TERNARY, UNARY, Arg, Binary, Const, PointwiseExpr, Scalar, Ternary, Unary

KINDS = ("softmax", "log_softmax", "layer_norm", "rms_norm")


@dataclass(frozen=True, eq=True)
class Col(PointwiseExpr):
    """A per-column vector ``[C]`` (a gain, a bias, a mask row) broadcast over the rows."""
    index: int


@dataclass(frozen=True, eq=True)
class Norm(PointwiseExpr):
    """The normalised value of the element, inside the epilogue expression."""


def _walk(e, fn):
    fn(e)
    for n in ("x", "a", "b", "c"):
        if hasattr(e, n):
            _walk(getattr(e, n), fn)


def _counts(*exprs) -> tuple[int, int, int]:
    a = c = s = 0

    def see(e):
        nonlocal a, c, s
        if isinstance(e, Arg):
            a = max(a, e.index + 1)
        elif isinstance(e, Col):
            c = max(c, e.index + 1)
        elif isinstance(e, Scalar):
            s = max(s, e.index + 1)
    for e in exprs:
        _walk(e, see)
    return a, c, s


def _emit(e, norm: str | None) -> str:
    if isinstance(e, Arg):
        return f"ld(in{e.index} + base + c)"
    if isinstance(e, Col):
        return f"ld(col{e.index} + c)"
    if isinstance(e, Scalar):
        return f"s{e.index}"
    if isinstance(e, Norm):
        if norm is None:
            raise ValueError("Norm() is only meaningful in the epilogue expression")
        return norm
    if isinstance(e, Const):
        v = float(e.value)
        if v != v:
            return "CUDART_NAN_F"
        if abs(v) == float("inf"):
            return "CUDART_INF_F" if v > 0 else "-CUDART_INF_F"
        return repr(v) + "f"
    if isinstance(e, Unary):
        return UNARY[e.op].format(x=_emit(e.x, norm))
    if isinstance(e, Binary):
        return BINARY[e.op].format(a=_emit(e.a, norm), b=_emit(e.b, norm))
    if isinstance(e, Ternary):
        return TERNARY[e.op].format(a=_emit(e.a, norm), b=_emit(e.b, norm), c=_emit(e.c, norm))
    raise TypeError(e)


@dataclass(frozen=True)
class RowKernelKey:
    digest: str
    kind: str
    dtype: str
    n_args: int
    n_cols: int
    n_scalars: int

    @property
    def entry(self) -> str:
        return f"incin_row_{self.kind}_{self.dtype}_{self.digest[:16]}"


def render_row_cuda(kind: str, pre: PointwiseExpr, post: PointwiseExpr | None = None, dtype: str = "bf16") -> tuple[str, RowKernelKey]:
    """CUDA C source.  Signature: ``(out, in0.., col0.., s0.., float eps, long long rows, int C)``."""
    if kind not in KINDS:
        raise ValueError(f"unknown row kind {kind} (one of {', '.join(KINDS)})")
    if dtype not in CTYPES:
        raise ValueError(f"unsupported dtype {dtype}")
    post = Norm() if post is None else post
    found = []
    _walk(pre, lambda e: found.append(isinstance(e, Norm)))
    if any(found):
        raise ValueError("the prologue cannot refer to Norm()")
    n_in, n_col, n_sc = _counts(pre, post)
    if n_in < 1:
        raise ValueError("the prologue must read at least one row tensor (Arg(0))")
    ct = CTYPES[dtype][0]
    key = RowKernelKey(hashlib.sha256(repr((kind, pre, post)).encode()).hexdigest(), kind, dtype, n_in, n_col, n_sc)
    ld = {"float": "(*(p))", "__nv_bfloat16": "__bfloat162float(*(p))", "__half": "__half2float(*(p))"}[ct]
    st = {"float": "(v)", "__nv_bfloat16": "__float2bfloat16(v)", "__half": "__float2half(v)"}[ct]
    ins = "".join(f", const {ct}* __restrict__ in{i}" for i in range(n_in))
    cols = "".join(f", const {ct}* __restrict__ col{i}" for i in range(n_col))
    scs = "".join(f", float s{i}" for i in range(n_sc))
    v = _emit(pre, None)
    if kind in ("softmax", "log_softmax"):
        stats = f"""
    float m = -CUDART_INF_F;
    for (int c = lane; c < C; c += 32) m = fmaxf(m, {v});
    m = warp_max(m);
    float z = 0.f;
    for (int c = lane; c < C; c += 32) z += __expf(({v}) - m);
    z = warp_sum(z);"""
        normed = f"(__expf(({v}) - m) / z)" if kind == "softmax" else f"((({v}) - m) - __logf(z))"
    elif kind == "layer_norm":
        stats = f"""
    float mu = 0.f;
    for (int c = lane; c < C; c += 32) mu += {v};
    mu = warp_sum(mu) / C;
    float var = 0.f;
    for (int c = lane; c < C; c += 32) {{ const float d = ({v}) - mu; var += d * d; }}
    const float rstd = rsqrtf(warp_sum(var) / C + eps);"""
        normed = f"((({v}) - mu) * rstd)"
    else:
        stats = f"""
    float ss = 0.f;
    for (int c = lane; c < C; c += 32) {{ const float t = {v}; ss += t * t; }}
    const float rstd = rsqrtf(warp_sum(ss) / C + eps);"""
        normed = f"(({v}) * rstd)"
    body = _emit(post, normed)
    src = f"""#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>
#define ld(p) {ld}
__device__ __forceinline__ float warp_sum(float x) {{
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}}
__device__ __forceinline__ float warp_max(float x) {{
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}}
extern "C" __global__ void __launch_bounds__(256) {key.entry}({ct}* __restrict__ out{ins}{cols}{scs}, float eps, long long rows, int C) {{
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {{
    const long long base = row * C;{stats}
    for (int c = lane; c < C; c += 32) {{
      const float v = {body};
      out[base + c] = {st};
    }}
  }}
}}
"""
    return src, key


_TORCH_NAMES = None


def _dtype_name(t) -> str:
    import torch
    return {torch.float32: "f32", torch.bfloat16: "bf16", torch.float16: "f16"}[t]


class RowKernel:
    def __init__(self, kind: str, pre: PointwiseExpr, post: PointwiseExpr | None, dtype: str):
        self.source, self.key = render_row_cuda(kind, pre, post, dtype)
        self._fn = None

    def _load(self):
        from cuda.bindings import driver
        from .runtime import CompileError, cubin_for
        err, mod = driver.cuModuleLoadData(cubin_for(self.source, self.key))
        if err != driver.CUresult.CUDA_SUCCESS:
            raise CompileError(f"cuModuleLoadData: {err}")
        err, fn = driver.cuModuleGetFunction(mod, self.key.entry.encode())
        if err != driver.CUresult.CUDA_SUCCESS:
            raise CompileError(f"cuModuleGetFunction({self.key.entry}): {err}")
        self._mod, self._fn = mod, fn

    def __call__(self, rows_in, cols=(), scalars=(), eps: float = 1e-5, out=None):
        import torch
        from cuda.bindings import driver
        from .runtime import CompileError
        k = self.key
        if len(rows_in) != k.n_args or len(cols) != k.n_cols or len(scalars) != k.n_scalars:
            raise ValueError(f"kernel takes {k.n_args} row tensors, {k.n_cols} column vectors and {k.n_scalars} scalars")
        x = rows_in[0]
        C = x.shape[-1]
        if any(t.shape != x.shape or not t.is_contiguous() or t.dtype != x.dtype for t in rows_in):
            raise ValueError("row tensors must be dense, of one shape and dtype")
        if any(v.shape != (C,) or not v.is_contiguous() or v.dtype != x.dtype for v in cols):
            raise ValueError(f"column vectors must be dense [{C}] tensors of the rows' dtype")
        torch.cuda.current_stream()
        if self._fn is None:
            self._load()
        out = torch.empty_like(x) if out is None else out
        rows = x.numel() // C if C else 0
        if rows == 0:
            return out
        args = [out.data_ptr()] + [t.data_ptr() for t in rows_in] + [v.data_ptr() for v in cols] + \
               [float(s) for s in scalars] + [float(eps), rows, C]
        types = [ctypes.c_void_p] * (1 + len(rows_in) + len(cols)) + [ctypes.c_float] * (len(scalars) + 1) + \
                [ctypes.c_longlong, ctypes.c_int]
        blocks = max(1, min((rows + 7) // 8, 148 * 8))
        (err,) = driver.cuLaunchKernel(self._fn, blocks, 1, 1, 256, 1, 1, 0, torch.cuda.current_stream().cuda_stream,
                                       (tuple(args), tuple(types)), 0)
        if err != driver.CUresult.CUDA_SUCCESS:
            raise CompileError(f"cuLaunchKernel({k.entry}): {err}")
        return out


_cache: "collections.OrderedDict[tuple, RowKernel]" = collections.OrderedDict()


def fused_rows(kind: str, pre: PointwiseExpr, rows_in, *, post: PointwiseExpr | None = None, cols=(), scalars=(),
               eps: float = 1e-5, out=None):
    """Run ``post(norm_kind(pre(rows_in, cols, scalars)))`` over the last axis as one kernel (compiled once per
    expression and dtype, cached like the pointwise kernels)."""
    from .runtime import CACHE_BOUND
    dt = _dtype_name(rows_in[0].dtype)
    ck = (kind, pre, post, dt)
    k = _cache.get(ck)
    if k is None:
        k = _cache[ck] = RowKernel(kind, pre, post, dt)
        while len(_cache) > CACHE_BOUND:
            _cache.popitem(last=False)
    else:
        _cache.move_to_end(ck)
    return k(tuple(rows_in), tuple(cols), tuple(scalars), eps, out)


def reference_rows(kind: str, pre, rows_in, *, post=None, cols=(), scalars=(), eps: float = 1e-5):
    """The same chain in plain fp32 PyTorch (any device): the oracle the tests hold the kernel to, and the CPU path."""
    import torch
    fn = {"relu": torch.relu, "step": lambda x: (x > 0).float(), "sigmoid": torch.sigmoid, "tanh": torch.tanh,
          "swish": torch.nn.functional.silu, "softplus": torch.nn.functional.softplus, "elu": torch.nn.functional.elu,
          "gelu": torch.nn.functional.gelu, "gelu_tanh": lambda x: torch.nn.functional.gelu(x, approximate="tanh"),
          "exp": torch.exp, "log": torch.log, "sqrt": torch.sqrt, "rsqrt": torch.rsqrt, "neg": torch.neg, "abs": torch.abs,
          "sign": torch.sign, "mish": torch.nn.functional.mish, "recip": torch.reciprocal, "square": torch.square,
          "sin": torch.sin, "cos": torch.cos, "floor": torch.floor, "ceil": torch.ceil}
    bi = {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div, "max": torch.maximum,
          "min": torch.minimum, "pow": torch.pow}
    R = [t.float() for t in rows_in]
    V = [v.float() for v in cols]

    def ev(e, norm=None):
        if isinstance(e, Arg):
            return R[e.index]
        if isinstance(e, Col):
            return V[e.index]
        if isinstance(e, Scalar):
            return torch.tensor(float(scalars[e.index]), device=R[0].device)
        if isinstance(e, Const):
            return torch.tensor(float(e.value), device=R[0].device)
        if isinstance(e, Norm):
            return norm
        if isinstance(e, Unary):
            return fn[e.op](ev(e.x, norm))
        if isinstance(e, Binary):
            return bi[e.op](ev(e.a, norm), ev(e.b, norm))
        if isinstance(e, Ternary):
            a, b, c = ev(e.a, norm), ev(e.b, norm), ev(e.c, norm)
            return {"clamp": lambda: torch.minimum(torch.maximum(a, b), c), "fma": lambda: a * b + c,
                    "where": lambda: torch.where(a != 0, b, c)}[e.op]()
        raise TypeError(e)
    v = ev(pre) + torch.zeros_like(R[0])
    if kind == "softmax":
        n = torch.softmax(v, -1)
    elif kind == "log_softmax":
        n = torch.log_softmax(v, -1)
    elif kind == "layer_norm":
        n = (v - v.mean(-1, keepdim=True)) * torch.rsqrt(v.var(-1, unbiased=False, keepdim=True) + eps)
    elif kind == "rms_norm":
        n = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    else:
        raise ValueError(kind)
    return ev(Norm() if post is None else post, n)
