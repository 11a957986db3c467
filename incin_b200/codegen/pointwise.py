"""Pointwise expression AST and its CUDA renderer.

Counterpart of crates/incin-backends/src/codegen/pointwise.rs (``PointwiseExpr``: Arg / Const /
Unary(17) / Binary(7) / Ternary(Clamp, Fma); layouts Contiguous / Strided / ScalarBroadcast; renderers for
CUDA, WGSL and MSL) and of the template renderer crates/incin-backends/src/kernel.rs (dtype / layout / access
specialisation, ``KernelKey`` cache ids).  The CUDA target is the one that runs; :mod:`incin_b200.codegen.shading`
renders the same expressions as WGSL and MSL source text (``gelu_tanh`` is the WGSL shader's GELU).

Differences by design: a whole chain of ops becomes ONE kernel (the reference fuses adjacent pairs at most),
scalars are kernel ARGUMENTS (the reference bakes each scalar into the source text and recompiles per value:
crates/incin-backends/src/cuda/backend.rs:930-945), 16-bit types compute in fp32 and move 128 bits per
access on the contiguous path.
"""
from __future__ import annotations

import enum
import hashlib
from dataclasses import dataclass

UNARY = {
    "relu": "fmaxf({x}, 0.0f)", "step": "({x} > 0.0f ? 1.0f : 0.0f)", "sigmoid": "(1.0f / (1.0f + __expf(-{x})))",
    "tanh": "tanhf({x})", "swish": "({x} / (1.0f + __expf(-{x})))", "softplus": "log1pf(__expf({x}))",
    "elu": "({x} > 0.0f ? {x} : expm1f({x}))", "gelu": "(0.5f * {x} * (1.0f + erff({x} * 0.70710678f)))",
    "gelu_tanh": "(0.5f * {x} * (1.0f + tanhf(0.79788456f * ({x} + 0.044715f * {x} * {x} * {x}))))",
    "exp": "__expf({x})", "log": "__logf({x})", "sqrt": "sqrtf({x})", "rsqrt": "rsqrtf({x})", "neg": "(-{x})",
    "abs": "fabsf({x})", "sign": "(({x} > 0.0f) - ({x} < 0.0f))", "mish": "({x} * tanhf(log1pf(__expf({x}))))",
    "recip": "(1.0f / {x})", "square": "({x} * {x})", "sin": "__sinf({x})", "cos": "__cosf({x})",
    "floor": "floorf({x})", "ceil": "ceilf({x})",
}
BINARY = {"add": "({a} + {b})", "sub": "({a} - {b})", "mul": "({a} * {b})", "div": "({a} / {b})",
          "max": "fmaxf({a}, {b})", "min": "fminf({a}, {b})", "pow": "powf({a}, {b})"}
TERNARY = {"clamp": "fminf(fmaxf({a}, {b}), {c})", "fma": "fmaf({a}, {b}, {c})",
           "where": "({a} != 0.0f ? {b} : {c})"}


class PointwiseExpr:
    def __add__(self, o): return Binary("add", self, _lift(o))
    def __radd__(self, o): return Binary("add", _lift(o), self)
    def __sub__(self, o): return Binary("sub", self, _lift(o))
    def __rsub__(self, o): return Binary("sub", _lift(o), self)
    def __mul__(self, o): return Binary("mul", self, _lift(o))
    def __rmul__(self, o): return Binary("mul", _lift(o), self)
    def __truediv__(self, o): return Binary("div", self, _lift(o))
    def __neg__(self): return Unary("neg", self)


@dataclass(frozen=True, eq=True)
class Arg(PointwiseExpr):
    index: int


@dataclass(frozen=True, eq=True)
class Const(PointwiseExpr):
    value: float


@dataclass(frozen=True, eq=True)
class Scalar(PointwiseExpr):
    """A runtime scalar passed as a kernel argument: changing its value never triggers a recompile."""
    index: int


@dataclass(frozen=True, eq=True)
class Unary(PointwiseExpr):
    op: str
    x: PointwiseExpr

    def __post_init__(self):
        if self.op not in UNARY:
            raise ValueError(f"unknown unary op {self.op}")


@dataclass(frozen=True, eq=True)
class Binary(PointwiseExpr):
    op: str
    a: PointwiseExpr
    b: PointwiseExpr

    def __post_init__(self):
        if self.op not in BINARY:
            raise ValueError(f"unknown binary op {self.op}")


@dataclass(frozen=True, eq=True)
class Ternary(PointwiseExpr):
    op: str
    a: PointwiseExpr
    b: PointwiseExpr
    c: PointwiseExpr

    def __post_init__(self):
        if self.op not in TERNARY:
            raise ValueError(f"unknown ternary op {self.op}")


def _lift(v) -> PointwiseExpr:
    return v if isinstance(v, PointwiseExpr) else Const(float(v))


class Layout(enum.Enum):
    CONTIGUOUS = "contiguous"   # every tensor dense and same shape: 128-bit accesses
    STRIDED = "strided"         # per-tensor strides (broadcast = stride 0), rank <= 6


CTYPES = {"f32": ("float", 4, 4), "bf16": ("__nv_bfloat16", 2, 8), "f16": ("__half", 2, 8)}


def _emit(e: PointwiseExpr, args: int, scalars: int) -> str:
    if isinstance(e, Arg):
        if not 0 <= e.index < args:
            raise ValueError(f"Arg({e.index}) out of range for {args} inputs")
        return f"v{e.index}"
    if isinstance(e, Scalar):
        if not 0 <= e.index < scalars:
            raise ValueError(f"Scalar({e.index}) out of range for {scalars} scalars")
        return f"s{e.index}"
    if isinstance(e, Const):
        return repr(float(e.value)) + "f" if e.value == e.value and abs(e.value) != float("inf") else \
            ("CUDART_NAN_F" if e.value != e.value else ("CUDART_INF_F" if e.value > 0 else "-CUDART_INF_F"))
    if isinstance(e, Unary):
        return UNARY[e.op].format(x=_emit(e.x, args, scalars))
    if isinstance(e, Binary):
        return BINARY[e.op].format(a=_emit(e.a, args, scalars), b=_emit(e.b, args, scalars))
    if isinstance(e, Ternary):
        return TERNARY[e.op].format(a=_emit(e.a, args, scalars), b=_emit(e.b, args, scalars), c=_emit(e.c, args, scalars))
    raise TypeError(e)


def count_args(e: PointwiseExpr) -> tuple[int, int]:
    """(number of tensor inputs, number of runtime scalars) an expression refers to."""
    if isinstance(e, Arg):
        return e.index + 1, 0
    if isinstance(e, Scalar):
        return 0, e.index + 1
    if isinstance(e, Const):
        return 0, 0
    kids = [getattr(e, n) for n in ("x", "a", "b", "c") if hasattr(e, n)]
    a = s = 0
    for k in kids:
        ka, ks = count_args(k)
        a, s = max(a, ka), max(s, ks)
    return a, s


@dataclass(frozen=True)
class KernelKey:
    digest: str
    dtype: str
    layout: Layout
    n_args: int
    n_scalars: int

    @property
    def entry(self) -> str:
        return f"incin_pw_{self.layout.value}_{self.dtype}_{self.digest[:16]}"


def kernel_key(expr: PointwiseExpr, dtype: str, layout: Layout) -> KernelKey:
    a, s = count_args(expr)
    return KernelKey(hashlib.sha256(repr(expr).encode()).hexdigest(), dtype, layout, a, s)


def render_cuda(expr: PointwiseExpr, dtype: str = "bf16", layout: Layout = Layout.CONTIGUOUS) -> tuple[str, KernelKey]:
    """CUDA C source of one fused kernel.  Signature:
    contiguous: (out, in0..inN-1, s0..sM-1, long long n)
    strided   : (out, in0.., s0.., long long n, int rank, const long long* meta)   meta = shape[6] then strides of
                out and each input, 6 entries each (element strides, 0 = broadcast)."""
    if dtype not in CTYPES:
        raise ValueError(f"unsupported dtype {dtype}")
    key = kernel_key(expr, dtype, layout)
    ct, esz, vec = CTYPES[dtype]
    n_in, n_sc = key.n_args, key.n_scalars
    body = _emit(expr, n_in, n_sc)
    acc = "float"   # 16-bit types compute in fp32
    ins = "".join(f", const {ct}* __restrict__ in{i}" for i in range(n_in))
    scs = "".join(f", float s{i}" for i in range(n_sc))
    ld = {"float": "{p}", "__nv_bfloat16": "__bfloat162float({p})", "__half": "__half2float({p})", "double": "{p}"}[ct]
    st = {"float": "{v}", "__nv_bfloat16": "__float2bfloat16({v})", "__half": "__float2half({v})", "double": "{v}"}[ct]
    head = "#include <cuda_bf16.h>\n#include <cuda_fp16.h>\n#include <math_constants.h>\n"
    if layout is Layout.CONTIGUOUS:
        loads = "".join(f"      Vec a{i} = reinterpret_cast<const Vec*>(in{i})[i];\n" for i in range(n_in))
        unpack = "".join(f"        {acc} v{i} = {ld.format(p=f'a{i}.e[k]')};\n" for i in range(n_in))
        tail = "".join(f"      {acc} v{i} = {ld.format(p=f'in{i}[j]')};\n" for i in range(n_in))
        src = f"""{head}
struct __align__(16) Vec {{ {ct} e[{vec}]; }};
extern "C" __global__ void __launch_bounds__(256) {key.entry}({ct}* __restrict__ out{ins}{scs}, long long n) {{
  const long long nv = n / {vec};
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {{
{loads}      Vec o;
#pragma unroll
      for (int k = 0; k < {vec}; ++k) {{
{unpack}        o.e[k] = {st.format(v=body)};
      }}
      reinterpret_cast<Vec*>(out)[i] = o;
  }}
  for (long long j = nv * {vec} + (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += stride) {{
{tail}      out[j] = {st.format(v=body)};
  }}
}}
"""
    else:
        offs = "".join(f"      long long o{i} = 0;\n" for i in range(n_in))
        walk = "".join(f"        o{i} += c * meta[6 * ({i} + 2) + d];\n" for i in range(n_in))
        vals = "".join(f"      {acc} v{i} = {ld.format(p=f'in{i}[o{i}]')};\n" for i in range(n_in))
        src = f"""{head}
extern "C" __global__ void __launch_bounds__(256) {key.entry}({ct}* __restrict__ out{ins}{scs}, long long n, int rank,
                                                   const long long* __restrict__ meta) {{
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += stride) {{
      long long rem = j, oo = 0;
{offs}      for (int d = rank - 1; d >= 0; --d) {{
        const long long c = rem % meta[d];
        rem /= meta[d];
        oo += c * meta[6 + d];
{walk}      }}
{vals}      out[oo] = {st.format(v=body)};
  }}
}}
"""
    return src, key
