"""WGSL and MSL text renderers of the pointwise expression AST.

Counterpart of ``render_wgsl`` / ``render_msl`` in crates/incin-backends/src/codegen/pointwise.rs:181-291: the same
expression that :func:`incin_b200.codegen.pointwise.render_cuda` turns into a CUDA kernel is emitted as a WGSL compute
shader (storage buffers ``in0..`` / ``out_data``, one invocation per element, bounds check against ``arrayLength``) or as
an MSL kernel (``device const T* inN [[buffer(N)]]``, ``thread_position_in_grid``).  These are source emitters only:
this framework executes on sm_100a and neither shader language has a runtime here, so the text is checked by tests
that look for the constructs a consumer needs (bindings, entry point, the expression itself), as the reference's own
tests do.  Runtime scalars become a uniform / constant buffer after the tensors; 16-bit storage computes in f32.
"""
from __future__ import annotations

from .pointwise import Arg, Binary, Const, PointwiseExpr, Scalar, Ternary, Unary, count_args

WGSL_TYPES = {"f32": "f32", "f16": "f16", "bf16": "f16", "u32": "u32", "i64": "i32"}
MSL_TYPES = {"f32": "float", "f16": "half", "bf16": "half", "u32": "uint", "i64": "long"}

_GELU_TANH = "(0.5{f} * {x} * (1.0{f} + tanh(0.79788456{f} * ({x} + 0.044715{f} * {x} * {x} * {x}))))"

# op -> (WGSL, MSL); {x} / {a} {b} {c} are the rendered operands, {f} the float-literal suffix of the target
_UNARY = {
    "relu": ("max({x}, 0.0)", "fmax({x}, 0.0f)"),
    "step": ("select(0.0, 1.0, {x} > 0.0)", "({x} > 0.0f ? 1.0f : 0.0f)"),
    "sigmoid": ("(1.0 / (1.0 + exp(-({x}))))", "(1.0f / (1.0f + exp(-({x}))))"),
    "tanh": ("tanh({x})", "tanh({x})"),
    "swish": ("({x} / (1.0 + exp(-({x}))))", "({x} / (1.0f + exp(-({x}))))"),
    "softplus": ("log(1.0 + exp({x}))", "log(1.0f + exp({x}))"),
    "elu": ("select(exp({x}) - 1.0, {x}, {x} > 0.0)", "({x} > 0.0f ? {x} : exp({x}) - 1.0f)"),
    # WGSL and MSL have no erf: both targets use the tanh form, which is what the reference's shaders compute
    "gelu": (_GELU_TANH.format(x="{x}", f=""), _GELU_TANH.format(x="{x}", f="f")),
    "gelu_tanh": (_GELU_TANH.format(x="{x}", f=""), _GELU_TANH.format(x="{x}", f="f")),
    "exp": ("exp({x})", "exp({x})"), "log": ("log({x})", "log({x})"), "sqrt": ("sqrt({x})", "sqrt({x})"),
    "rsqrt": ("inverseSqrt({x})", "rsqrt({x})"), "neg": ("-({x})", "-({x})"), "abs": ("abs({x})", "fabs({x})"),
    "sign": ("sign({x})", "sign({x})"),
    "mish": ("({x} * tanh(log(1.0 + exp({x}))))", "({x} * tanh(log(1.0f + exp({x}))))"),
    "recip": ("(1.0 / ({x}))", "(1.0f / ({x}))"), "square": ("(({x}) * ({x}))", "(({x}) * ({x}))"),
    "sin": ("sin({x})", "sin({x})"), "cos": ("cos({x})", "cos({x})"),
    "floor": ("floor({x})", "floor({x})"), "ceil": ("ceil({x})", "ceil({x})"),
}
_BINARY = {
    "add": ("({a} + {b})",) * 2, "sub": ("({a} - {b})",) * 2, "mul": ("({a} * {b})",) * 2, "div": ("({a} / {b})",) * 2,
    "max": ("max({a}, {b})", "fmax({a}, {b})"), "min": ("min({a}, {b})", "fmin({a}, {b})"),
    "pow": ("pow({a}, {b})", "pow({a}, {b})"),
}
_TERNARY = {
    "clamp": ("clamp({a}, {b}, {c})", "clamp({a}, {b}, {c})"),
    "fma": ("fma({a}, {b}, {c})", "fma({a}, {b}, {c})"),
    "where": ("select({c}, {b}, {a} != 0.0)", "({a} != 0.0f ? {b} : {c})"),
}


def _lit(v: float, target: int) -> str:
    if v != v or v in (float("inf"), float("-inf")):
        raise ValueError("non-finite constants have no literal in WGSL / MSL")
    return repr(float(v)) + ("f" if target == 1 else "")


def _expr(e: PointwiseExpr, target: int, n_args: int, n_scalars: int) -> str:
    if isinstance(e, Arg):
        if not 0 <= e.index < n_args:
            raise ValueError(f"Arg({e.index}) out of range for {n_args} inputs")
        return f"val{e.index}"
    if isinstance(e, Scalar):
        if not 0 <= e.index < n_scalars:
            raise ValueError(f"Scalar({e.index}) out of range for {n_scalars} scalars")
        return f"scalars.s{e.index}" if target == 0 else f"scalars[{e.index}]"
    if isinstance(e, Const):
        return _lit(e.value, target)
    if isinstance(e, Unary):
        return _UNARY[e.op][target].format(x=_expr(e.x, target, n_args, n_scalars))
    if isinstance(e, Binary):
        return _BINARY[e.op][target].format(a=_expr(e.a, target, n_args, n_scalars), b=_expr(e.b, target, n_args, n_scalars))
    if isinstance(e, Ternary):
        return _TERNARY[e.op][target].format(a=_expr(e.a, target, n_args, n_scalars), b=_expr(e.b, target, n_args, n_scalars),
                                              c=_expr(e.c, target, n_args, n_scalars))
    raise TypeError(e)


def render_wgsl(expr: PointwiseExpr, dtype: str = "f32", *, workgroup_size: int = 256, scalar_broadcast: int | None = None) -> str:
    """WGSL compute shader; ``scalar_broadcast = i`` reads input ``i`` as a one-element buffer (``in{i}[0]``), the
    reference's ScalarBroadcast layout."""
    if dtype not in WGSL_TYPES:
        raise ValueError(f"unsupported dtype {dtype}")
    n_in, n_sc = count_args(expr)
    t = WGSL_TYPES[dtype]
    out = ["// Generated by incin_b200.codegen (WGSL)"]
    if t == "f16":
        out.append("enable f16;")
    out.append("")
    for i in range(n_in):
        out.append(f"@group(0) @binding({i}) var<storage, read> in{i}: array<{t}>;")
    out.append(f"@group(0) @binding({n_in}) var<storage, read_write> out_data: array<{t}>;")
    if n_sc:
        fields = " ".join(f"s{i}: f32," for i in range(n_sc))
        out.append(f"struct Scalars {{ {fields} }}")
        out.append(f"@group(0) @binding({n_in + 1}) var<uniform> scalars: Scalars;")
    out += ["", f"@compute @workgroup_size({workgroup_size}, 1, 1)",
            "fn main(@builtin(global_invocation_id) global_id: vec3<u32>) {", "    let idx = global_id.x;",
            "    if (idx >= arrayLength(&out_data)) { return; }"]
    for i in range(n_in):
        src = f"in{i}[0]" if scalar_broadcast == i else f"in{i}[idx]"
        out.append(f"    let val{i} = f32({src});")
    out.append(f"    out_data[idx] = {t}({_expr(expr, 0, n_in, n_sc)});")
    out.append("}")
    return "\n".join(out) + "\n"


def render_msl(expr: PointwiseExpr, dtype: str = "f32", *, name: str = "incin_pointwise", scalar_broadcast: int | None = None) -> str:
    """Metal Shading Language kernel of the same expression."""
    if dtype not in MSL_TYPES:
        raise ValueError(f"unsupported dtype {dtype}")
    n_in, n_sc = count_args(expr)
    t = MSL_TYPES[dtype]
    out = ["// Generated by incin_b200.codegen (MSL)", "#include <metal_stdlib>", "using namespace metal;", "", f"kernel void {name}("]
    for i in range(n_in):
        out.append(f"    device const {t}* in{i} [[buffer({i})]],")
    out.append(f"    device {t}* out_data [[buffer({n_in})]],")
    if n_sc:
        out.append(f"    constant float* scalars [[buffer({n_in + 1})]],")
    out.append(f"    constant uint& n [[buffer({n_in + 1 + (1 if n_sc else 0)})]],")
    out.append("    uint idx [[thread_position_in_grid]]\n) {")
    out.append("    if (idx >= n) { return; }")
    for i in range(n_in):
        src = f"in{i}[0]" if scalar_broadcast == i else f"in{i}[idx]"
        out.append(f"    const float val{i} = static_cast<float>({src});")
    out.append(f"    out_data[idx] = static_cast<{t}>({_expr(expr, 1, n_in, n_sc)});")
    out.append("}")
    return "\n".join(out) + "\n"
