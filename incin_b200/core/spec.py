"""Operation descriptors, validation proofs, tensor metadata and the capability registry.

Counterparts: crates/incin-core/src/exec/spec.rs (MatMulSpec, BroadcastSpec, ReductionSpec,
ReshapeSpec, Conv2dSpec, Pool2dSpec, ReduceOp), exec/proof.rs (``Validated<O>`` + ``ProofLevel``),
exec/meta.rs (TensorMeta, LayoutClass, Alignment), exec/capability.rs and
crates/incin-backends/src/capability.rs (static per-backend rule tables, queried before launch).

A descriptor is plain data describing one operation on tensor *metadata*.  ``validate()`` runs the shape
rule once and returns a :class:`Validated` wrapper; executors (:mod:`incin_b200.backends`) only accept
validated descriptors, so a kernel launch never re-derives or re-checks shapes.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Sequence

from .device import DeviceId, DeviceKind
from .dtype import DTypeId
from .shapes import OperationKind, ShapeError, broadcast_shapes, conv2d_out, reshape_infer, Shape


class LayoutClass(enum.Enum):
    CONTIGUOUS = "contiguous"
    STRIDED = "strided"
    BROADCAST = "broadcast"     # some stride is 0
    SCALAR = "scalar"


@dataclass(frozen=True)
class TensorMeta:
    shape: tuple[int, ...]
    strides: tuple[int, ...]
    dtype: DTypeId
    device: DeviceId
    offset: int = 0
    alignment: int = 16

    @staticmethod
    def contiguous(shape: Sequence[int], dtype: DTypeId, device: DeviceId) -> "TensorMeta":
        strides, acc = [], 1
        for d in reversed(shape):
            strides.append(acc)
            acc *= d
        return TensorMeta(tuple(shape), tuple(reversed(strides)), dtype, device)

    @staticmethod
    def of(t) -> "TensorMeta":
        from .dtype import from_torch
        dev = DeviceId(DeviceKind.CUDA, t.device.index or 0) if t.is_cuda else DeviceId(DeviceKind.CPU)
        align = 16 if t.data_ptr() % 16 == 0 else (t.data_ptr() & -t.data_ptr()) if t.data_ptr() else 16
        return TensorMeta(tuple(t.shape), tuple(t.stride()), from_torch(t.dtype), dev, t.storage_offset(), align)

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    @property
    def layout(self) -> LayoutClass:
        if self.numel == 1:
            return LayoutClass.SCALAR
        if any(s == 0 and d > 1 for s, d in zip(self.strides, self.shape)):
            return LayoutClass.BROADCAST
        dense = TensorMeta.contiguous(self.shape, self.dtype, self.device).strides
        return LayoutClass.CONTIGUOUS if self.strides == dense else LayoutClass.STRIDED

    def max_physical_index(self) -> int:
        """Largest element offset any index can touch: the bound a launch must prove is inside the allocation."""
        return self.offset + sum((d - 1) * abs(s) for d, s in zip(self.shape, self.strides) if d > 0)


class Alignment(enum.IntEnum):
    """Alignment classes of a tensor's first element (crates/incin-core/src/exec/meta.rs): what decides whether the
    vector paths (16-byte accesses, TMA, 32-byte accesses of sm_100) may be used."""
    BYTE = 1
    WORD = 4
    VEC16 = 16
    VEC32 = 32
    LINE = 128

    @staticmethod
    def of_address(addr: int) -> "Alignment":
        for a in (Alignment.LINE, Alignment.VEC32, Alignment.VEC16, Alignment.WORD):
            if addr % int(a) == 0:
                return a
        return Alignment.BYTE


@dataclass(frozen=True)
class AxisMask:
    """The axes a reduction removes, as a bit mask over at most MAX_RANK axes (exec/spec.rs ``AxisMask``)."""
    bits: int
    rank: int

    @staticmethod
    def from_axes(axes: Sequence[int], rank: int) -> "AxisMask":
        if not 0 < rank <= 8:
            raise ShapeError(OperationKind.REDUCE, f"rank {rank} out of range")
        bits = 0
        for a in axes:
            if not -rank <= a < rank:
                raise ShapeError(OperationKind.REDUCE, f"axis {a} out of range for rank {rank}")
            a %= rank
            if bits >> a & 1:
                raise ShapeError(OperationKind.REDUCE, f"axis {a} named twice")
            bits |= 1 << a
        return AxisMask(bits, rank)

    @staticmethod
    def all(rank: int) -> "AxisMask":
        return AxisMask((1 << rank) - 1, rank)

    def contains(self, axis: int) -> bool:
        return bool(self.bits >> (axis % self.rank) & 1)

    def axes(self) -> tuple[int, ...]:
        return tuple(a for a in range(self.rank) if self.bits >> a & 1)

    def __len__(self) -> int:
        return bin(self.bits).count("1")

    def reduced_shape(self, shape: Sequence[int], keepdim: bool = False) -> tuple[int, ...]:
        if len(shape) != self.rank:
            raise ShapeError(OperationKind.REDUCE, f"mask of rank {self.rank} applied to shape {tuple(shape)}")
        return tuple(1 if self.contains(a) else d for a, d in enumerate(shape) if keepdim or not self.contains(a))


@dataclass(frozen=True)
class TensorHandle:
    """What a backend needs to launch on a tensor without owning it: metadata, address, alignment class
    (exec/request.rs ``TensorHandle``)."""
    meta: TensorMeta
    address: int
    alignment: Alignment

    @staticmethod
    def of(t) -> "TensorHandle":
        return TensorHandle(TensorMeta.of(t), int(t.data_ptr()), Alignment.of_address(int(t.data_ptr())))


@dataclass(frozen=True)
class ExecutionContext:
    """Where and how a validated op runs: device, stream, and the execution / precision policies in force
    (exec/context.rs:24).  ``current()`` snapshots the ambient state."""
    device: DeviceId
    stream: int
    policy: object
    precision: object

    @staticmethod
    def current(device=None) -> "ExecutionContext":
        import torch
        from .policy import current_policy
        try:
            from .policy import current_precision
            precision = current_precision()
        except ImportError:
            precision = None
        if device is None:
            device = DeviceId(DeviceKind.CUDA, torch.cuda.current_device()) if torch.cuda.is_available() else DeviceId(DeviceKind.CPU)
        stream = torch.cuda.current_stream().cuda_stream if device.kind is DeviceKind.CUDA and torch.cuda.is_available() else 0
        return ExecutionContext(device, int(stream), current_policy(), precision)


class ProofLevel(enum.Enum):
    STATIC = "static"          # every extent was known when the descriptor was built
    RANKED = "ranked"          # rank known, some extents runtime
    DYNAMIC = "dynamic"

    def meet(self, other: "ProofLevel") -> "ProofLevel":
        order = [ProofLevel.STATIC, ProofLevel.RANKED, ProofLevel.DYNAMIC]
        return order[max(order.index(self), order.index(other))]


class ReduceOp(enum.Enum):
    SUM = "sum"
    MEAN = "mean"
    MAX = "max"
    MIN = "min"
    PROD = "prod"


@dataclass(frozen=True)
class MatMulSpec:
    a: TensorMeta
    b: TensorMeta
    kind = OperationKind.MATMUL

    def output_shape(self) -> tuple[int, ...]:
        if len(self.a.shape) < 2 or len(self.b.shape) < 2:
            raise ShapeError(OperationKind.MATMUL, "operands need rank >= 2")
        if self.a.shape[-1] != self.b.shape[-2]:
            raise ShapeError(OperationKind.MATMUL, f"inner extents {self.a.shape[-1]} and {self.b.shape[-2]} differ")
        batch = tuple(d.size for d in broadcast_shapes(self.a.shape[:-2], self.b.shape[:-2]).dims)
        return batch + (self.a.shape[-2], self.b.shape[-1])


@dataclass(frozen=True)
class BroadcastSpec:
    a: TensorMeta
    b: TensorMeta
    kind = OperationKind.BROADCAST

    def output_shape(self) -> tuple[int, ...]:
        return tuple(d.size for d in broadcast_shapes(self.a.shape, self.b.shape).dims)


@dataclass(frozen=True)
class ReductionSpec:
    x: TensorMeta
    op: ReduceOp
    axes: tuple[int, ...]
    keepdim: bool = False
    kind = OperationKind.REDUCE

    def output_shape(self) -> tuple[int, ...]:
        rank = len(self.x.shape)
        axes = set()
        for a in self.axes:
            if not -rank <= a < rank:
                raise ShapeError(OperationKind.REDUCE, f"axis {a} out of range for rank {rank}")
            axes.add(a % rank)
        if len(axes) != len(self.axes):
            raise ShapeError(OperationKind.REDUCE, "duplicate reduction axis")
        out = []
        for i, d in enumerate(self.x.shape):
            if i in axes:
                if self.keepdim:
                    out.append(1)
            else:
                out.append(d)
        return tuple(out)


@dataclass(frozen=True)
class ReshapeSpec:
    x: TensorMeta
    target: tuple[int, ...]
    kind = OperationKind.RESHAPE

    def output_shape(self) -> tuple[int, ...]:
        return reshape_infer(self.x.numel, self.target)


@dataclass(frozen=True)
class Conv2dSpec:
    x: TensorMeta       # [N, C, H, W]
    w: TensorMeta       # [O, C/groups, KH, KW]
    stride: tuple[int, int] = (1, 1)
    padding: tuple[int, int] = (0, 0)
    dilation: tuple[int, int] = (1, 1)
    groups: int = 1
    kind = OperationKind.CONV

    def output_shape(self) -> tuple[int, ...]:
        if len(self.x.shape) != 4 or len(self.w.shape) != 4:
            raise ShapeError(OperationKind.CONV, "conv2d takes NCHW input and OIHW weight")
        n, c, h, w = self.x.shape
        o, ci, kh, kw = self.w.shape
        if c % self.groups or o % self.groups or ci * self.groups != c:
            raise ShapeError(OperationKind.CONV, f"channels {c}/{ci} do not match groups={self.groups}")
        oh, ow = conv2d_out(h, w, (kh, kw), self.stride, self.padding, self.dilation)
        return (n, o, oh, ow)


@dataclass(frozen=True)
class Pool2dSpec:
    x: TensorMeta
    kernel: tuple[int, int]
    stride: tuple[int, int]
    padding: tuple[int, int] = (0, 0)
    kind = OperationKind.POOL

    def output_shape(self) -> tuple[int, ...]:
        if len(self.x.shape) != 4:
            raise ShapeError(OperationKind.POOL, "pool2d takes NCHW input")
        n, c, h, w = self.x.shape
        oh, ow = conv2d_out(h, w, self.kernel, self.stride, self.padding)
        return (n, c, oh, ow)


@dataclass(frozen=True)
class Validated:
    """A descriptor whose shape rule has run; carries the output shape and the strength of the proof."""
    descriptor: object
    output_shape: tuple[int, ...]
    proof_level: ProofLevel

    def audit(self) -> None:
        """Re-run the rule (debug aid): raises if the stored result no longer matches."""
        if tuple(self.descriptor.output_shape()) != self.output_shape:
            raise ShapeError(self.descriptor.kind, "validated descriptor failed its audit")


def validate(descriptor, proof: ProofLevel = ProofLevel.DYNAMIC) -> Validated:
    return Validated(descriptor, tuple(descriptor.output_shape()), proof)


# --------------------------------------------------------------------------------------------- capability
class SupportLevel(enum.Enum):
    NATIVE = "native"            # one hand-written kernel
    COMPOSED = "composed"        # built from several native kernels
    UNSUPPORTED = "unsupported"

    @property
    def is_supported(self) -> bool:
        return self is not SupportLevel.UNSUPPORTED


@dataclass(frozen=True)
class CapabilityQuery:
    op: str
    dtype: DTypeId
    device: DeviceKind
    layout: LayoutClass = LayoutClass.CONTIGUOUS


@dataclass(frozen=True)
class CapabilityRule:
    op: str
    dtypes: tuple[DTypeId, ...]
    level: SupportLevel
    implementation: str
    note: str = ""


_F = (DTypeId.BF16, DTypeId.F16, DTypeId.F32, DTypeId.F64)
_ALL = _F + (DTypeId.U8, DTypeId.U32, DTypeId.I64)

CPU_CAPABILITIES: tuple[CapabilityRule, ...] = tuple(
    CapabilityRule(op, _ALL if op in ("reshape", "transpose", "concat", "gather", "index_select") else _F,
                   SupportLevel.NATIVE, "torch-cpu / libincin_host oracle")
    for op in ("matmul", "bmm", "addmm", "add", "sub", "mul", "div", "unary", "softmax", "layer_norm", "rms_norm",
               "embedding", "cross_entropy", "sdpa", "conv1d", "conv2d", "conv_transpose2d", "max_pool2d", "avg_pool2d",
               "adaptive_avg_pool2d", "batch_norm", "sum", "mean",
               "max", "min", "argmax", "topk", "argsort", "cumsum", "reshape", "transpose", "concat", "gather",
               "index_select", "adamw", "sgd", "rope", "swiglu", "dropout")
) + (CapabilityRule("quantize_q8_0", (DTypeId.F32,), SupportLevel.NATIVE, "libincin_host oracle"),
     CapabilityRule("quantized_matmul", (DTypeId.Q8_0,), SupportLevel.COMPOSED, "dequantize + matmul"))

_BF = (DTypeId.BF16,)
CUDA_CAPABILITIES: tuple[CapabilityRule, ...] = (
    CapabilityRule("matmul", _BF, SupportLevel.NATIVE, "gemm_tcgen05 (TMA + tcgen05.mma + TMEM)"),
    CapabilityRule("bmm", _BF, SupportLevel.NATIVE, "gemm_tcgen05 batched (4-D tensor maps)"),
    CapabilityRule("addmm", _BF, SupportLevel.NATIVE, "gemm_tcgen05 bias/residual epilogue"),
    CapabilityRule("matmul", (DTypeId.F16,), SupportLevel.NATIVE, "gemm_tcgen05, fp16 operands, fp32 accumulate and output"),
    CapabilityRule("matmul", (DTypeId.F32,), SupportLevel.NATIVE, "gemm_tcgen05 kind::tf32 (MathMode.FAST; else cuBLAS fp32)"),
    CapabilityRule("sdpa", _BF, SupportLevel.NATIVE, "flash_fwd/flash_bwd (online softmax on tcgen05)"),
    CapabilityRule("layer_norm", _BF, SupportLevel.NATIVE, "norm_fwd/norm_bwd"),
    CapabilityRule("rms_norm", _BF, SupportLevel.NATIVE, "norm_fwd/norm_bwd<RMS>"),
    CapabilityRule("embedding", _BF, SupportLevel.NATIVE, "embedding_fwd/bwd"),
    CapabilityRule("cross_entropy", _BF, SupportLevel.NATIVE, "xent_fwd/bwd (online log-sum-exp)"),
    CapabilityRule("linear_cross_entropy", _BF, SupportLevel.NATIVE, "gemm_tcgen05 + xent_fused (loss and gradient in one pass)"),
    CapabilityRule("softmax", _BF + (DTypeId.F32,), SupportLevel.NATIVE, "fused pointwise/row kernels"),
    CapabilityRule("unary", _F, SupportLevel.NATIVE, "NVRTC-fused pointwise chain (sm_100a)"),
    CapabilityRule("add", _F, SupportLevel.NATIVE, "NVRTC-fused pointwise chain (sm_100a)"),
    CapabilityRule("sub", _F, SupportLevel.NATIVE, "NVRTC-fused pointwise chain (sm_100a)"),
    CapabilityRule("mul", _F, SupportLevel.NATIVE, "NVRTC-fused pointwise chain (sm_100a)"),
    CapabilityRule("div", _F, SupportLevel.NATIVE, "NVRTC-fused pointwise chain (sm_100a)"),
    CapabilityRule("sum", _F, SupportLevel.NATIVE, "reduce kernels"),
    CapabilityRule("mean", _F, SupportLevel.NATIVE, "reduce kernels"),
    CapabilityRule("max", _F, SupportLevel.NATIVE, "reduce kernels"),
    CapabilityRule("min", _F, SupportLevel.NATIVE, "reduce kernels"),
    CapabilityRule("adamw", (DTypeId.F32,), SupportLevel.NATIVE, "adamw_flat / dp_reduce_adamw"),
    CapabilityRule("sgd", (DTypeId.F32,), SupportLevel.NATIVE, "sgd_flat"),
    CapabilityRule("rope", _BF, SupportLevel.NATIVE, "rope"),
    CapabilityRule("swiglu", _BF, SupportLevel.NATIVE, "swiglu_fwd/bwd"),
    CapabilityRule("dropout", _BF, SupportLevel.NATIVE, "philox dropout"),
    CapabilityRule("quantize_q8_0", (DTypeId.F32,), SupportLevel.NATIVE, "q8_0 quantize/dequantize"),
    CapabilityRule("conv2d", _BF, SupportLevel.COMPOSED, "im2col + gemm_tcgen05"),
    CapabilityRule("conv1d", _BF, SupportLevel.COMPOSED, "im2col (height 1) + gemm_tcgen05"),
    CapabilityRule("conv_transpose2d", _BF, SupportLevel.COMPOSED, "gemm_tcgen05 + col2im (gather, no atomics)"),
    CapabilityRule("adaptive_avg_pool2d", _BF + (DTypeId.F32,), SupportLevel.NATIVE, "adaptive_avgpool2d fwd/bwd"),
    CapabilityRule("argmax", _BF + (DTypeId.F32,), SupportLevel.NATIVE, "reduce kernels (index output)"),
    CapabilityRule("cumsum", _BF + (DTypeId.F32,), SupportLevel.NATIVE, "block scan"),
    CapabilityRule("max_pool2d", _BF + (DTypeId.F32,), SupportLevel.NATIVE, "maxpool2d fwd (argmax kept) / gather bwd"),
    CapabilityRule("avg_pool2d", _BF + (DTypeId.F32,), SupportLevel.NATIVE, "avgpool2d fwd/bwd"),
    CapabilityRule("batch_norm", _BF + (DTypeId.F32,), SupportLevel.NATIVE, "batchnorm train fwd/bwd + eval"),
    CapabilityRule("concat", _ALL, SupportLevel.NATIVE, "strided copy"),
    CapabilityRule("gather", _BF + (DTypeId.F32, DTypeId.U32), SupportLevel.NATIVE, "gather_last / scatter_last"),
    CapabilityRule("index_select", _BF + (DTypeId.F32, DTypeId.U32), SupportLevel.NATIVE, "gather_rows / scatter_add_rows"),
    CapabilityRule("quantized_matmul", (DTypeId.Q8_0,), SupportLevel.COMPOSED, "dequantize_q8_0 (bf16) + gemm_tcgen05"),
    CapabilityRule("reshape", _ALL, SupportLevel.NATIVE, "view"),
    CapabilityRule("transpose", _ALL, SupportLevel.NATIVE, "view (GEMM reads either major)"),
)


class CapabilityRegistry:
    def __init__(self, device: DeviceKind, rules: Sequence[CapabilityRule]):
        self.device, self.rules = device, tuple(rules)

    def query(self, q: CapabilityQuery) -> CapabilityRule:
        best = None
        for r in self.rules:
            if r.op == q.op and q.dtype in r.dtypes:
                if best is None or (r.level is SupportLevel.NATIVE and best.level is not SupportLevel.NATIVE):
                    best = r
        return best or CapabilityRule(q.op, (q.dtype,), SupportLevel.UNSUPPORTED, "-",
                                      f"no {self.device.value} kernel for {q.op}/{q.dtype.value}")

    def supports(self, op: str, dtype: DTypeId) -> bool:
        return self.query(CapabilityQuery(op, dtype, self.device)).level.is_supported


REGISTRIES = {DeviceKind.CPU: CapabilityRegistry(DeviceKind.CPU, CPU_CAPABILITIES),
              DeviceKind.CUDA: CapabilityRegistry(DeviceKind.CUDA, CUDA_CAPABILITIES)}


def capability_table_markdown() -> str:
    """The generated capability matrix (the reference keeps docs/capabilities.md in sync the same way)."""
    ops = sorted({r.op for reg in REGISTRIES.values() for r in reg.rules})
    lines = ["| op | cpu | cuda (sm_100a) |", "|---|---|---|"]
    for op in ops:
        cells = []
        for kind in (DeviceKind.CPU, DeviceKind.CUDA):
            rs = [r for r in REGISTRIES[kind].rules if r.op == op]
            cells.append("; ".join(f"{r.level.value} [{','.join(d.value for d in r.dtypes)}]" for r in rs) or "unsupported")
        lines.append(f"| {op} | {cells[0]} | {cells[1]} |")
    return "\n".join(lines) + "\n"
