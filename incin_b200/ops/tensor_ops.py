"""Reductions, data-movement ops, pooling, batch norm and convolution helpers on the native sm_100a kernels.

Counterparts: ``ReductionOps`` (20 methods) and the shape half of ``TensorOps`` (crates/incin-core/src/tensor/
backend.rs:587-646, 345-530), ``ModuleOps`` pooling / batch_norm / conv (backend.rs:651-739).  Every function takes
and returns torch tensors.  On CUDA with bf16 or fp32 data the native kernel runs (and raises if the library is
missing); on CPU the same semantics come from PyTorch CPU math, which is what the tests compare the kernels with.
Forward/backward pairs that training needs are wrapped in autograd functions at the bottom.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as nat

c_int, c_ll, c_float, c_void_p = C.c_int, C.c_longlong, C.c_float, C.c_void_p


class ConvGeom(C.Structure):
    _fields_ = [(n, c_int) for n in ("N", "C", "H", "W", "KH", "KW", "stride_h", "stride_w", "pad_h", "pad_w", "dil_h", "dil_w")]


nat.register_cuda_signatures({
    "incin_reduce_axis": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_ll, c_int, c_int, c_void_p]),
    "incin_reduce_all": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p]),
    "incin_cumsum": (c_int, [c_void_p, c_void_p, c_ll, c_ll, c_ll, c_int, c_void_p]),
    "incin_strided_copy": (c_int, [c_void_p, c_void_p, c_int, C.POINTER(c_ll), C.POINTER(c_ll), C.POINTER(c_ll), c_int, c_void_p]),
    "incin_gather_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_ll, c_int, c_void_p, c_void_p]),
    "incin_scatter_add_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_ll, c_int, c_void_p, c_void_p]),
    "incin_gather_last": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_ll, c_int, c_void_p, c_void_p]),
    "incin_scatter_last": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_ll, c_int, c_void_p, c_void_p]),
    "incin_masked_fill": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_ll, c_int, c_void_p]),
    "incin_where": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p]),
    "incin_tri": (c_int, [c_void_p, c_void_p, c_ll, c_ll, c_ll, c_ll, c_int, c_int, c_void_p]),
    "incin_conv_out_hw": (c_int, [C.POINTER(ConvGeom), C.POINTER(c_int), C.POINTER(c_int)]),
    "incin_im2col": (c_int, [c_void_p, c_void_p, C.POINTER(ConvGeom), c_int, c_void_p]),
    "incin_col2im": (c_int, [c_void_p, c_void_p, C.POINTER(ConvGeom), c_int, c_void_p]),
    "incin_maxpool2d_fwd": (c_int, [c_void_p, c_void_p, c_void_p, C.POINTER(ConvGeom), c_int, c_void_p]),
    "incin_maxpool2d_bwd": (c_int, [c_void_p, c_void_p, c_void_p, C.POINTER(ConvGeom), c_int, c_void_p]),
    "incin_avgpool2d": (c_int, [c_void_p, c_void_p, C.POINTER(ConvGeom), c_int, c_int, c_void_p]),
    "incin_adaptive_avgpool2d": (c_int, [c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "incin_softmax_lastdim_fwd": (c_int, [c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p]),
    "incin_softmax_lastdim_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p]),
    "incin_batchnorm_train_fwd": (c_int, [c_void_p] * 8 + [c_int, c_int, c_ll, c_float, c_float, c_int, c_void_p]),
    "incin_batchnorm_eval": (c_int, [c_void_p] * 6 + [c_int, c_int, c_ll, c_float, c_int, c_void_p]),
    "incin_batchnorm_bwd": (c_int, [c_void_p] * 8 + [c_int, c_int, c_ll, c_int, c_void_p]),
    "incin_quantize_q8_0": (c_int, [c_void_p, c_void_p, c_ll, c_int, c_void_p]),
    "incin_dequantize_q8_0": (c_int, [c_void_p, c_void_p, c_ll, c_int, c_void_p]),
    "incin_embedding_bwd_sorted": (c_int, [c_void_p] * 4 + [c_ll, c_void_p, c_void_p, c_ll, c_int, c_int, c_ll, c_void_p]),
})

_OPS = {"sum": 0, "mean": 1, "max": 2, "min": 3, "prod": 4, "argmax": 5, "argmin": 6}


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype in (torch.bfloat16, torch.float32)


def _s() -> int:
    return nat.stream_ptr()


def _bf(t: torch.Tensor) -> int:
    return int(t.dtype == torch.bfloat16)


_err: dict[int, torch.Tensor] = {}


def _err_flag(dev: torch.device) -> torch.Tensor:
    i = dev.index if dev.index is not None else torch.cuda.current_device()
    if i not in _err:
        _err[i] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _err[i]


def check_indices(dev: torch.device) -> None:
    """Synchronising check: raises if an indexed op since the last check met an out-of-range index (it was skipped)."""
    f = _err_flag(dev)
    if int(f.item()):
        f.zero_()
        raise IndexError("an index passed to gather/scatter/index_select was out of range")


# ---------------------------------------------------------------------------------------------------- reductions
def reduce(x: torch.Tensor, op: str, dim: int | None = None, keepdim: bool = False) -> torch.Tensor:
    """``sum / mean / max / min / prod / argmax / argmin`` over one axis, or over everything when ``dim`` is None."""
    code = _OPS[op]
    arg = code >= 5
    if not _native(x):
        f = getattr(torch, op if not arg else op)
        if dim is None:
            return f(x)
        r = f(x, dim=dim, keepdim=keepdim)
        return r if arg or op in ("sum", "mean", "prod") else r.values
    x = x.contiguous()
    if dim is None:
        out = torch.empty((), dtype=torch.float32, device=x.device)
        idx = torch.empty((), dtype=torch.int64, device=x.device) if arg else None
        nat.check(nat.cuda().incin_reduce_all(x.data_ptr(), out.data_ptr(), nat.ptr(idx), x.numel(), code, _bf(x), _s()),
                  "reduce_all")
        return idx if arg else out.to(x.dtype)
    dim = dim % x.dim()
    outer = 1
    for d in x.shape[:dim]:
        outer *= d
    inner = 1
    for d in x.shape[dim + 1:]:
        inner *= d
    shape = list(x.shape)
    shape[dim] = 1
    out = torch.empty(shape, dtype=torch.int64 if arg else x.dtype, device=x.device)
    nat.check(nat.cuda().incin_reduce_axis(x.data_ptr(), None if arg else out.data_ptr(), out.data_ptr() if arg else None,
                                          outer, x.shape[dim], inner, code, _bf(x), _s()), "reduce_axis")
    return out if keepdim else out.squeeze(dim)


def var(x: torch.Tensor, dim: int, unbiased: bool = True, keepdim: bool = False) -> torch.Tensor:
    m = reduce(x.float(), "mean", dim, True)
    d = (x.float() - m)
    n = x.shape[dim]
    v = reduce(d * d, "sum", dim, keepdim) / max(1, n - (1 if unbiased else 0))
    return v.to(x.dtype)


def std(x, dim, unbiased=True, keepdim=False):
    return var(x, dim, unbiased, keepdim).sqrt()


def norm(x: torch.Tensor) -> torch.Tensor:
    return reduce((x.float() * x.float()), "sum").sqrt().to(x.dtype)


def cumsum(x: torch.Tensor, dim: int) -> torch.Tensor:
    if not _native(x):
        return torch.cumsum(x, dim)
    x = x.contiguous()
    dim = dim % x.dim()
    outer = 1
    for d in x.shape[:dim]:
        outer *= d
    inner = 1
    for d in x.shape[dim + 1:]:
        inner *= d
    out = torch.empty_like(x)
    nat.check(nat.cuda().incin_cumsum(x.data_ptr(), out.data_ptr(), outer, x.shape[dim], inner, _bf(x), _s()), "cumsum")
    return out


# ---------------------------------------------------------------------------------------------------- movement
def _arr(vals):
    return (c_ll * len(vals))(*vals)


def strided_copy(src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    """``dst[...] = src[...]`` for two views of the same shape (any strides, broadcast strides allowed on ``src``)."""
    if tuple(src.shape) != tuple(dst.shape):
        src = src.expand(dst.shape)
    if not (src.is_cuda and dst.is_cuda) or src.dtype != dst.dtype or src.dim() > 6 or src.dim() == 0 or src.numel() == 0:
        dst.copy_(src)
        return dst
    nat.check(nat.cuda().incin_strided_copy(src.data_ptr(), dst.data_ptr(), src.dim(), _arr(list(src.shape)),
                                           _arr(list(src.stride())), _arr(list(dst.stride())), src.element_size(), _s()),
              "strided_copy")
    return dst


def materialize(view: torch.Tensor) -> torch.Tensor:
    """Dense copy of any view (transpose, narrow, broadcast, ...)."""
    out = torch.empty(view.shape, dtype=view.dtype, device=view.device)
    return strided_copy(view, out)


def transpose(x: torch.Tensor, a: int, b: int) -> torch.Tensor:
    return materialize(x.transpose(a, b))


def narrow(x: torch.Tensor, dim: int, start: int, length: int) -> torch.Tensor:
    return materialize(x.narrow(dim, start, length))


def paste(dst: torch.Tensor, src: torch.Tensor, dim: int, start: int) -> torch.Tensor:
    """Write ``src`` into ``dst`` at ``start`` along ``dim`` (in place; the adjoint of ``narrow``)."""
    strided_copy(src, dst.narrow(dim, start, src.shape[dim]))
    return dst


def broadcast_to(x: torch.Tensor, shape) -> torch.Tensor:
    return materialize(x.expand(shape))


def concat(tensors, dim: int = 0) -> torch.Tensor:
    shape = list(tensors[0].shape)
    shape[dim] = sum(t.shape[dim] for t in tensors)
    out = torch.empty(shape, dtype=tensors[0].dtype, device=tensors[0].device)
    off = 0
    for t in tensors:
        paste(out, t, dim, off)
        off += t.shape[dim]
    return out


def pad(x: torch.Tensor, pads: list[tuple[int, int]], value: float = 0.0) -> torch.Tensor:
    """``pads[d] = (before, after)`` per axis."""
    shape = [s + a + b for s, (a, b) in zip(x.shape, pads)]
    out = torch.full(shape, value, dtype=x.dtype, device=x.device)
    view = out
    for d, (a, _) in enumerate(pads):
        view = view.narrow(d, a, x.shape[d])
    strided_copy(x, view)
    return out


def index_select(x: torch.Tensor, dim: int, index: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda or x.element_size() not in (2, 4):
        return torch.index_select(x, dim, index)
    if dim % x.dim() != 0:
        return transpose(index_select(transpose(x, 0, dim), 0, index), 0, dim)
    x = x.contiguous()
    row = x.numel() // x.shape[0] if x.shape[0] else 0
    out = torch.empty((index.numel(),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    nat.check(nat.cuda().incin_gather_rows(x.data_ptr(), index.contiguous().data_ptr(), out.data_ptr(), index.numel(), row,
                                          x.shape[0], x.element_size(), _err_flag(x.device).data_ptr(), _s()), "gather_rows")
    return out


def index_add_rows(dst_f32: torch.Tensor, index: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """``dst[index[i]] += src[i]`` (fp32 destination; the adjoint of ``index_select`` along axis 0)."""
    if not dst_f32.is_cuda:
        return dst_f32.index_add_(0, index, src.float())
    src = src.contiguous()
    row = src.numel() // max(1, src.shape[0])
    nat.check(nat.cuda().incin_scatter_add_rows(src.data_ptr(), index.contiguous().data_ptr(), dst_f32.data_ptr(), index.numel(),
                                               row, dst_f32.shape[0], _bf(src), _err_flag(src.device).data_ptr(), _s()),
              "scatter_add_rows")
    return dst_f32


def gather_last(x: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda or x.element_size() not in (2, 4):
        return torch.gather(x, -1, index)
    x, index = x.contiguous(), index.contiguous()
    rows = x.numel() // x.shape[-1]
    out = torch.empty(index.shape, dtype=x.dtype, device=x.device)
    nat.check(nat.cuda().incin_gather_last(x.data_ptr(), index.data_ptr(), out.data_ptr(), rows, x.shape[-1], index.shape[-1],
                                          x.element_size(), _err_flag(x.device).data_ptr(), _s()), "gather_last")
    return out


def scatter_last(dst: torch.Tensor, index: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    if not dst.is_cuda or dst.element_size() not in (2, 4):
        return dst.scatter_(-1, index, src)
    assert dst.is_contiguous()
    rows = dst.numel() // dst.shape[-1]
    nat.check(nat.cuda().incin_scatter_last(src.contiguous().data_ptr(), index.contiguous().data_ptr(), dst.data_ptr(), rows,
                                           dst.shape[-1], index.shape[-1], dst.element_size(), _err_flag(dst.device).data_ptr(),
                                           _s()), "scatter_last")
    return dst


def masked_fill(x: torch.Tensor, mask: torch.Tensor, value: float) -> torch.Tensor:
    if not _native(x):
        return x.masked_fill(mask, value)
    x = x.contiguous()
    m = mask.expand(x.shape).contiguous().view(torch.uint8)
    out = torch.empty_like(x)
    nat.check(nat.cuda().incin_masked_fill(x.data_ptr(), m.data_ptr(), out.data_ptr(), float(value), x.numel(), _bf(x), _s()),
              "masked_fill")
    return out


def where(cond: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if not a.is_cuda or a.element_size() not in (2, 4):
        return torch.where(cond, a, b)
    shape = torch.broadcast_shapes(cond.shape, a.shape, b.shape)
    a, b = a.expand(shape).contiguous(), b.expand(shape).contiguous()
    c = cond.expand(shape).contiguous().view(torch.uint8)
    out = torch.empty_like(a)
    nat.check(nat.cuda().incin_where(c.data_ptr(), a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), a.element_size(), _s()),
              "where")
    return out


def _tri(x, diagonal, upper):
    if not x.is_cuda or x.element_size() not in (2, 4):
        return torch.triu(x, diagonal) if upper else torch.tril(x, diagonal)
    x = x.contiguous()
    rows, cols = x.shape[-2], x.shape[-1]
    out = torch.empty_like(x)
    nat.check(nat.cuda().incin_tri(x.data_ptr(), out.data_ptr(), x.numel() // (rows * cols), rows, cols, diagonal, int(upper),
                                  x.element_size(), _s()), "tri")
    return out


def triu(x, diagonal: int = 0):
    return _tri(x, diagonal, True)


def tril(x, diagonal: int = 0):
    return _tri(x, diagonal, False)


# ---------------------------------------------------------------------------------------------------- spatial
def _geom(x_shape, kernel, stride, padding, dilation=(1, 1)) -> ConvGeom:
    N, Cc, H, W = x_shape
    return ConvGeom(N, Cc, H, W, kernel[0], kernel[1], stride[0], stride[1], padding[0], padding[1], dilation[0], dilation[1])


def conv_out_hw(g: ConvGeom) -> tuple[int, int]:
    oh = (g.H + 2 * g.pad_h - g.dil_h * (g.KH - 1) - 1) // g.stride_h + 1
    ow = (g.W + 2 * g.pad_w - g.dil_w * (g.KW - 1) - 1) // g.stride_w + 1
    return oh, ow


def im2col(x: torch.Tensor, kernel, stride=(1, 1), padding=(0, 0), dilation=(1, 1)) -> torch.Tensor:
    """``[N, C, H, W] -> [N*OH*OW, C*KH*KW]`` (the A operand of the convolution GEMM)."""
    g = _geom(x.shape, kernel, stride, padding, dilation)
    oh, ow = conv_out_hw(g)
    if not _native(x):
        cols = torch.nn.functional.unfold(x.float(), kernel, dilation, padding, stride)      # [N, C*KH*KW, OH*OW]
        return cols.transpose(1, 2).reshape(g.N * oh * ow, -1).to(x.dtype)
    x = x.contiguous()
    out = torch.empty(g.N * oh * ow, g.C * g.KH * g.KW, dtype=x.dtype, device=x.device)
    nat.check(nat.cuda().incin_im2col(x.data_ptr(), out.data_ptr(), C.byref(g), _bf(x), _s()), "im2col")
    return out


def col2im(cols: torch.Tensor, x_shape, kernel, stride=(1, 1), padding=(0, 0), dilation=(1, 1)) -> torch.Tensor:
    g = _geom(x_shape, kernel, stride, padding, dilation)
    oh, ow = conv_out_hw(g)
    if not _native(cols):
        c = cols.float().reshape(g.N, oh * ow, -1).transpose(1, 2)
        return torch.nn.functional.fold(c, (g.H, g.W), kernel, dilation, padding, stride).to(cols.dtype)
    out = torch.empty(tuple(x_shape), dtype=cols.dtype, device=cols.device)
    nat.check(nat.cuda().incin_col2im(cols.contiguous().data_ptr(), out.data_ptr(), C.byref(g), _bf(cols), _s()), "col2im")
    return out


class _MaxPool2d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kernel, stride, padding):
        g = _geom(x.shape, kernel, stride, padding)
        oh, ow = conv_out_hw(g)
        x = x.contiguous()
        y = torch.empty(g.N, g.C, oh, ow, dtype=x.dtype, device=x.device)
        arg = torch.empty(g.N, g.C, oh, ow, dtype=torch.int32, device=x.device)
        nat.check(nat.cuda().incin_maxpool2d_fwd(x.data_ptr(), y.data_ptr(), arg.data_ptr(), C.byref(g), _bf(x), _s()), "maxpool_fwd")
        ctx.save_for_backward(arg)
        ctx.g, ctx.shape = g, x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        (arg,) = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty(ctx.shape, dtype=dy.dtype, device=dy.device)
        nat.check(nat.cuda().incin_maxpool2d_bwd(dy.data_ptr(), arg.data_ptr(), dx.data_ptr(), C.byref(ctx.g), _bf(dy), _s()),
                  "maxpool_bwd")
        return dx, None, None, None


class _AvgPool2d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kernel, stride, padding):
        g = _geom(x.shape, kernel, stride, padding)
        oh, ow = conv_out_hw(g)
        x = x.contiguous()
        y = torch.empty(g.N, g.C, oh, ow, dtype=x.dtype, device=x.device)
        nat.check(nat.cuda().incin_avgpool2d(x.data_ptr(), y.data_ptr(), C.byref(g), 0, _bf(x), _s()), "avgpool_fwd")
        ctx.g, ctx.shape = g, x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        dy = dy.contiguous()
        dx = torch.empty(ctx.shape, dtype=dy.dtype, device=dy.device)
        nat.check(nat.cuda().incin_avgpool2d(dy.data_ptr(), dx.data_ptr(), C.byref(ctx.g), 1, _bf(dy), _s()), "avgpool_bwd")
        return dx, None, None, None


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def max_pool2d(x, kernel, stride=None, padding=0):
    kernel, stride, padding = _pair(kernel), _pair(stride if stride is not None else kernel), _pair(padding)
    if not _native(x):
        return torch.nn.functional.max_pool2d(x, kernel, stride, padding)
    return _MaxPool2d.apply(x, kernel, stride, padding)


def avg_pool2d(x, kernel, stride=None, padding=0):
    kernel, stride, padding = _pair(kernel), _pair(stride if stride is not None else kernel), _pair(padding)
    if not _native(x):
        return torch.nn.functional.avg_pool2d(x, kernel, stride, padding)
    return _AvgPool2d.apply(x, kernel, stride, padding)


class _AdaptiveAvgPool2d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_hw):
        x = x.contiguous()
        N, Cc, H, W = x.shape
        oh, ow = out_hw
        y = torch.empty(N, Cc, oh, ow, dtype=x.dtype, device=x.device)
        nat.check(nat.cuda().incin_adaptive_avgpool2d(x.data_ptr(), y.data_ptr(), N * Cc, H, W, oh, ow, 0, _bf(x), _s()),
                  "adaptive_avgpool_fwd")
        ctx.dims = (N, Cc, H, W, oh, ow)
        return y

    @staticmethod
    def backward(ctx, dy):
        N, Cc, H, W, oh, ow = ctx.dims
        dy = dy.contiguous()
        dx = torch.empty(N, Cc, H, W, dtype=dy.dtype, device=dy.device)
        nat.check(nat.cuda().incin_adaptive_avgpool2d(dy.data_ptr(), dx.data_ptr(), N * Cc, H, W, oh, ow, 1, _bf(dy), _s()),
                  "adaptive_avgpool_bwd")
        return dx, None


def adaptive_avg_pool2d(x, output_size):
    """``[N, C, H, W] -> [N, C, OH, OW]``; cell (i, j) averages rows ``floor(i H / OH) .. ceil((i + 1) H / OH)`` and the
    same in w (crates/incin-backends/src/cuda/backend.rs:1753).  ``None`` in ``output_size`` keeps that extent."""
    oh, ow = _pair(output_size)
    oh = x.shape[-2] if oh is None else oh
    ow = x.shape[-1] if ow is None else ow
    if not _native(x):
        return torch.nn.functional.adaptive_avg_pool2d(x, (oh, ow))
    return _AdaptiveAvgPool2d.apply(x, (oh, ow))


class _SoftmaxLast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        x = x.contiguous()
        Cc = x.shape[-1]
        y = torch.empty_like(x)
        nat.check(nat.cuda().incin_softmax_lastdim_fwd(x.data_ptr(), y.data_ptr(), x.numel() // Cc, Cc, _bf(x), _s()), "softmax_fwd")
        ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        dy = dy.contiguous()
        Cc = y.shape[-1]
        dx = torch.empty_like(y)
        nat.check(nat.cuda().incin_softmax_lastdim_bwd(dy.data_ptr(), y.data_ptr(), dx.data_ptr(), y.numel() // Cc, Cc, _bf(y), _s()),
                  "softmax_bwd")
        return dx


def softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """Softmax over ``dim``: one native launch (forward) / one (backward) on bf16 / fp32 CUDA tensors; another axis is
    moved to the end with the native strided copy and back."""
    if not _native(x) or x.numel() == 0:
        return torch.softmax(x, dim)
    dim = dim % x.dim()
    if dim == x.dim() - 1:
        return _SoftmaxLast.apply(x)
    return _SoftmaxLast.apply(x.transpose(dim, -1)).transpose(dim, -1)


# ---------------------------------------------------------------------------------------------------- convolutions
def _nchw_rows(x: torch.Tensor) -> torch.Tensor:
    """``[N, C, H, W] -> [N*H*W, C]`` (channels last rows), native strided copy."""
    N, Cc, H, W = x.shape
    return materialize(x.permute(0, 2, 3, 1)).reshape(N * H * W, Cc)


def _rows_nchw(rows: torch.Tensor, N: int, H: int, W: int) -> torch.Tensor:
    return materialize(rows.reshape(N, H, W, rows.shape[-1]).permute(0, 3, 1, 2))


def _conv_gemm_ok(*dims) -> bool:
    return all(d % 8 == 0 for d in dims)      # 16-byte rows for the TMA-fed GEMM


class _Conv2d(torch.autograd.Function):
    """Convolution as unfold + tcgen05 GEMM, backward as GEMMs + fold: every step a kernel of this library
    (crates/incin-backends/src/cuda/backend.rs:1604-1719 does the same with its SGEMM, per batch and group)."""

    @staticmethod
    def forward(ctx, x, w, b, stride, padding, dilation):
        from . import gemm as G
        N, Cin, H, W = x.shape
        O, _, KH, KW = w.shape
        cols = im2col(x, (KH, KW), stride, padding, dilation)                      # [N*L, Cin*KH*KW]
        wk = w.reshape(O, Cin * KH * KW).contiguous()
        y_rows = G.mm_nt(cols, wk, bias=b)                                         # [N*L, O]
        g = _geom(x.shape, (KH, KW), stride, padding, dilation)
        oh, ow = conv_out_hw(g)
        ctx.save_for_backward(cols, wk)
        ctx.meta = (x.shape, w.shape, stride, padding, dilation, oh, ow, b is not None)
        return _rows_nchw(y_rows, N, oh, ow)

    @staticmethod
    def backward(ctx, dy):
        from . import gemm as G
        from . import kernels as K
        cols, wk = ctx.saved_tensors
        x_shape, w_shape, stride, padding, dilation, oh, ow, has_b = ctx.meta
        dy_rows = _nchw_rows(dy.contiguous())                                      # [N*L, O]
        dx = dw = db = None
        if ctx.needs_input_grad[1]:
            dwf = torch.zeros(wk.shape, dtype=torch.float32, device=dy.device)
            G.mm_tn_accum(dy_rows, cols, dwf)                                      # dy^T @ cols
            dw = dwf.to(wk.dtype).reshape(w_shape)
        if has_b and ctx.needs_input_grad[2]:
            dbf = torch.zeros(w_shape[0], dtype=torch.float32, device=dy.device)
            K.colsum_accum(dy_rows, dbf)
            db = dbf.to(wk.dtype)
        if ctx.needs_input_grad[0]:
            dcols = G.mm_nn(dy_rows, wk)                                           # [N*L, Cin*KH*KW]
            dx = col2im(dcols, x_shape, w_shape[2:], stride, padding, dilation)
        return dx, dw, db, None, None, None


def conv2d(x, w, b=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1)):
    """NCHW convolution (groups = 1).  bf16 CUDA tensors whose GEMM dimensions are multiples of 8 run on the native
    unfold / tcgen05 GEMM / fold kernels; everything else is evaluated by PyTorch."""
    stride, padding, dilation = _pair(stride), _pair(padding), _pair(dilation)
    O, Cin, KH, KW = w.shape
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and _conv_gemm_ok(O, Cin * KH * KW):
        return _Conv2d.apply(x, w, b, stride, padding, dilation)
    return torch.nn.functional.conv2d(x, w, b, stride, padding, dilation)


def conv1d(x, w, b=None, stride: int = 1, padding: int = 0, dilation: int = 1):
    """``[N, C, L]`` convolution as the 2-D one over a height of 1 (im2col_1d + GEMM in the reference:
    crates/incin-backends/src/cuda/backend.rs:1576, kernels/conv.cu:106-181)."""
    y = conv2d(x.unsqueeze(2), w.unsqueeze(2), b, (1, stride), (0, padding), (1, dilation))
    return y.squeeze(2)


class _ConvTranspose2d(torch.autograd.Function):
    """Transposed convolution: one GEMM produces the column matrix, the fold kernel scatters it into the output
    (gather form, no atomics); the backward is unfold + two GEMMs."""

    @staticmethod
    def forward(ctx, x, w, b, stride, padding, dilation, out_hw):
        from . import gemm as G
        N, Cin, H, W = x.shape
        _, Cout, KH, KW = w.shape
        x_rows = _nchw_rows(x)                                                     # [N*H*W, Cin]
        wm = w.reshape(Cin, Cout * KH * KW).contiguous()
        cols = G.mm_nn(x_rows, wm)                                                 # [N*H*W, Cout*KH*KW]
        y_shape = (N, Cout, out_hw[0], out_hw[1])
        y = col2im(cols, y_shape, (KH, KW), stride, padding, dilation)
        if b is not None:
            y = y + b.view(1, -1, 1, 1)
        ctx.save_for_backward(x_rows, wm)
        ctx.meta = (x.shape, w.shape, stride, padding, dilation, b is not None)
        return y

    @staticmethod
    def backward(ctx, dy):
        from . import gemm as G
        x_rows, wm = ctx.saved_tensors
        x_shape, w_shape, stride, padding, dilation, has_b = ctx.meta
        N, Cin, H, W = x_shape
        dcols = im2col(dy.contiguous(), w_shape[2:], stride, padding, dilation)    # [N*H*W, Cout*KH*KW]
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = _rows_nchw(G.mm_nt(dcols, wm), N, H, W)                           # dcols @ wm^T -> [N*H*W, Cin]
        if ctx.needs_input_grad[1]:
            dwf = torch.zeros(wm.shape, dtype=torch.float32, device=dy.device)
            G.mm_tn_accum(x_rows, dcols, dwf)                                      # x^T @ dcols
            dw = dwf.to(wm.dtype).reshape(w_shape)
        if has_b and ctx.needs_input_grad[2]:
            db = reduce(reduce(reduce(dy.float(), "sum", 3), "sum", 2), "sum", 0).to(dy.dtype)
        return dx, dw, db, None, None, None, None


def conv_transpose2d(x, w, b=None, stride=(1, 1), padding=(0, 0), output_padding=(0, 0), dilation=(1, 1)):
    """``x [N, Cin, H, W]``, ``w [Cin, Cout, KH, KW]`` -> ``[N, Cout, OH, OW]`` with
    ``OH = (H - 1) stride - 2 padding + dilation (KH - 1) + output_padding + 1`` (groups = 1;
    crates/incin-backends/src/cuda/backend.rs:1604)."""
    stride, padding, dilation, opad = _pair(stride), _pair(padding), _pair(dilation), _pair(output_padding)
    Cin, Cout, KH, KW = w.shape
    H, W = x.shape[-2:]
    oh = (H - 1) * stride[0] - 2 * padding[0] + dilation[0] * (KH - 1) + opad[0] + 1
    ow = (W - 1) * stride[1] - 2 * padding[1] + dilation[1] * (KW - 1) + opad[1] + 1
    if x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and _conv_gemm_ok(Cin, Cout * KH * KW):
        return _ConvTranspose2d.apply(x, w, b, stride, padding, dilation, (oh, ow))
    return torch.nn.functional.conv_transpose2d(x, w, b, stride, padding, opad, 1, dilation)


class _BatchNormTrain(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, running_mean, running_var, eps, momentum):
        x = x.contiguous()
        N, Cc = x.shape[0], x.shape[1]
        HW = x.numel() // (N * Cc)
        y = torch.empty_like(x)
        mean = torch.empty(Cc, dtype=torch.float32, device=x.device)
        rstd = torch.empty(Cc, dtype=torch.float32, device=x.device)
        nat.check(nat.cuda().incin_batchnorm_train_fwd(x.data_ptr(), nat.ptr(gamma), nat.ptr(beta), y.data_ptr(), mean.data_ptr(),
                                                      rstd.data_ptr(), nat.ptr(running_mean), nat.ptr(running_var), N, Cc, HW,
                                                      eps, momentum, _bf(x), _s()), "batchnorm_fwd")
        ctx.save_for_backward(x, gamma, mean, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gamma, mean, rstd = ctx.saved_tensors
        dy = dy.contiguous()
        N, Cc = x.shape[0], x.shape[1]
        HW = x.numel() // (N * Cc)
        dx = torch.empty_like(x)
        dg = torch.zeros(Cc, dtype=torch.float32, device=x.device)
        db = torch.zeros(Cc, dtype=torch.float32, device=x.device)
        nat.check(nat.cuda().incin_batchnorm_bwd(dy.data_ptr(), x.data_ptr(), nat.ptr(gamma), mean.data_ptr(), rstd.data_ptr(),
                                                dx.data_ptr(), dg.data_ptr(), db.data_ptr(), N, Cc, HW, _bf(x), _s()),
                  "batchnorm_bwd")
        return dx, (dg if gamma is not None else None), db, None, None, None, None


def batch_norm(x, gamma, beta, running_mean, running_var, training: bool, momentum: float = 0.1, eps: float = 1e-5):
    """``[N, C, *]`` batch normalisation; gamma/beta/running statistics are fp32 ``[C]``."""
    if not _native(x):
        return torch.nn.functional.batch_norm(x, running_mean, running_var, gamma, beta, training, momentum, eps)
    if training:
        return _BatchNormTrain.apply(x, gamma, beta, running_mean, running_var, eps, momentum)
    x = x.contiguous()
    N, Cc = x.shape[0], x.shape[1]
    y = torch.empty_like(x)
    nat.check(nat.cuda().incin_batchnorm_eval(x.data_ptr(), nat.ptr(gamma), nat.ptr(beta), running_mean.data_ptr(),
                                             running_var.data_ptr(), y.data_ptr(), N, Cc, x.numel() // (N * Cc), eps, _bf(x), _s()),
              "batchnorm_eval")
    return y


# ---------------------------------------------------------------------------------------------------- Q8_0 on device
def quantize_q8_0_cuda(x: torch.Tensor) -> torch.Tensor:
    x = x.contiguous()
    n = x.numel()
    out = torch.empty((n + 31) // 32 * 34, dtype=torch.uint8, device=x.device)
    nat.check(nat.cuda().incin_quantize_q8_0(x.data_ptr(), out.data_ptr(), n, _bf(x), _s()), "quantize_q8_0")
    return out


def dequantize_q8_0_cuda(packed: torch.Tensor, numel: int, dtype=torch.bfloat16) -> torch.Tensor:
    out = torch.empty(numel, dtype=dtype, device=packed.device)
    nat.check(nat.cuda().incin_dequantize_q8_0(packed.contiguous().data_ptr(), out.data_ptr(), numel,
                                              int(dtype == torch.bfloat16), _s()), "dequantize_q8_0")
    return out


# ---------------------------------------------------------------------------------------------------- embedding
def embedding_bwd_deterministic(dout: torch.Tensor, tokens: torch.Tensor, dwte: torch.Tensor, dwpe: torch.Tensor | None,
                                T: int) -> None:
    """Accumulate the embedding gradient with a fixed summation order (sort by token, one block per distinct token)."""
    flat = tokens.reshape(-1)
    sorted_tok, order = torch.sort(flat, stable=True)
    uniq, counts = torch.unique_consecutive(sorted_tok, return_counts=True)
    starts = torch.zeros(uniq.numel() + 1, dtype=torch.int64, device=flat.device)
    starts[1:] = torch.cumsum(counts, 0)
    Cc = dout.shape[-1]
    nat.check(nat.cuda().incin_embedding_bwd_sorted(dout.contiguous().data_ptr(), order.data_ptr(), starts.data_ptr(),
                                                   uniq.data_ptr(), uniq.numel(), dwte.data_ptr(), nat.ptr(dwpe),
                                                   flat.numel() // T, T, Cc, dwte.shape[0], _s()), "embedding_bwd_sorted")
