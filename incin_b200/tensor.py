"""Tensor creation and the remaining tensor-level ops under the names the reference uses.

Counterparts: ``Tensor::{zeros, ones, rand, randn, full, arange, linspace, from_slice, from_bytes, sample}``
(crates/incin-core/src/tensor/base.rs:527-678), ``to_scalar / to_vec1``, and the ops of tensor/ops/*.rs that have no
kernel of their own here because they are views or thin compositions (``chunk / split / stack / expand / unfold /
pixel_shuffle / group_norm / instance_norm / topk / argsort / dot / outer / addmm / bmm``).  Tensors ARE
``torch.Tensor``; placement on a mesh is metadata carried beside them (:mod:`incin_b200.parallel.placement`).

Random creation uses the Philox4x32-10 generator of the kernel library, which produces the same stream on the CPU
oracle and on the device, so a seed means the same numbers on every backend.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _native as nat
from .core.dtype import DTypeId, to_torch

_seed = [0x1234ABCD, 0]      # seed, running offset (advanced by the number of values drawn)


builtins_slice = slice      # the module defines its own ``slice`` further down (the reference's name for the op)


def manual_seed(seed: int) -> None:
    _seed[0], _seed[1] = int(seed), 0


def _dev(device):
    return torch.device(device) if device is not None else torch.device("cpu")


def _dt(dtype):
    if isinstance(dtype, str):      # "bf16", "f32", ... : the ids' short names
        dtype = DTypeId(dtype)
    return to_torch(dtype) if isinstance(dtype, DTypeId) else (dtype or torch.float32)


def zeros(*shape, dtype=None, device=None):
    return torch.zeros(*shape, dtype=_dt(dtype), device=_dev(device))


def ones(*shape, dtype=None, device=None):
    return torch.ones(*shape, dtype=_dt(dtype), device=_dev(device))


def full(shape, value, dtype=None, device=None):
    return torch.full(tuple(shape), value, dtype=_dt(dtype), device=_dev(device))


def arange(start, end=None, step=1, dtype=None, device=None):
    if end is None:
        start, end = 0, start
    return torch.arange(start, end, step, dtype=_dt(dtype) if dtype else None, device=_dev(device))


def linspace(start, end, steps, dtype=None, device=None):
    return torch.linspace(start, end, steps, dtype=_dt(dtype), device=_dev(device))


def from_slice(values, shape=None, dtype=None, device=None):
    t = torch.tensor(list(values), dtype=_dt(dtype), device=_dev(device))
    return t.reshape(shape) if shape is not None else t


def from_bytes(raw: bytes, shape, dtype=None, device=None):
    t = torch.frombuffer(bytearray(raw), dtype=_dt(dtype)).reshape(tuple(shape)).clone()
    return t.to(_dev(device))


def _philox(n: int, normal: bool, device: torch.device, mean=0.0, std=1.0) -> torch.Tensor:
    seed, off = _seed
    _seed[1] += (n + 3) // 4 * 4
    if device.type == "cuda":
        out = torch.empty(n, dtype=torch.float32, device=device)
        lib = nat.cuda()
        if normal:
            nat.check(lib.incin_philox_normal_f32(out.data_ptr(), n, seed, off, mean, std, nat.stream_ptr()), "philox_normal")
        else:
            nat.check(lib.incin_philox_uniform_f32(out.data_ptr(), n, seed, off, nat.stream_ptr()), "philox_uniform")
        return out
    out = torch.empty(n, dtype=torch.float32)
    h = nat.host()
    if normal:
        h.incin_cpu_philox_normal_f32.argtypes = [C.c_void_p, C.c_int64, C.c_uint64, C.c_uint64, C.c_float, C.c_float]
        h.incin_cpu_philox_normal_f32(out.data_ptr(), n, seed, off, mean, std)
    else:
        h.incin_cpu_philox_uniform_f32.argtypes = [C.c_void_p, C.c_int64, C.c_uint64, C.c_uint64]
        h.incin_cpu_philox_uniform_f32(out.data_ptr(), n, seed, off)
    return out


def rand(*shape, dtype=None, device=None):
    n = int(torch.Size(shape).numel())
    return _philox(n, False, _dev(device)).reshape(shape).to(_dt(dtype))


def randn(*shape, dtype=None, device=None, mean: float = 0.0, std: float = 1.0):
    n = int(torch.Size(shape).numel())
    return _philox(n, True, _dev(device), mean, std).reshape(shape).to(_dt(dtype))


def from_raw(ptr: int, shape, dtype=None, device=None, owner=None):
    """A tensor over memory this process already owns (crates/incin-core/src/tensor/base.rs ``from_raw``): ``ptr`` is
    a host address (``device`` = cpu) or a device address of the given CUDA device.  Nothing is copied and nothing is
    freed: ``owner`` (any object) is kept alive with the tensor, the caller keeps the allocation alive otherwise."""
    import ctypes
    dt = _dt(dtype)
    shape = tuple(int(s) for s in shape)
    n = 1
    for s in shape:
        n *= s
    nbytes = n * torch.empty((), dtype=dt).element_size()
    dev = _dev(device)
    if dev.type == "cuda":
        class _Mem:
            pass
        m = _Mem()
        m.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 3}
        m._owner = owner
        flat = torch.as_tensor(m, device=dev)
    else:
        buf = (ctypes.c_ubyte * nbytes).from_address(int(ptr))
        buf._owner = owner
        flat = torch.frombuffer(buf, dtype=torch.uint8)
    return flat.view(dt).reshape(shape)


def sample(distribution, shape, device=None):
    """Draw from a :mod:`incin_b200.distributions` object."""
    return distribution.sample(tuple(shape)).to(_dev(device))


def to_scalar(t: torch.Tensor):
    if t.numel() != 1:
        raise ValueError(f"to_scalar needs exactly one element, the tensor has {t.numel()}")
    return t.item()


def to_vec1(t: torch.Tensor) -> list:
    if t.dim() != 1:
        raise ValueError("to_vec1 needs a rank-1 tensor")
    return t.tolist()


# ---- thin compositions (views or one or two kernels) -----------------------------------------------------------
chunk, split, stack, expand = torch.chunk, torch.split, torch.stack, lambda t, *shape: t.expand(*shape)


def flatten(t, start_dim: int = 0, end_dim: int = -1):
    return t.flatten(start_dim, end_dim)


def slice(t, dim: int, start: int, end: int, step: int = 1):      # noqa: A001 - the reference's name
    """``t[..., start:end:step, ...]`` along ``dim`` (a view)."""
    idx = [builtins_slice(None)] * t.dim()
    idx[dim] = builtins_slice(start, end, step)
    return t[tuple(idx)]


def to_dtype(t, dtype):
    return t.to(_dt(dtype))


def where_cond(cond, a, b):
    from .ops import tensor_ops as TO
    return TO.where(cond, a, b)


def gather(t, dim: int, index):
    """Last-axis gathers of CUDA tensors run on the native kernel, every other case on the PyTorch op."""
    from .ops import tensor_ops as TO
    if dim in (-1, t.dim() - 1):
        return TO.gather_last(t, index)
    return torch.gather(t, dim, index)


def scatter(t, dim: int, index, src):
    from .ops import tensor_ops as TO
    if dim in (-1, t.dim() - 1):
        return TO.scatter_last(t.clone(), index, src)
    return torch.scatter(t, dim, index, src)


def _reduction(name):
    def run(t, dim=None, keepdim: bool = False):
        from .ops import tensor_ops as TO
        return TO.reduce(t, name, dim, keepdim)
    run.__name__ = name
    run.__doc__ = f"``{name}`` over all elements or over ``dim`` (native reduction kernels on CUDA)."
    return run


sum, mean, max, min, argmax, argmin = (_reduction(n) for n in ("sum", "mean", "max", "min", "argmax", "argmin"))  # noqa: A001


def unfold(t, dim, size, step):
    return t.unfold(dim, size, step)


def pixel_shuffle(t, r: int):
    return torch.nn.functional.pixel_shuffle(t, r)


def group_norm(t, groups: int, weight=None, bias=None, eps: float = 1e-5):
    N, Cc = t.shape[:2]
    x = t.reshape(N, groups, -1).float()
    m = x.mean(-1, keepdim=True)
    v = x.var(-1, unbiased=False, keepdim=True)
    y = ((x - m) * torch.rsqrt(v + eps)).reshape(t.shape)
    if weight is not None:
        shape = [1, Cc] + [1] * (t.dim() - 2)
        y = y * weight.float().reshape(shape) + (bias.float().reshape(shape) if bias is not None else 0.0)
    return y.to(t.dtype)


def instance_norm(t, weight=None, bias=None, eps: float = 1e-5):
    return group_norm(t, t.shape[1], weight, bias, eps)


def topk(t, k: int, dim: int = -1, largest: bool = True):
    return torch.topk(t, k, dim, largest)


def argsort(t, dim: int = -1, descending: bool = False):
    return torch.argsort(t, dim, descending, stable=True)


def dot(a, b):
    return (a.float() * b.float()).sum().to(a.dtype)


def outer(a, b):
    return a[:, None] * b[None, :]


def addmm(bias, a, b):
    from .ops.functional import linear
    return linear(a, b.t().contiguous(), bias) if a.is_cuda and a.dtype == torch.bfloat16 else torch.addmm(bias, a, b)


def bmm(a, b):
    from .ops import gemm as G
    if a.is_cuda and a.dtype == torch.bfloat16:
        return G.matmul(a, b)
    return torch.bmm(a, b)
