"""NVRTC compilation (target sm_100a only) and launch of rendered pointwise kernels.

Compiled modules are cached in memory by :class:`KernelKey` (bounded LRU, 1024 entries like the reference's
``autotune/cuda/kernel_cache`` bound) and, as cubins, on disk in the autotune cache directory so a second
process skips NVRTC.  Launches go through the driver API on PyTorch's current stream, so they are
stream-ordered with every other kernel of the step and capturable in CUDA graphs.
"""
from __future__ import annotations

import collections
import ctypes
import hashlib
import os
from pathlib import Path

import torch

from .pointwise import CTYPES, KernelKey, Layout, PointwiseExpr, render_cuda

_TORCH = {torch.float32: "f32", torch.bfloat16: "bf16", torch.float16: "f16"}
CACHE_BOUND = 1024


class CompileError(RuntimeError):
    pass


def _include_dirs() -> list[str]:
    out = []
    for var in ("CUDA_INCLUDE_PATH", "CUDA_PATH", "CUDA_HOME", "CUDA_ROOT"):
        v = os.environ.get(var)
        if v:
            out.append(v if var == "CUDA_INCLUDE_PATH" else os.path.join(v, "include"))
    out.append("/usr/local/cuda/include")
    return [d for d in out if os.path.isdir(d)]


def cache_dir() -> Path:
    p = Path(os.environ.get("INCIN_AUTOTUNE_CACHE_DIR", os.path.expanduser("~/.cache/incin/autotune")))
    p.mkdir(parents=True, exist_ok=True)
    return p


def nvrtc_compile(source: str, name: str = "kernel.cu", arch: str = "sm_100a") -> bytes:
    """CUDA C -> cubin for sm_100a.  Needs no GPU."""
    from cuda.bindings import nvrtc
    err, prog = nvrtc.nvrtcCreateProgram(source.encode(), name.encode(), 0, [], [])
    if err != nvrtc.nvrtcResult.NVRTC_SUCCESS:
        raise CompileError(f"nvrtcCreateProgram: {err}")
    opts = [f"--gpu-architecture={arch}".encode(), b"--std=c++17", b"--use_fast_math"] + \
           [f"--include-path={d}".encode() for d in _include_dirs()]
    (err,) = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
    if err != nvrtc.nvrtcResult.NVRTC_SUCCESS:
        _, n = nvrtc.nvrtcGetProgramLogSize(prog)
        log = b" " * n
        nvrtc.nvrtcGetProgramLog(prog, log)
        nvrtc.nvrtcDestroyProgram(prog)
        raise CompileError(f"NVRTC failed for {name}:\n{log.decode(errors='replace')}")
    _, n = nvrtc.nvrtcGetCUBINSize(prog)
    cubin = b" " * n
    nvrtc.nvrtcGetCUBIN(prog, cubin)
    nvrtc.nvrtcDestroyProgram(prog)
    return cubin


def cubin_for(source: str, key: KernelKey) -> bytes:
    tag = hashlib.sha256((source + "|sm_100a|nvrtc").encode()).hexdigest()[:32]
    f = cache_dir() / f"{key.entry}_{tag}.cubin"
    if f.exists():
        return f.read_bytes()
    cubin = nvrtc_compile(source, key.entry + ".cu")
    tmp = f.with_suffix(f".tmp{os.getpid()}")
    tmp.write_bytes(cubin)
    os.replace(tmp, f)
    return cubin


class FusedKernel:
    def __init__(self, expr: PointwiseExpr, dtype: str, layout: Layout):
        self.source, self.key = render_cuda(expr, dtype, layout)
        self.expr, self.dtype, self.layout = expr, dtype, layout
        self._fn = None

    def _load(self):
        from cuda.bindings import driver
        cubin = cubin_for(self.source, self.key)
        err, mod = driver.cuModuleLoadData(cubin)
        if err != driver.CUresult.CUDA_SUCCESS:
            raise CompileError(f"cuModuleLoadData: {err}")
        err, fn = driver.cuModuleGetFunction(mod, self.key.entry.encode())
        if err != driver.CUresult.CUDA_SUCCESS:
            raise CompileError(f"cuModuleGetFunction({self.key.entry}): {err}")
        self._mod, self._fn = mod, fn

    def __call__(self, *tensors: torch.Tensor, scalars=(), out: torch.Tensor | None = None) -> torch.Tensor:
        from cuda.bindings import driver
        if len(tensors) != self.key.n_args or len(scalars) != self.key.n_scalars:
            raise ValueError(f"kernel takes {self.key.n_args} tensors and {self.key.n_scalars} scalars")
        torch.cuda.current_stream()  # binds the primary context on this thread
        if self._fn is None:
            self._load()
        if self.layout is Layout.CONTIGUOUS:
            shape = tensors[0].shape
            if any(t.shape != shape or not t.is_contiguous() for t in tensors):
                raise ValueError("contiguous kernel needs dense tensors of one shape")
            out = torch.empty_like(tensors[0]) if out is None else out
            n = out.numel()
            args = [out.data_ptr()] + [t.data_ptr() for t in tensors] + [float(s) for s in scalars] + [n]
            types = [ctypes.c_void_p] * (1 + len(tensors)) + [ctypes.c_float] * len(scalars) + [ctypes.c_longlong]
        else:
            shape = torch.broadcast_shapes(*[t.shape for t in tensors])
            if len(shape) > 6:
                raise ValueError("strided kernels support rank <= 6")
            out = torch.empty(shape, dtype=tensors[0].dtype, device=tensors[0].device) if out is None else out
            n = out.numel()
            rank = len(shape)
            meta = list(shape) + [1] * (6 - rank)
            for t in (out,) + tuple(x.expand(shape) for x in tensors):
                meta += list(t.stride()) + [0] * (6 - rank)
            meta_t = torch.tensor(meta, dtype=torch.int64, device=out.device)
            self._keep = meta_t
            args = [out.data_ptr()] + [t.data_ptr() for t in tensors] + [float(s) for s in scalars] + \
                   [n, rank, meta_t.data_ptr()]
            types = [ctypes.c_void_p] * (1 + len(tensors)) + [ctypes.c_float] * len(scalars) + \
                    [ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p]
        if n == 0:
            return out
        vec = CTYPES[self.dtype][2] if self.layout is Layout.CONTIGUOUS else 1
        blocks = max(1, min((n // vec + 255) // 256, 148 * 8))
        (err,) = driver.cuLaunchKernel(self._fn, blocks, 1, 1, 256, 1, 1, 0, torch.cuda.current_stream().cuda_stream,
                                       (tuple(args), tuple(types)), 0)
        if err != driver.CUresult.CUDA_SUCCESS:
            raise CompileError(f"cuLaunchKernel({self.key.entry}): {err}")
        return out


_cache: "collections.OrderedDict[tuple, FusedKernel]" = collections.OrderedDict()


def compile_pointwise(expr: PointwiseExpr, dtype: str = "bf16", layout: Layout = Layout.CONTIGUOUS) -> FusedKernel:
    k = (repr(expr), dtype, layout)
    if k in _cache:
        _cache.move_to_end(k)
        return _cache[k]
    fk = FusedKernel(expr, dtype, layout)
    _cache[k] = fk
    if len(_cache) > CACHE_BOUND:
        _cache.popitem(last=False)
    return fk


def fused(expr: PointwiseExpr, *tensors: torch.Tensor, scalars=()) -> torch.Tensor:
    """Evaluate a pointwise expression over CUDA tensors with one fused kernel (layout chosen from the inputs)."""
    dt = _TORCH[tensors[0].dtype]
    same = all(t.shape == tensors[0].shape and t.is_contiguous() for t in tensors)
    return compile_pointwise(expr, dt, Layout.CONTIGUOUS if same else Layout.STRIDED)(*tensors, scalars=scalars)
