"""Tensor-level front end of the tcgen05 GEMM (``incin_gemm_bf16``).

The kernel computes ``C[b] = epi(alpha * A[b] @ B[b]^T)`` with A logically
``[M, K]`` and B logically ``[N, K]``; either operand may instead be stored
transposed ("MN-major"), which is how the three GEMMs of a Linear layer map
onto one kernel without transposes:

=========  =====================  ==========  ==========
product    math                   A           B
=========  =====================  ==========  ==========
forward    y  = x  @ W^T          x  K-major  W  K-major
dgrad      dx = dy @ W            dy K-major  W  MN-major
wgrad      dW = dy^T @ x          dy MN-major x  MN-major
=========  =====================  ==========  ==========

Counterpart of ``Tensor::matmul`` / ``MatMulSpec`` in the reference
(crates/incin-core/src/tensor/matmul.rs:349-444, exec/spec.rs:226).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native as nat

_status: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait gave up."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


def check_status(device: torch.device | None = None) -> None:
    """Synchronising check of the device status word; raises if any kernel timed out."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    code = int(status_word(device).item())
    if code != 0:
        status_word(device).zero_()
        raise nat.NativeError(f"a device-side wait timed out (status {code}); results of this step are invalid")


def auto_splits(M: int, N: int, K: int, batch: int = 1, sms: int = 148) -> int:
    """Split-K factor for accumulating fp32 outputs (weight gradients).  0 = let the kernel library choose the
    factor together with the tile from its measured cost model (the default for every shape)."""
    return 0


def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, *, M: int, N: int, K: int, lda: int, ldb: int,
         ldc: int, a_mn: bool = False, b_mn: bool = False, batch: tuple[int, int] = (1, 1),
         a_strides: tuple[int, int] = (0, 0), b_strides: tuple[int, int] = (0, 0),
         c_strides: tuple[int, int] = (0, 0), accumulate: bool = False, alpha: float = 1.0,
         bias: torch.Tensor | None = None, residual: torch.Tensor | None = None, act: int = nat.ACT_NONE,
         aux: torch.Tensor | None = None, splits: int = 1, tile_n: int = 0, max_ctas: int = 0,
         a_offset: int = 0, b_offset: int = 0, c_offset: int = 0, gather: dict | None = None,
         scatter: dict | None = None, alpha_dev: torch.Tensor | None = None) -> torch.Tensor:
    """Launch one (batched) GEMM on the current stream.  Offsets/strides are in elements.
    ``gather`` = {world, rank, rows_per_rank, src: [ptr]*world, flags: tensor, copy_ctas} turns the launch into the
    fused all-gather -> GEMM (``a`` is then the local gathered buffer); ``scatter`` = {world, rank, rows_per_rank,
    dst: [ptr]*world, slot_stride} makes the epilogue store partial tiles into the owners' slot buffers."""
    assert a.dtype == b.dtype and a.dtype in _IN_KIND, "operands must both be bf16, fp16 or fp32 (multiplied as tf32)"
    in_kind = _IN_KIND[a.dtype]
    assert out.dtype in (torch.bfloat16, torch.float32)
    if in_kind != nat.GEMM_IN_BF16:
        # fp16 / tf32 operands: fp32 output, no fused epilogue; tf32 wants K-contiguous operands
        assert out.dtype == torch.float32 and bias is None and residual is None and aux is None and act == nat.ACT_NONE
        assert gather is None and scatter is None and tile_n != 512
        assert in_kind == nat.GEMM_IN_FP16 or not (a_mn or b_mn)
    if tile_n == 0 and not accumulate and gather is None and scatter is None and in_kind == nat.GEMM_IN_BF16:
        tile_n = _tuned_tile_n(locals())
    d = nat.GemmDesc()
    d.in_dtype = in_kind
    d.A = a.data_ptr() + a.element_size() * a_offset
    d.B = b.data_ptr() + b.element_size() * b_offset
    d.C = out.data_ptr() + out.element_size() * c_offset
    d.M, d.N, d.K = M, N, K
    d.lda, d.ldb, d.ldc = lda, ldb, ldc
    d.a_mn_major, d.b_mn_major = int(a_mn), int(b_mn)
    d.batch_lo, d.batch_hi = batch
    d.a_stride_lo, d.a_stride_hi = a_strides
    d.b_stride_lo, d.b_stride_hi = b_strides
    d.c_stride_lo, d.c_stride_hi = c_strides
    d.out_fp32 = int(out.dtype == torch.float32)
    d.accumulate = int(accumulate)
    d.alpha = alpha
    if alpha_dev is not None:   # fp32 device scalar multiplied into alpha by the epilogue
        assert alpha_dev.dtype == torch.float32 and alpha_dev.numel() == 1 and alpha_dev.is_cuda
        d.alpha_ptr = alpha_dev.data_ptr()
    d.bias = nat.ptr(bias)
    d.residual = nat.ptr(residual)
    d.act = act
    d.aux = nat.ptr(aux)
    d.splits = splits
    d.tile_n = tile_n
    d.max_ctas = max_ctas
    d.status = status_word(a.device).data_ptr()
    if gather is not None:
        d.ag_world, d.ag_rank, d.ag_rows_per_rank = gather["world"], gather["rank"], gather["rows_per_rank"]
        d.ag_copy_ctas = gather.get("copy_ctas", 8)
        for r, ptr in enumerate(gather["src"]):
            d.ag_src[r] = ptr
        d.ag_flags = gather["flags"].data_ptr()
    if scatter is not None:
        d.rs_world, d.rs_rank, d.rs_rows_per_rank = scatter["world"], scatter["rank"], scatter["rows_per_rank"]
        for r, ptr in enumerate(scatter["dst"]):
            d.rs_dst[r] = ptr
        d.rs_slot_stride = scatter["slot_stride"]
        if scatter.get("copy_ctas", 0) > 0:
            d.rs_copy_ctas, d.rs_ready = scatter["copy_ctas"], scatter["ready"].data_ptr()
    nat.check(nat.cuda().incin_gemm_bf16(ctypes.byref(d), nat.stream_ptr()), "gemm")
    return out


_IN_KIND = {torch.bfloat16: nat.GEMM_IN_BF16, torch.float16: nat.GEMM_IN_FP16, torch.float32: nat.GEMM_IN_TF32}


def _tuned_tile_n(kw: dict) -> int:
    """Ask the autotune service for the N tile of this problem.  With the default policy this is a dictionary
    lookup that falls through to the kernel's own heuristic (0); under ``coordinated_warmup`` /
    ``profile_guided`` the tile widths (512 = the CTA-pair tile) are timed once per (shape, layout) and the winner is cached."""
    from ..tuning import TuningPolicy, candidates, service, time_cuda
    svc = service()
    if svc.policy in (TuningPolicy.DISABLED, TuningPolicy.HEURISTIC) and not svc.lru:
        return 0
    key = (f"gemm/{kw['M']}x{kw['N']}x{kw['K']}/{int(kw['a_mn'])}{int(kw['b_mn'])}/b{kw['batch'][0] * kw['batch'][1]}"
           f"/e{kw['act']}{int(kw['bias'] is not None)}{int(kw['residual'] is not None)}")
    if torch.cuda.is_current_stream_capturing():   # nothing can be timed inside a capture: use what warm-up found
        rec = svc.lookup(key)
        return rec.best["tile_n"] if rec is not None else 0

    def measure(params):
        args = {k: kw[k] for k in ("M", "N", "K", "lda", "ldb", "ldc", "a_mn", "b_mn", "batch", "a_strides", "b_strides",
                                   "c_strides", "alpha", "bias", "residual", "act", "aux", "splits", "max_ctas",
                                   "a_offset", "b_offset", "c_offset")}
        return time_cuda(lambda: gemm(kw["a"], kw["b"], kw["out"], tile_n=params["tile_n"], **args))
    return svc.choose(key, candidates(tile_n=[64, 128, 192, 256, 512]), lambda: {"tile_n": 0}, measure)["tile_n"]


def _rows(x: torch.Tensor) -> int:
    return x.numel() // x.shape[-1]


def mm_nt(x: torch.Tensor, w: torch.Tensor, *, bias=None, residual=None, act=nat.ACT_NONE, aux=None,
          out: torch.Tensor | None = None, alpha: float = 1.0, max_ctas: int = 0) -> torch.Tensor:
    """y[..., N] = x[..., K] @ w[N, K]^T with the fused epilogue (forward of Linear)."""
    assert x.is_contiguous() and w.is_contiguous()
    M, K = _rows(x), x.shape[-1]
    N = w.shape[0]
    if out is None:
        out = torch.empty(*x.shape[:-1], N, dtype=torch.bfloat16, device=x.device)
    return gemm(x, w, out, M=M, N=N, K=K, lda=K, ldb=K, ldc=N, bias=bias, residual=residual, act=act, aux=aux,
                alpha=alpha, max_ctas=max_ctas)


def mm_nt_f32out(x: torch.Tensor, w: torch.Tensor, *, alpha: float = 1.0, out: torch.Tensor | None = None,
                 accumulate: bool = False) -> torch.Tensor:
    """fp32 y[..., N] = x[..., K] @ w[N, K]^T on the tensor cores for bf16, fp16 or fp32 operands (fp32 operands are
    multiplied as tf32: 10 mantissa bits per factor, fp32 accumulation).  K must be a multiple of 8 (16-bit types)
    or 4 (fp32) so that every row starts on a 16-byte boundary."""
    assert x.is_contiguous() and w.is_contiguous() and x.dtype == w.dtype
    M, K = _rows(x), x.shape[-1]
    N = w.shape[0]
    if out is None:
        out = torch.empty(*x.shape[:-1], N, dtype=torch.float32, device=x.device)
    return gemm(x, w, out, M=M, N=N, K=K, lda=K, ldb=K, ldc=N, alpha=alpha, accumulate=accumulate)


def mm_nn(dy: torch.Tensor, w: torch.Tensor, *, act=nat.ACT_NONE, aux=None, out: torch.Tensor | None = None,
          max_ctas: int = 0, alpha_dev: torch.Tensor | None = None) -> torch.Tensor:
    """dx[..., K] = dy[..., N] @ w[N, K] (data gradient of Linear); optional act'(aux) mask."""
    assert dy.is_contiguous() and w.is_contiguous()
    M, N = _rows(dy), dy.shape[-1]
    K = w.shape[1]
    if out is None:
        out = torch.empty(*dy.shape[:-1], K, dtype=torch.bfloat16, device=dy.device)
    # reduction runs over N: A = dy (k-contiguous), B[K, N] is w stored [N(k)][K(n)] -> MN-major
    return gemm(dy, w, out, M=M, N=K, K=N, lda=N, ldb=K, ldc=K, b_mn=True, act=act, aux=aux, max_ctas=max_ctas,
                alpha_dev=alpha_dev)


def mm_tn_accum(dy: torch.Tensor, x: torch.Tensor, grad: torch.Tensor, *, splits: int | None = None,
                max_ctas: int = 0, alpha_dev: torch.Tensor | None = None) -> torch.Tensor:
    """grad[N, K] (fp32) += dy[M, N]^T @ x[M, K] (weight gradient, split-K with fp32 atomics)."""
    assert dy.is_contiguous() and x.is_contiguous() and grad.dtype == torch.float32
    M, N = _rows(dy), dy.shape[-1]
    K = x.shape[-1]
    if splits is None:
        splits = auto_splits(N, K, M)
    return gemm(dy, x, grad, M=N, N=K, K=M, lda=N, ldb=K, ldc=K, a_mn=True, b_mn=True, accumulate=True,
                splits=splits, max_ctas=max_ctas, alpha_dev=alpha_dev)


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """General ``a @ b`` for 2-D / batched 3-D bf16 tensors (b is [.., K, N], read MN-major)."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    a = a.contiguous()
    b = b.contiguous()
    if a.dim() == 2 and b.dim() == 2:
        M, K = a.shape
        N = b.shape[1]
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
        return gemm(a, b, out, M=M, N=N, K=K, lda=K, ldb=N, ldc=N, b_mn=True)
    assert a.dim() == 3 and b.dim() == 3 and a.shape[0] == b.shape[0]
    Bt, M, K = a.shape
    N = b.shape[2]
    out = torch.empty(Bt, M, N, dtype=torch.bfloat16, device=a.device)
    return gemm(a, b, out, M=M, N=N, K=K, lda=K, ldb=N, ldc=N, b_mn=True, batch=(Bt, 1),
                a_strides=(M * K, 0), b_strides=(K * N, 0), c_strides=(M * N, 0))
