"""ctypes bindings of the two native libraries.

``cuda()`` returns ``libincin_sm100.so`` (hand-written sm_100a kernels behind a C
ABI, see ``csrc/include/incin_b200.h``); ``host()`` returns ``libincin_host.so``
(CPU oracle and host runtime).  Both are built in-tree on first use when a
compiler is present.  On a machine with a GPU a missing CUDA library is an
error, never a silent fallback: every op in ``incin_b200.ops`` that is given a
CUDA tensor calls into this module.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

_LIBDIR = Path(__file__).resolve().parent / "lib"
_lock = threading.Lock()
_cuda = None
_host = None

c_void_p, c_int, c_ll, c_float, c_u64 = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_uint64

STATUS_NAMES = {
    0: "ok", 1: "bad argument", 2: "misaligned operand (TMA needs 16-byte aligned bases and strides)",
    3: "CUDA driver entry point unavailable", 4: "tensor map encode failed", 5: "kernel launch failed",
    6: "unsupported", 7: "size beyond the compiled-in maximum", 8: "peer access unavailable",
}

ACT_NONE, ACT_GELU, ACT_SILU, ACT_DGELU, ACT_DSILU = 0, 1, 2, 3, 4


class NativeError(RuntimeError):
    pass


LAUNCH_CALLS = 0  # number of native launch calls made by this process (each enqueues >= 1 kernel)
LAUNCH_HOOK = None  # set by incin_b200.telemetry.trace while NVTX marks / the per-step device trace are switched on


def check(rc: int, what: str = "") -> None:
    global LAUNCH_CALLS
    LAUNCH_CALLS += 1
    if LAUNCH_HOOK is not None:
        LAUNCH_HOOK(what)
    if rc != 0:
        raise NativeError(f"{what or 'native call'} failed: {STATUS_NAMES.get(rc, rc)}")


class GemmDesc(C.Structure):
    _fields_ = [
        ("A", c_void_p), ("B", c_void_p), ("C", c_void_p),
        ("M", c_int), ("N", c_int), ("K", c_int),
        ("lda", c_ll), ("ldb", c_ll), ("ldc", c_ll),
        ("a_mn_major", c_int), ("b_mn_major", c_int),
        ("batch_lo", c_int), ("batch_hi", c_int),
        ("a_stride_lo", c_ll), ("a_stride_hi", c_ll), ("b_stride_lo", c_ll), ("b_stride_hi", c_ll),
        ("c_stride_lo", c_ll), ("c_stride_hi", c_ll),
        ("out_fp32", c_int), ("accumulate", c_int), ("alpha", c_float),
        ("bias", c_void_p), ("residual", c_void_p), ("act", c_int), ("aux", c_void_p),
        ("splits", c_int), ("tile_n", c_int), ("max_ctas", c_int), ("status", c_void_p),
        ("ag_world", c_int), ("ag_rank", c_int), ("ag_rows_per_rank", c_int), ("ag_copy_ctas", c_int),
        ("ag_src", c_void_p * 8), ("ag_flags", c_void_p),
        ("rs_world", c_int), ("rs_rank", c_int), ("rs_rows_per_rank", c_int), ("rs_copy_ctas", c_int),
        ("rs_dst", c_void_p * 8), ("rs_slot_stride", c_ll), ("rs_ready", c_void_p),
        ("in_dtype", c_int), ("alpha_ptr", c_void_p),
    ]


GEMM_IN_BF16, GEMM_IN_FP16, GEMM_IN_TF32 = 0, 1, 2

_CUDA_SIGS = {
    "incin_gemm_bf16": (c_int, [C.POINTER(GemmDesc), c_void_p]),
    "incin_layernorm_fwd": (c_int, [c_void_p] * 6 + [c_ll, c_int, c_float, c_void_p]),
    "incin_layernorm_bwd_scratch_floats": (c_ll, [c_ll, c_int]),
    "incin_layernorm_bwd": (c_int, [c_void_p] * 10 + [c_ll, c_int, c_void_p]),
    "incin_layernorm_bwd_colsum_scratch_floats": (c_ll, [c_ll, c_int]),
    "incin_layernorm_bwd_colsum": (c_int, [c_void_p] * 11 + [c_ll, c_int, c_void_p]),
    "incin_rmsnorm_fwd": (c_int, [c_void_p] * 4 + [c_ll, c_int, c_float, c_void_p]),
    "incin_rmsnorm_bwd": (c_int, [c_void_p] * 8 + [c_ll, c_int, c_void_p]),
    "incin_embedding_fwd": (c_int, [c_void_p] * 4 + [c_ll, c_int, c_int, c_void_p]),
    "incin_embedding_bwd": (c_int, [c_void_p] * 4 + [c_ll, c_int, c_int, c_void_p]),
    "incin_xent_fwd": (c_int, [c_void_p] * 4 + [c_ll, c_int, c_ll, c_void_p]),
    "incin_xent_bwd": (c_int, [c_void_p] * 4 + [c_float, c_ll, c_int, c_ll, c_void_p]),
    "incin_xent_fused": (c_int, [c_void_p] * 4 + [c_float, c_ll, c_int, c_ll, c_void_p]),
    "incin_mean_f32": (c_int, [c_void_p, c_void_p, c_ll, c_void_p]),
    "incin_causal_softmax_fwd": (c_int, [c_void_p, c_ll, c_int, c_float, c_void_p]),
    "incin_causal_softmax_bwd": (c_int, [c_void_p, c_void_p, c_ll, c_int, c_float, c_void_p]),
    "incin_colsum_accum": (c_int, [c_void_p, c_void_p, c_ll, c_int, c_ll, c_void_p]),
    "incin_sumsq_nonfinite_f32": (c_int, [c_void_p, c_ll, c_void_p, c_void_p]),
    "incin_fill_f32": (c_int, [c_void_p, c_float, c_ll, c_void_p]),
    "incin_cast_f32_to_bf16": (c_int, [c_void_p, c_void_p, c_ll, c_void_p]),
    "incin_cast_bf16_to_f32": (c_int, [c_void_p, c_void_p, c_ll, c_void_p]),
    "incin_act_fwd": (c_int, [c_void_p, c_void_p, c_ll, c_int, c_void_p]),
    "incin_act_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p]),
    "incin_swiglu_fwd": (c_int, [c_void_p, c_void_p, c_ll, c_int, c_void_p]),
    "incin_swiglu_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p]),
    "incin_rope": (c_int, [c_void_p, c_ll, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_float, c_int, c_void_p]),
    "incin_adamw_flat": (c_int, [c_void_p] * 5 + [c_ll, c_ll, c_void_p, c_void_p]),
    "incin_sgd_flat": (c_int, [c_void_p] * 4 + [c_ll, c_ll, c_void_p, c_void_p]),
    "incin_philox_uniform_f32": (c_int, [c_void_p, c_ll, c_u64, c_u64, c_void_p]),
    "incin_philox_normal_f32": (c_int, [c_void_p, c_ll, c_u64, c_u64, c_float, c_float, c_void_p]),
    "incin_philox_normal_bf16": (c_int, [c_void_p, c_ll, c_u64, c_u64, c_float, c_float, c_void_p]),
    "incin_dropout_bf16": (c_int, [c_void_p, c_void_p, c_ll, c_float, c_u64, c_u64, c_void_p]),
    "incin_slot_reduce": (c_int, [c_void_p, c_ll, c_int, c_void_p, c_void_p, c_ll, c_int, c_ll, c_void_p]),
    "incin_sm100_version": (C.c_char_p, []),
    "incin_sm100_num_sms": (c_int, []),
}


def _bind(lib, sigs, strict: bool = False) -> None:
    for name, (res, args) in sigs.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            if strict:
                raise
            continue
        fn.restype = res
        fn.argtypes = args


def register_cuda_signatures(sigs: dict) -> None:
    """Let other modules (attention, fused collectives, ...) declare their entry points."""
    _CUDA_SIGS.update(sigs)
    if _cuda is not None:
        _bind(_cuda, sigs)


def cuda_library_path() -> Path:
    return _LIBDIR / "libincin_sm100.so"


def host_library_path() -> Path:
    return _LIBDIR / "libincin_host.so"


def cuda():
    """The sm_100a kernel library.  Raises when it cannot be loaded or built."""
    global _cuda
    if _cuda is None:
        with _lock:
            if _cuda is None:
                path = cuda_library_path()
                if not path.exists() or os.environ.get("INCIN_REBUILD"):
                    from . import _build
                    built = _build.build_cuda()
                    if built is None:
                        raise NativeError("libincin_sm100.so is missing and nvcc is not available to build it")
                lib = C.CDLL(str(path))
                _bind(lib, _CUDA_SIGS)
                _cuda = lib
    return _cuda


def host():
    """The host runtime / CPU oracle library."""
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                path = host_library_path()
                if not path.exists() or os.environ.get("INCIN_REBUILD"):
                    from . import _build
                    built = _build.build_host()
                    if built is None:
                        raise NativeError("libincin_host.so is missing and g++ is not available to build it")
                _host = C.CDLL(str(path))
    return _host


def cuda_loaded() -> bool:
    return _cuda is not None


def stream_ptr() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()
