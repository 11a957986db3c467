"""The allocation-free LayerNorm backward, called the way a C program would call it: through the
exported symbol of libincin_sm100.so with raw pointers and a raw stream handle.

Some users of this library cannot allocate device memory at the call site (no PyTorch allocator behind
them, or a thread that must stay away from the allocator while another one captures a graph).  For them
the library keeps the scratch of this one kernel in a fixed device array.  The test checks that the
variant returns what the regular entry point returns, on two calls in a row (the second call sees the
first call's leftovers in the shared scratch), and that an oversized problem is refused.

This file sorts last on purpose: a run that stops at the first failure has then already run every other
test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from incin_b200 import _native as nat
    lib = nat.cuda()
    c_void_p, c_ll, c_int = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    lib.incin_layernorm_bwd_noalloc.restype = c_int
    lib.incin_layernorm_bwd_noalloc.argtypes = [c_void_p] * 9 + [c_ll, c_int, c_void_p]
    return lib


def _case(rows, C, seed):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).cuda()
    return mk(rows, C), mk(C), mk(C), mk(rows, C), mk(rows, C)


@pytest.mark.parametrize("rows,C", [(512, 768), (1000, 1024)])
def test_noalloc_matches_regular_entry_point_twice(rows, C):
    from incin_b200.ops import kernels as K
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):  # second call runs over the first call's scratch contents
        x, gamma, beta, dy, add = _case(rows, C, 100 + call)
        _, mean, rstd = K.layernorm_fwd(x, gamma, beta, 1e-5)
        dg_ref = torch.zeros(C, device="cuda")
        db_ref = torch.zeros(C, device="cuda")
        dx_ref = K.layernorm_bwd(dy, x, gamma, mean, rstd, add, dg_ref, db_ref)
        dx = torch.empty_like(x)
        dg = torch.zeros(C, device="cuda")
        db = torch.zeros(C, device="cuda")
        rc = lib.incin_layernorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(),
                                             rstd.data_ptr(), add.data_ptr(), dx.data_ptr(), dg.data_ptr(),
                                             db.data_ptr(), rows, C, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(dx, dx_ref)
        for got, ref in ((dg, dg_ref), (db, db_ref)):
            err = (got - ref).abs().max().item()
            assert err <= 2e-2 * (ref.abs().max().item() + 1e-6), err


@pytest.mark.parametrize("rows,C,with_add,with_params", [(300, 4096, True, True),     # C > 1024: the two-pass path
                                                         (2048, 2048, False, True),   # no residual gradient to add
                                                         (512, 768, True, False),     # dx only (dgamma = dbeta = NULL)
                                                         (96, 8192, False, True)])    # the widest row the scratch admits
def test_noalloc_other_paths_against_fp32_math(rows, C, with_add, with_params):
    """The paths the first test does not reach (two-pass kernels for wide rows, no dx_add, no parameter gradients),
    checked against plain PyTorch fp32 math of the same backward, again on two calls in a row."""
    import torch.nn.functional as TF
    from _tol import check_close
    from incin_b200.ops import kernels as K
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        x, gamma, beta, dy, add = _case(rows, C, 200 + call)
        _, mean, rstd = K.layernorm_fwd(x, gamma, beta, 1e-5)
        xf, gf, bf = x.float().requires_grad_(), gamma.float().requires_grad_(), beta.float().requires_grad_()
        TF.layer_norm(xf, (C,), gf, bf, 1e-5).backward(dy.float())
        dx = torch.empty_like(x)
        dg = torch.zeros(C, device="cuda")
        db = torch.zeros(C, device="cuda")
        rc = lib.incin_layernorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                             add.data_ptr() if with_add else None, dx.data_ptr(),
                                             dg.data_ptr() if with_params else None, db.data_ptr() if with_params else None,
                                             rows, C, stream)
        assert rc == 0
        torch.cuda.synchronize()
        check_close(dx, xf.grad + (add.float() if with_add else 0.0), rtol=1.6e-2, atol_rms=1.5e-2, what=f"noalloc dx C{C}")
        if with_params:
            check_close(dg, gf.grad, rtol=1e-2, atol_rms=1e-2, what=f"noalloc dgamma C{C}")
            check_close(db, bf.grad, rtol=1e-2, atol_rms=1e-2, what=f"noalloc dbeta C{C}")


def test_noalloc_rejects_sizes_beyond_the_fixed_scratch():
    lib = _lib()
    rows, C = 8192, 16384  # 64 chunks * 2 * 16384 floats > the compiled-in maximum
    z = torch.zeros(8, device="cuda")
    rc = lib.incin_layernorm_bwd_noalloc(z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), None,
                                         z.data_ptr(), z.data_ptr(), z.data_ptr(), rows, C,
                                         torch.cuda.current_stream().cuda_stream)
    assert rc == 7  # INCIN_ERR_TOO_LARGE, nothing launched
    torch.cuda.synchronize()
