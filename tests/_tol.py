"""Tolerance check shared by the GPU numerics tests.

A comparison of the largest error against the largest reference value passes a kernel that zeroes or garbles the
small-magnitude part of its output, so every GPU test also applies this elementwise criterion

    |actual - ref| <= atol_rms * rms(ref) + rtol * |ref|        for every element

(the absolute floor is tied to the RMS of the reference, not to its maximum, and stays a few percent of it), and
requires the cosine between the two tensors to be at least ``min_cos``.  bf16 outputs: rtol 1.6e-2 (two bf16 ulps),
fp32 outputs of bf16 products: a few 1e-3.  With ``INCIN_TOL_REPORT=1`` the observed figures are printed instead of
only asserted, which is how the constants were calibrated on the device.
"""
import os

import torch


def check_close(actual: torch.Tensor, ref: torch.Tensor, *, rtol: float = 1.6e-2, atol_rms: float = 1.5e-2,
                min_cos: float = 0.9999, what: str = "") -> None:
    a = actual.detach().float().reshape(-1).cpu().double()
    r = ref.detach().float().reshape(-1).cpu().double()
    assert a.shape == r.shape, (what, a.shape, r.shape)
    assert torch.isfinite(a).all(), f"{what}: non-finite values in the output"
    if r.numel() == 0:
        return
    rms = r.pow(2).mean().sqrt().item()
    diff = (a - r).abs()
    tol = atol_rms * rms + rtol * r.abs() + 1e-30
    worst = (diff / tol).max().item()
    na, nr = a.norm().item(), r.norm().item()
    cos = 1.0 if nr == 0.0 and na == 0.0 else float((a @ r).item() / (na * nr + 1e-300))
    if os.environ.get("INCIN_TOL_REPORT"):
        print(f"TOL {what or '?'} n={r.numel()} rms={rms:.3e} max_abs_err={diff.max().item():.3e} "
              f"worst_err_over_tol={worst:.3f} cos={cos:.7f}", flush=True)
    assert worst <= 1.0, (f"{what}: element error {worst:.2f}x the tolerance (rtol {rtol}, atol {atol_rms} x rms {rms:.3e}); "
                          f"max abs err {diff.max().item():.3e}")
    if nr > 0.0:
        assert cos >= min_cos, f"{what}: cosine {cos:.6f} < {min_cos}"
