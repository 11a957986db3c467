"""Finite-difference check of analytic gradients.

Counterpart of the reference's CPU gradcheck (crates/incin-backends/src/cpu/gradcheck.rs: central differences used by
the op tests of the CPU backend).  ``gradcheck(fn, inputs)`` perturbs every element (or a seeded sample of elements) of
every differentiable input by +-eps, forms ``(f(x + eps) - f(x - eps)) / (2 eps)`` of the scalarised output and compares
with what ``backward`` produced.  It works on any device; the tolerances default to what float32 arithmetic supports.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Sequence

import torch


@dataclass
class GradcheckFinding:
    input_index: int
    flat_index: int
    analytic: float
    numeric: float

    def __str__(self) -> str:
        return (f"input {self.input_index}[{self.flat_index}]: backward says {self.analytic:.6g}, "
                f"central difference says {self.numeric:.6g}")


def gradcheck(fn: Callable[..., torch.Tensor], inputs: Sequence[torch.Tensor], *, eps: float = 1e-2, rtol: float = 2e-2,
              atol: float = 2e-3, max_elements: int = 64, seed: int = 0, raise_on_failure: bool = True
              ) -> list[GradcheckFinding]:
    """Compare ``backward`` of ``fn(*inputs)`` with central differences.

    ``fn`` may return a tensor of any shape: it is reduced to a scalar with a fixed random weighting, so that errors in
    individual output elements cannot cancel.  Inputs that do not require grad are passed through untouched.  At most
    ``max_elements`` elements per input are perturbed (a seeded sample), which keeps the check linear in that number.
    Returns the list of mismatches (empty = pass) or raises ``AssertionError`` listing them.
    """
    inputs = [t.detach().clone().requires_grad_(t.requires_grad) if isinstance(t, torch.Tensor) else t for t in inputs]
    gen = torch.Generator().manual_seed(seed)
    out = fn(*inputs)
    weight = torch.randn(out.shape, generator=gen).to(device=out.device, dtype=torch.float32)

    def scalar(*args) -> torch.Tensor:
        return (fn(*args).float() * weight).sum()

    loss = (out.float() * weight).sum()
    diff_inputs = [t for t in inputs if isinstance(t, torch.Tensor) and t.requires_grad]
    grads = torch.autograd.grad(loss, diff_inputs, allow_unused=True)
    findings: list[GradcheckFinding] = []
    gi = 0
    for idx, t in enumerate(inputs):
        if not (isinstance(t, torch.Tensor) and t.requires_grad):
            continue
        g = grads[gi]
        gi += 1
        g = torch.zeros_like(t) if g is None else g
        n = t.numel()
        picks = range(n) if n <= max_elements else torch.randperm(n, generator=gen)[:max_elements].tolist()
        base = t.detach().clone()
        for k in picks:
            with torch.no_grad():
                args_p = [a.detach() if isinstance(a, torch.Tensor) else a for a in inputs]
                plus, minus = base.clone(), base.clone()
                plus.view(-1)[k] += eps
                minus.view(-1)[k] -= eps
                args_p[idx] = plus
                fp = scalar(*args_p).item()
                args_p[idx] = minus
                fm = scalar(*args_p).item()
            numeric = (fp - fm) / (2.0 * eps)
            analytic = g.reshape(-1)[k].item()
            if abs(numeric - analytic) > atol + rtol * max(abs(numeric), abs(analytic)):
                findings.append(GradcheckFinding(idx, int(k), analytic, numeric))
    if findings and raise_on_failure:
        raise AssertionError("gradcheck failed:\n  " + "\n  ".join(map(str, findings[:8])) +
                             (f"\n  ... and {len(findings) - 8} more" if len(findings) > 8 else ""))
    return findings
