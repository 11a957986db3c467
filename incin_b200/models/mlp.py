"""The CPU-backend MLP benchmark: Linear(784 -> 256) -> ReLU -> Linear(256 -> 10), softmax cross-entropy,
plain SGD, f32, batch 64.

Two implementations of the same arithmetic from the same seed-0 data:

* :func:`train_native` — the C++ tape-autograd engine in ``libincin_host.so`` (csrc/cpu_ref/tape.cpp), the
  CPU backend's own training loop;
* :func:`train_torch` — PyTorch CPU autograd over tensors drawn from the same generator, used to cross-check
  the loss curve.

Seed-0 generator (the reference has no seeding API, so it is defined here): Philox4x32-10 keyed by the seed;
stream offsets 0/1 = layer-1 weight/bias, 2/3 = layer-2 weight/bias (Kaiming-uniform, a = sqrt(5):
U(-1/sqrt(fan_in), +1/sqrt(fan_in)), bias with the same bound), 16 = inputs ~ N(0,1), 17 = labels
``floor(u * 10)``.
"""
from __future__ import annotations

import ctypes as C
import math
import time

import torch

from .. import _native as nat
from ..distributions import _normal, _uniform


def seed0_tensors(seed: int = 0, batch: int = 64, n_in: int = 784, hidden: int = 256, n_out: int = 10):
    def kaiming(shape, fan_in, off):
        return (2.0 * _uniform(shape, seed, off, "cpu") - 1.0) / math.sqrt(fan_in)
    w1, b1 = kaiming((hidden, n_in), n_in, 0), kaiming((hidden,), n_in, 1)
    w2, b2 = kaiming((n_out, hidden), hidden, 2), kaiming((n_out,), hidden, 3)
    x = _normal((batch, n_in), seed, 16, "cpu")
    y = (_uniform((batch,), seed, 17, "cpu") * n_out).long().clamp_(max=n_out - 1)
    return w1, b1, w2, b2, x, y


def train_native(steps: int = 100, batch: int = 64, n_in: int = 784, hidden: int = 256, n_out: int = 10,
                 lr: float = 0.01, seed: int = 0) -> tuple[list[float], float]:
    """Returns (loss per step, seconds)."""
    h = nat.host()
    h.incin_cpu_mlp_train.argtypes = [C.c_int] * 5 + [C.c_float, C.c_uint64, C.c_void_p, C.c_void_p]
    h.incin_cpu_mlp_train.restype = C.c_int
    losses = torch.zeros(steps, dtype=torch.float32)
    t0 = time.perf_counter()
    rc = h.incin_cpu_mlp_train(steps, batch, n_in, hidden, n_out, lr, seed, losses.data_ptr(), None)
    dt = time.perf_counter() - t0
    if rc:
        raise RuntimeError(f"native MLP training failed ({rc})")
    return losses.tolist(), dt


def train_torch(steps: int = 100, lr: float = 0.01, seed: int = 0) -> tuple[list[float], float]:
    w1, b1, w2, b2, x, y = seed0_tensors(seed)
    ps = [p.clone().requires_grad_() for p in (w1, b1, w2, b2)]
    losses = []
    t0 = time.perf_counter()
    for _ in range(steps):
        hdn = torch.relu(x @ ps[0].t() + ps[1])
        loss = torch.nn.functional.cross_entropy(hdn @ ps[2].t() + ps[3], y)
        losses.append(float(loss.detach()))
        grads = torch.autograd.grad(loss, ps)
        with torch.no_grad():
            for p, g in zip(ps, grads):
                p -= lr * g
    return losses, time.perf_counter() - t0
