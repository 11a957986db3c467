"""Sampling distributions (crates/incin-core/src/distributions/mod.rs:10-216): Uniform, Normal, Bernoulli,
Exponential, Gumbel.  Sampling is seeded: CUDA tensors come from the device Philox4x32-10 kernels (stream =
(seed, offset)), CPU tensors from the bit-identical host implementation in libincin_host, so a (seed, offset)
pair names one sequence on every backend."""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _native as nat


def _uniform(shape, seed: int, offset: int, device) -> torch.Tensor:
    device = torch.device(device)
    if device.type == "cuda":
        from .ops import kernels as K
        return K.philox_uniform(tuple(shape), seed, offset, device)
    out = torch.empty(tuple(shape), dtype=torch.float32)
    h = nat.host()
    h.incin_cpu_philox_uniform_f32.argtypes = [C.c_void_p, C.c_int64, C.c_uint64, C.c_uint64]
    h.incin_cpu_philox_uniform_f32(out.data_ptr(), out.numel(), seed, offset)
    return out


def _normal(shape, seed: int, offset: int, device) -> torch.Tensor:
    device = torch.device(device)
    if device.type == "cuda":
        from .ops import kernels as K
        return K.philox_normal(tuple(shape), seed, offset, device)
    out = torch.empty(tuple(shape), dtype=torch.float32)
    h = nat.host()
    h.incin_cpu_philox_normal_f32.argtypes = [C.c_void_p, C.c_int64, C.c_uint64, C.c_uint64, C.c_float, C.c_float]
    h.incin_cpu_philox_normal_f32(out.data_ptr(), out.numel(), seed, offset, 0.0, 1.0)
    return out


class Distribution:
    def sample(self, shape, seed: int = 0, offset: int = 0, device="cpu") -> torch.Tensor:
        raise NotImplementedError


class Uniform(Distribution):
    def __init__(self, low: float = 0.0, high: float = 1.0):
        if not high > low:
            raise ValueError("high must exceed low")
        self.low, self.high = low, high

    def sample(self, shape, seed=0, offset=0, device="cpu"):
        return self.low + (self.high - self.low) * _uniform(shape, seed, offset, device)


class Normal(Distribution):
    def __init__(self, mean: float = 0.0, std: float = 1.0):
        if std <= 0:
            raise ValueError("std must be positive")
        self.mean, self.std = mean, std

    def sample(self, shape, seed=0, offset=0, device="cpu"):
        return self.mean + self.std * _normal(shape, seed, offset, device)


class Bernoulli(Distribution):
    def __init__(self, p: float):
        if not 0.0 <= p <= 1.0:
            raise ValueError("p must be in [0, 1]")
        self.p = p

    def sample(self, shape, seed=0, offset=0, device="cpu"):
        return (_uniform(shape, seed, offset, device) < self.p).float()


class Exponential(Distribution):
    def __init__(self, rate: float = 1.0):
        if rate <= 0:
            raise ValueError("rate must be positive")
        self.rate = rate

    def sample(self, shape, seed=0, offset=0, device="cpu"):
        return -torch.log(_uniform(shape, seed, offset, device)) / self.rate


class Gumbel(Distribution):
    def __init__(self, loc: float = 0.0, scale: float = 1.0):
        self.loc, self.scale = loc, scale

    def sample(self, shape, seed=0, offset=0, device="cpu"):
        return self.loc - self.scale * torch.log(-torch.log(_uniform(shape, seed, offset, device)))
