"""Execution policy scopes, gradient mode, and mixed-precision policy with loss scaling.

Counterparts in the reference: crates/incin-core/src/exec/policy.rs (MathMode, Determinism,
FallbackPolicy, AllocatorPolicy, NanPolicy, ExecutionPolicy — independent axes a scope can carry),
crates/incin-core/src/tensor/grad.rs (no_grad / check_gradients scopes) and
crates/incin-core/src/exec/precision.rs (PrecisionPolicy presets and LossScaling growth/backoff).
"""
from __future__ import annotations

import contextlib
import enum
import threading
from dataclasses import dataclass, replace

from .dtype import DTypeId


class MathMode(enum.Enum):
    PRECISE = "precise"
    FAST = "fast"


class Determinism(enum.Enum):
    PERMITTED = "permitted"   # atomics / split-K reductions in any order are fine
    REQUIRED = "required"     # fixed reduction order: split-K off, sorted embedding backward


class FallbackPolicy(enum.Enum):
    DENY = "deny"
    ALLOW_COMPOSITION = "allow_composition"   # build the op from smaller kernels (composed attention)
    ALLOW_TRANSFER = "allow_transfer"         # move to another device that has the kernel


class AllocatorPolicy(enum.Enum):
    DIRECT = "direct"
    POOLED = "pooled"


class NanPolicy(enum.Enum):
    IGNORE = "ignore"
    REPORT = "report"   # backward reports non-finite gradients instead of propagating them silently
    RAISE = "raise"


class GradMode(enum.Enum):
    ENABLED = "enabled"
    DISABLED = "disabled"


@dataclass(frozen=True)
class ExecutionPolicy:
    math: MathMode = MathMode.PRECISE
    determinism: Determinism = Determinism.PERMITTED
    fallback: FallbackPolicy = FallbackPolicy.ALLOW_COMPOSITION
    allocator: AllocatorPolicy = AllocatorPolicy.POOLED
    nan: NanPolicy = NanPolicy.IGNORE

    def cache_key(self) -> str:
        """Stable text used in kernel / autotune cache keys so two policies never alias."""
        return "|".join((self.math.value, self.determinism.value, self.fallback.value, self.allocator.value,
                         self.nan.value))


_tls = threading.local()


def current_policy() -> ExecutionPolicy:
    return getattr(_tls, "policy", None) or ExecutionPolicy()


@contextlib.contextmanager
def policy_scope(**changes):
    """``with policy_scope(determinism=Determinism.REQUIRED): ...`` — nested scopes restore on exit."""
    prev = getattr(_tls, "policy", None)
    _tls.policy = replace(current_policy(), **changes)
    try:
        yield _tls.policy
    finally:
        _tls.policy = prev


def grad_mode() -> GradMode:
    import torch
    return GradMode.ENABLED if torch.is_grad_enabled() else GradMode.DISABLED


@contextlib.contextmanager
def no_grad():
    import torch
    with torch.no_grad():
        yield


@contextlib.contextmanager
def check_gradients():
    """Backward passes inside the scope report non-finite gradients (NanPolicy.REPORT)."""
    with policy_scope(nan=NanPolicy.REPORT) as p:
        yield p


# --------------------------------------------------------------------------------------------- precision
class LossScaling:
    """``none`` / ``static(scale)`` / ``dynamic``: halve on overflow (never below 1), double after
    ``growth_interval`` clean steps."""

    def __init__(self, kind: str = "none", scale: float = 1.0, growth_factor: float = 2.0,
                 backoff_factor: float = 0.5, growth_interval: int = 2000):
        assert kind in ("none", "static", "dynamic")
        self.kind = kind
        self._scale = float(scale) if kind != "none" else 1.0
        self.growth_factor, self.backoff_factor, self.growth_interval = growth_factor, backoff_factor, growth_interval
        self.steps_since_last_overflow = 0

    @staticmethod
    def none() -> "LossScaling":
        return LossScaling("none")

    @staticmethod
    def static(scale: float) -> "LossScaling":
        return LossScaling("static", scale)

    @staticmethod
    def dynamic_default() -> "LossScaling":
        return LossScaling("dynamic", 65536.0, 2.0, 0.5, 2000)

    @staticmethod
    def dynamic(initial_scale, growth_factor, backoff_factor, growth_interval) -> "LossScaling":
        return LossScaling("dynamic", initial_scale, growth_factor, backoff_factor, growth_interval)

    def scale(self) -> float:
        return self._scale

    def update(self, found_nan_or_inf: bool) -> None:
        if self.kind != "dynamic":
            return
        if found_nan_or_inf:
            self._scale = max(self._scale * self.backoff_factor, 1.0)
            self.steps_since_last_overflow = 0
        else:
            self.steps_since_last_overflow += 1
            if self.steps_since_last_overflow >= self.growth_interval:
                self._scale *= self.growth_factor
                self.steps_since_last_overflow = 0


@dataclass
class PrecisionPolicy:
    parameter: DTypeId
    compute: DTypeId
    accumulator: DTypeId
    output: DTypeId
    loss_scaling: LossScaling

    @staticmethod
    def fp32() -> "PrecisionPolicy":
        return PrecisionPolicy(DTypeId.F32, DTypeId.F32, DTypeId.F32, DTypeId.F32, LossScaling.none())

    @staticmethod
    def mixed_f16() -> "PrecisionPolicy":
        return PrecisionPolicy(DTypeId.F32, DTypeId.F16, DTypeId.F32, DTypeId.F16, LossScaling.dynamic_default())

    @staticmethod
    def mixed_bf16() -> "PrecisionPolicy":
        """fp32 master parameters, bf16 tensor-core compute, fp32 accumulation: the sm_100a training path."""
        return PrecisionPolicy(DTypeId.F32, DTypeId.BF16, DTypeId.F32, DTypeId.BF16, LossScaling.none())
