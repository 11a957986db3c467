"""Device vocabulary: kinds, ids, sets, preferences and detection.

Counterpart of crates/incin-core/src/tensor/device.rs (Cpu, Cuda(n), DeviceKind, DeviceId, DeviceSet,
DevicePreference) and crates/incin-backends/src/detect.rs (probe order CUDA first, CPU last; the
default backend stays the CPU whatever accelerators are present).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Iterable, Iterator

import torch


class DeviceKind(enum.Enum):
    CPU = "cpu"
    CUDA = "cuda"
    WGPU = "wgpu"    # graphics-API backends of the reference: named, never available here
    METAL = "metal"


@dataclass(frozen=True, order=True)
class DeviceId:
    kind: DeviceKind
    index: int = 0

    def torch(self) -> torch.device:
        if self.kind is DeviceKind.CPU:
            return torch.device("cpu")
        if self.kind is DeviceKind.CUDA:
            return torch.device("cuda", self.index)
        raise RuntimeError(f"{self.kind.value} devices are not available in this build")

    def __str__(self) -> str:
        return "cpu" if self.kind is DeviceKind.CPU else f"{self.kind.value}:{self.index}"


Cpu = DeviceId(DeviceKind.CPU, 0)


def Cuda(index: int = 0) -> DeviceId:
    if index < 0:
        raise ValueError("device index must be >= 0")
    return DeviceId(DeviceKind.CUDA, index)


class DeviceSetError(ValueError):
    pass


class DeviceSet:
    """An ordered, duplicate-free, single-kind set of devices (what a Trainer plan runs on)."""

    def __init__(self, devices: Iterable[DeviceId]):
        devs = list(devices)
        if not devs:
            raise DeviceSetError("a device set cannot be empty")
        if len(set(devs)) != len(devs):
            raise DeviceSetError("duplicate device in set")
        if len({d.kind for d in devs}) != 1:
            raise DeviceSetError("a device set holds devices of one kind")
        self.devices = tuple(devs)

    @staticmethod
    def cpu() -> "DeviceSet":
        return DeviceSet([Cpu])

    @staticmethod
    def cuda(indices: Iterable[int] | range) -> "DeviceSet":
        return DeviceSet([Cuda(i) for i in indices])

    @property
    def kind(self) -> DeviceKind:
        return self.devices[0].kind

    def __len__(self) -> int:
        return len(self.devices)

    def __iter__(self) -> Iterator[DeviceId]:
        return iter(self.devices)

    def __repr__(self) -> str:
        return "DeviceSet(" + ", ".join(map(str, self.devices)) + ")"


class DevicePreference(enum.Enum):
    DEFAULT = "default"          # the CPU: enabling an accelerator never changes the default backend
    FASTEST = "fastest"          # first available in probe order
    CPU_ONLY = "cpu"
    CUDA_ONLY = "cuda"


def cuda_available() -> bool:
    try:
        return torch.cuda.is_available()
    except Exception:
        return False


def detect_device(preference: DevicePreference = DevicePreference.FASTEST) -> DeviceId:
    """Probe order CUDA -> CPU (Metal and WGPU are never present in this build)."""
    if preference in (DevicePreference.DEFAULT, DevicePreference.CPU_ONLY):
        return Cpu
    if cuda_available():
        return Cuda(torch.cuda.current_device())
    if preference is DevicePreference.CUDA_ONLY:
        raise RuntimeError("no CUDA device is visible")
    return Cpu
