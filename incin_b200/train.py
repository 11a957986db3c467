"""``Trainer``: plan devices, explain the plan, fit.

Counterpart of crates/incin/src/train.rs: ``Trainer::plan().devices(..).epochs(n).build() -> Plan`` with
stable decision codes and ``explain()`` / ``explain_json()`` (:137-207), the ``Machine`` probe trait
(:68-101), ``TrainError`` (:220-255) and ``Trainer::new(plan).fit(model, opt, loader, loss_fn)`` (:546-617).
The reference refuses a multi-device fit (:594-598); here a multi-device plan runs data parallel with the
fused peer-memory reducer when the process was launched one-per-GPU (``torch.distributed`` initialised and
world size == number of planned devices).
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Callable, Iterable, Protocol

import torch

from .core.device import Cpu, DeviceId, DeviceKind, DeviceSet, cuda_available
from .engine import TrainStep
from . import telemetry


class TrainError(RuntimeError):
    pass


class NotCompiledIn(TrainError):
    pass


class DeviceUnavailable(TrainError):
    pass


class NoDeviceAvailable(TrainError):
    pass


class CollectivesUnavailable(TrainError):
    pass


class StepError(TrainError):
    pass


class Machine(Protocol):
    def compiled_in(self, kind: DeviceKind) -> bool: ...
    def has_device(self, device: DeviceId) -> bool: ...
    def collectives_available(self, n: int) -> bool: ...


class HostMachine:
    """The real machine: CUDA is compiled in when the sm_100a library exists or can be built."""

    def compiled_in(self, kind: DeviceKind) -> bool:
        if kind is DeviceKind.CPU:
            return True
        if kind is DeviceKind.CUDA:
            from . import _native, _build
            return _native.cuda_library_path().exists() or _build._nvcc() is not None
        return False   # wgpu / metal: graphics-API backends, not part of this build

    def has_device(self, device: DeviceId) -> bool:
        if device.kind is DeviceKind.CPU:
            return True
        return device.kind is DeviceKind.CUDA and cuda_available() and device.index < torch.cuda.device_count()

    def collectives_available(self, n: int) -> bool:
        import torch.distributed as dist
        return dist.is_available() and dist.is_initialized() and dist.get_world_size() == n


@dataclass(frozen=True)
class Decision:
    code: str
    detail: str


@dataclass(frozen=True)
class Plan:
    devices: DeviceSet
    epochs: int
    decisions: tuple[Decision, ...]

    @property
    def is_multi_device(self) -> bool:
        return len(self.devices) > 1

    def explain(self) -> str:
        return "\n".join(f"[{d.code}] {d.detail}" for d in self.decisions)

    def explain_json(self) -> str:
        return json.dumps({"devices": [str(d) for d in self.devices], "epochs": self.epochs,
                           "decisions": [{"code": d.code, "detail": d.detail} for d in self.decisions]})


class TrainerBuilder:
    def __init__(self):
        self._devices: DeviceSet | None = None
        self._epochs = 1

    def devices(self, devices: DeviceSet) -> "TrainerBuilder":
        self._devices = devices
        return self

    def epochs(self, n: int) -> "TrainerBuilder":
        if n < 1:
            raise ValueError("epochs must be >= 1")
        self._epochs = n
        return self

    def build(self) -> Plan:
        return self.build_on(HostMachine())

    def build_on(self, machine: Machine) -> Plan:
        ds: list[Decision] = []
        want = self._devices or DeviceSet.cpu()
        ds.append(Decision("devices-requested", f"{want}" if self._devices else "none requested: the default backend is the CPU"))
        if not machine.compiled_in(want.kind):
            ds.append(Decision("family-not-compiled", f"{want.kind.value} support is not part of this build"))
            raise NotCompiledIn(ds[-1].detail)
        missing = [d for d in want if not machine.has_device(d)]
        if missing:
            ds.append(Decision("family-unavailable", f"{', '.join(map(str, missing))} not present on this machine"))
            raise DeviceUnavailable(ds[-1].detail)
        ds.append(Decision("devices-resolved", f"{len(want)} device(s): {want}"))
        if len(want) > 1:
            ds.append(Decision("collectives-required",
                               f"{len(want)} devices train data-parallel: one process per GPU, gradients reduced by the "
                               "fused peer-memory kernel over NVLink"))
        ds.append(Decision("epochs", f"{self._epochs} epoch(s)"))
        return Plan(want, self._epochs, tuple(ds))


class Trainer:
    def __init__(self, plan: Plan, machine: Machine | None = None):
        self.plan, self.machine = plan, machine or HostMachine()
        self.history: list[float] = []

    @staticmethod
    def plan() -> TrainerBuilder:
        return TrainerBuilder()

    def _local_device(self) -> torch.device:
        if self.plan.devices.kind is DeviceKind.CPU:
            return torch.device("cpu")
        if self.plan.is_multi_device:
            import torch.distributed as dist
            return self.plan.devices.devices[dist.get_rank()].torch()
        return self.plan.devices.devices[0].torch()

    def fit(self, model: torch.nn.Module, optimizer, loader: Iterable, loss_fn: Callable | None = None, *,
            scheduler=None, use_graph: bool = True, on_step: Callable[[int, float], None] | None = None,
            log_every: int = 1) -> list[float]:
        """``loss_fn(model, *batch) -> scalar loss``.  ``optimizer`` is a flat optimiser over the model's
        :class:`ParamStore`.  Returns the per-step losses (read back to the host every ``log_every`` steps)."""
        reducer = None
        if self.plan.is_multi_device:
            if not self.machine.collectives_available(len(self.plan.devices)):
                raise CollectivesUnavailable(
                    f"a {len(self.plan.devices)}-device plan needs {len(self.plan.devices)} processes with "
                    "torch.distributed initialised (launch with python -m torch.distributed.run)")
            reducer = getattr(optimizer, "reducer", None)
            if reducer is None:
                raise CollectivesUnavailable("build the optimiser with incin_b200.parallel.dp.make_reducer for a multi-device fit")
        device = self._local_device()
        step = TrainStep(model, optimizer, loss_fn=loss_fn, use_graph=use_graph, reducer=reducer)
        n = 0
        for epoch in range(self.plan.epochs):
            for batch in loader:
                batch = batch if isinstance(batch, (tuple, list)) else (batch,)
                batch = tuple(b.to(device, non_blocking=True) if isinstance(b, torch.Tensor) else b for b in batch)
                try:
                    loss = step(*batch)
                except Exception as e:   # surface the step index with the failure
                    raise StepError(f"step {n} failed: {e}") from e
                n += 1
                if scheduler is not None:
                    scheduler.step()
                if n % log_every == 0:
                    v = float(loss)
                    self.history.append(v)
                    telemetry.emit_scalar("loss", v, n)
                    if on_step:
                        on_step(n, v)
            telemetry.emit_epoch(epoch + 1, steps=n)
        if device.type == "cuda":
            from .ops.gemm import check_status
            check_status(device)
        return self.history
