"""Distributed context: environment rendezvous, fail-stop state machine, launch plans.

Counterpart of crates/incin-core/src/dist/context.rs: env vars ``INCIN_{RANK, WORLD_SIZE,
RENDEZVOUS_ADDR, RUN_ID, LOCAL_CUDA_DEVICE, RENDEZVOUS_TIMEOUT_MS}`` (:42-52),
``DistributedContext::from_env`` (:513), states Active / ShuttingDown / Shutdown / Failed with a shared
handle that every transport operation checks and any transport error invalidates (:196-221),
``abort`` / ``wait_for_peer`` / ``shutdown`` (:382-461) and ``LaunchPlan`` / ``RankLaunch::environment``
(:270-280).  The wire protocol lives in C++ (csrc/comm/rendezvous.cpp) and works for any world size;
``torchrun``'s RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT are accepted as fallbacks so one launcher
serves both the rendezvous here and ``torch.distributed``.
"""
from __future__ import annotations

import ctypes as C
import enum
import os
from dataclasses import dataclass

from .. import _native as nat

ENV_RANK = "INCIN_RANK"
ENV_WORLD = "INCIN_WORLD_SIZE"
ENV_ADDR = "INCIN_RENDEZVOUS_ADDR"
ENV_RUN_ID = "INCIN_RUN_ID"
ENV_DEVICE = "INCIN_LOCAL_CUDA_DEVICE"
ENV_TIMEOUT = "INCIN_RENDEZVOUS_TIMEOUT_MS"


class ContextState(enum.Enum):
    ACTIVE = 0
    SHUTTING_DOWN = 1
    SHUTDOWN = 2
    FAILED = 3


class ContextFailure(enum.Enum):
    TIMEOUT = 1
    IO = 2
    BAD_MAGIC = 3
    WORLD_MISMATCH = 4
    BAD_RANK = 5
    RUN_ID_MISMATCH = 6
    REJECTED = 7
    BAD_STATE = 8
    PEER_ABORTED = 9
    BAD_ARGUMENT = 10
    DUPLICATE_RANK = 11
    DEVICE_TIMEOUT = 100     # a bounded device-side wait gave up (kernel status word)
    PLAN_MISMATCH = 101


class RendezvousError(RuntimeError):
    def __init__(self, failure: ContextFailure, what: str = ""):
        super().__init__(f"{what + ': ' if what else ''}{failure.name.lower()}")
        self.failure = failure


def _fail(code: int, what: str):
    try:
        f = ContextFailure(code)
    except ValueError:
        f = ContextFailure.IO
    raise RendezvousError(f, what)


@dataclass(frozen=True)
class RendezvousConfig:
    rank: int
    world: int
    addr: str
    run_id: str
    local_device: int = 0
    timeout_ms: int = 30000

    @staticmethod
    def from_env(env=None) -> "RendezvousConfig":
        e = os.environ if env is None else env
        rank = e.get(ENV_RANK, e.get("RANK"))
        world = e.get(ENV_WORLD, e.get("WORLD_SIZE"))
        if rank is None or world is None:
            raise KeyError(f"{ENV_RANK} and {ENV_WORLD} (or RANK / WORLD_SIZE) must be set")
        addr = e.get(ENV_ADDR)
        if addr is None:
            addr = f"{e.get('MASTER_ADDR', '127.0.0.1')}:{int(e.get('MASTER_PORT', '29400')) + 1}"
        return RendezvousConfig(int(rank), int(world), addr, e.get(ENV_RUN_ID, "incin-run"),
                                int(e.get(ENV_DEVICE, e.get("LOCAL_RANK", "0"))), int(e.get(ENV_TIMEOUT, "30000")))


@dataclass(frozen=True)
class RankLaunch:
    rank: int
    config: RendezvousConfig

    def environment(self) -> dict[str, str]:
        c = self.config
        return {ENV_RANK: str(c.rank), ENV_WORLD: str(c.world), ENV_ADDR: c.addr, ENV_RUN_ID: c.run_id,
                ENV_DEVICE: str(c.local_device), ENV_TIMEOUT: str(c.timeout_ms)}


def launch_plan(world: int, addr: str, run_id: str, devices=None, timeout_ms: int = 30000) -> list[RankLaunch]:
    """One :class:`RankLaunch` per rank; ``environment()`` is what a process launcher exports."""
    devices = list(devices) if devices is not None else list(range(world))
    if len(devices) != world:
        raise ValueError("one local device per rank")
    return [RankLaunch(r, RendezvousConfig(r, world, addr, run_id, devices[r], timeout_ms)) for r in range(world)]


def _lib():
    h = nat.host()
    if not getattr(h, "_rdv_bound", False):
        h.incin_rdv_connect.restype = C.c_int
        h.incin_rdv_connect.argtypes = [C.c_int, C.c_int, C.c_char_p, C.c_char_p, C.c_int64, C.c_int,
                                        C.POINTER(C.c_int64)]
        for name, args in (("incin_rdv_state", [C.c_int64]), ("incin_rdv_failure_code", [C.c_int64]),
                           ("incin_rdv_ensure_active", [C.c_int64]), ("incin_rdv_abort", [C.c_int64, C.c_int, C.c_int]),
                           ("incin_rdv_shutdown", [C.c_int64, C.c_int]),
                           ("incin_rdv_wait_for_peer", [C.c_int64, C.c_int] + [C.POINTER(C.c_int)] * 3),
                           ("incin_rdv_allgather", [C.c_int64, C.c_void_p, C.c_int, C.c_void_p, C.c_int])):
            getattr(h, name).restype = C.c_int
            getattr(h, name).argtypes = args
        h.incin_rdv_invalidate.restype = None
        h.incin_rdv_invalidate.argtypes = [C.c_int64, C.c_int]
        h.incin_rdv_destroy.restype = None
        h.incin_rdv_destroy.argtypes = [C.c_int64]
        h.incin_rdv_peer_device.restype = C.c_int64
        h.incin_rdv_peer_device.argtypes = [C.c_int64, C.c_int]
        h._rdv_bound = True
    return h


class DistributedContext:
    """Owns the control channel of one rank.  Every distributed operation goes through ``ensure_active``;
    any failure calls ``invalidate`` so later operations fail fast instead of hanging (fail-stop)."""

    def __init__(self, config: RendezvousConfig, handle: int):
        self.config, self._h = config, handle

    @staticmethod
    def rendezvous(config: RendezvousConfig) -> "DistributedContext":
        h = C.c_int64()
        rc = _lib().incin_rdv_connect(config.rank, config.world, config.addr.encode(), config.run_id.encode(),
                                      config.local_device, config.timeout_ms, C.byref(h))
        if rc:
            _fail(rc, f"rendezvous of rank {config.rank}/{config.world} at {config.addr}")
        return DistributedContext(config, h.value)

    @staticmethod
    def from_env(env=None) -> "DistributedContext":
        return DistributedContext.rendezvous(RendezvousConfig.from_env(env))

    @property
    def rank(self) -> int:
        return self.config.rank

    @property
    def world(self) -> int:
        return self.config.world

    @property
    def state(self) -> ContextState:
        return ContextState(_lib().incin_rdv_state(self._h))

    def ensure_active(self) -> None:
        if _lib().incin_rdv_ensure_active(self._h):
            raise RendezvousError(ContextFailure.BAD_STATE, f"context is {self.state.name.lower()}")

    def invalidate(self, failure: ContextFailure) -> None:
        _lib().incin_rdv_invalidate(self._h, failure.value)

    def abort(self, failure: ContextFailure = ContextFailure.PEER_ABORTED, timeout_ms: int = 2000) -> None:
        """Tell every peer this rank failed; all contexts of the job end up Failed."""
        _lib().incin_rdv_abort(self._h, failure.value, timeout_ms)

    def wait_for_peer(self, timeout_ms: int):
        """Next control message ``(kind, code, from_rank)`` or None on timeout; raises if a peer vanished."""
        k, c, f = C.c_int(), C.c_int(), C.c_int()
        rc = _lib().incin_rdv_wait_for_peer(self._h, timeout_ms, C.byref(k), C.byref(c), C.byref(f))
        if rc == ContextFailure.TIMEOUT.value:
            return None
        if rc:
            _fail(rc, "wait_for_peer")
        return k.value, c.value, f.value

    def allgather_bytes(self, blob: bytes, timeout_ms: int = 30000) -> list[bytes]:
        """All-gather of one equal-size blob per rank over the control star (plan hashes, IPC handles)."""
        self.ensure_active()
        n = len(blob)
        out = C.create_string_buffer(n * self.world)
        rc = _lib().incin_rdv_allgather(self._h, blob, n, out, timeout_ms)
        if rc:
            _fail(rc, "allgather")
        return [out.raw[i * n:(i + 1) * n] for i in range(self.world)]

    def preflight(self, plan) -> "object":
        """Exchange (mesh id, plan hash, count) and reject divergent ranks before any communicator exists."""
        from .plan import PreflightError, preflight
        mine = plan.mesh_id.to_bytes(8, "little") + plan.hash.to_bytes(8, "little") + len(plan.descriptors).to_bytes(8, "little")
        reports = [(int.from_bytes(b[:8], "little"), int.from_bytes(b[8:16], "little"), int.from_bytes(b[16:], "little"))
                   for b in self.allgather_bytes(mine)]
        try:
            return preflight(self.world, reports, plan)
        except PreflightError:
            self.invalidate(ContextFailure.PLAN_MISMATCH)
            raise

    def peer_device(self, rank: int) -> int:
        return _lib().incin_rdv_peer_device(self._h, rank)

    def shutdown(self, timeout_ms: int = 10000) -> None:
        rc = _lib().incin_rdv_shutdown(self._h, timeout_ms)
        if rc:
            _fail(rc, "shutdown")

    def close(self) -> None:
        if self._h:
            _lib().incin_rdv_destroy(self._h)
            self._h = 0
