"""Device meshes: spec, topology probing, collective groups, stable fingerprints, binding.

Counterpart of crates/incin-core/src/dist/mesh.rs: ``MeshSpec<Data<DP>, TensorParallel<TP>,
Pipeline<PP>>`` (:58-170), ``TopologyProbe`` / ``DeviceIdentity`` / ``LinkClass`` (:193-290),
``CollectiveGroups`` with ``rank = d*PP*TP + p*TP + t`` (:431-551), the FNV-1a ``TopologyFingerprint``
and ``MeshId`` (:553-691) and ``DeviceMesh::bind`` with its ordered guards (:787-1016).  The reference
fixes the world at two ranks; here any dp x tp x pp product up to the GPUs of one NVSwitch node binds.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Protocol, Sequence

from ..core.device import DeviceId, DeviceKind


class Digest:
    """Streaming FNV-1a 64: stable across processes and releases, unlike Python's hash()."""
    OFFSET, PRIME, MASK = 0xCBF29CE484222325, 0x100000001B3, (1 << 64) - 1

    def __init__(self, state: int | None = None):
        self.state = self.OFFSET if state is None else state

    def bytes(self, b: bytes) -> "Digest":
        s = self.state
        for x in b:
            s = ((s ^ x) * self.PRIME) & self.MASK
        self.state = s
        return self

    def number(self, v: int) -> "Digest":
        return self.bytes((v & self.MASK).to_bytes(8, "little"))

    def field(self, b: bytes) -> "Digest":
        return self.number(len(b)).bytes(b)

    def text(self, t: str) -> "Digest":
        return self.field(t.encode())

    def finish(self) -> int:
        return self.state


class Axis(enum.Enum):
    DATA = "data"
    TENSOR = "tensor"
    PIPELINE = "pipeline"


@dataclass(frozen=True)
class MeshSpec:
    """``mesh(dp=2, tp=4, pp=1)``: extents of the three parallel axes; world = dp * tp * pp."""
    dp: int = 1
    tp: int = 1
    pp: int = 1

    def __post_init__(self):
        for n, v in (("dp", self.dp), ("tp", self.tp), ("pp", self.pp)):
            if v < 1:
                raise ValueError(f"mesh axis {n} must be >= 1")

    @property
    def world(self) -> int:
        return self.dp * self.tp * self.pp

    def extent(self, axis: Axis) -> int:
        return {Axis.DATA: self.dp, Axis.TENSOR: self.tp, Axis.PIPELINE: self.pp}[axis]

    def rank_of(self, d: int, p: int, t: int) -> int:
        return d * self.pp * self.tp + p * self.tp + t

    def coords(self, rank: int) -> tuple[int, int, int]:
        """(data, pipeline, tensor) coordinates of a rank."""
        t = rank % self.tp
        p = (rank // self.tp) % self.pp
        d = rank // (self.tp * self.pp)
        return d, p, t


def mesh(dp: int = 1, tp: int = 1, pp: int = 1) -> MeshSpec:
    return MeshSpec(dp, tp, pp)


class LinkClass(enum.Enum):
    SAME_DEVICE = "same_device"
    HIGH_BANDWIDTH = "high_bandwidth"   # NVLink / NVSwitch
    PEER_CAPABLE = "peer_capable"       # PCIe P2P
    HOST_BOUNCE = "host_bounce"
    NETWORK = "network"
    UNREACHABLE = "unreachable"

    @property
    def weight(self) -> int:
        """Relative cost used by the hybrid planner (crates/incin-core/src/dist/plan.rs:956-1054)."""
        return {"same_device": 1, "high_bandwidth": 2, "peer_capable": 3, "host_bounce": 6, "network": 8,
                "unreachable": 1 << 20}[self.value]


@dataclass(frozen=True)
class DeviceIdentity:
    persistent_id: str      # GPU UUID: the ordinal is not an identity (visibility masks alias ordinals)
    family: str             # backend family, e.g. "cuda"
    architecture: str       # e.g. "sm_100"
    memory_bytes: int = 0


class TopologyProbe(Protocol):
    def identity(self, device: DeviceId) -> DeviceIdentity | None: ...
    def link(self, a: DeviceId, b: DeviceId) -> LinkClass: ...


class CudaTopologyProbe:
    """Real probe: CUDA device properties + peer-access capability, refined by NVML where it is importable: a pair that
    NVML reports as NVLink-connected is HIGH_BANDWIDTH, a pair that can only reach each other's memory over PCIe is
    PEER_CAPABLE, a pair without peer access bounces through the host.  NVML is only READ (P2P status queries);
    ``nvml`` takes a stand-in module for tests."""

    def __init__(self, nvml=None):
        self._nvml, self._nvml_ready = nvml, nvml is not None
        if nvml is None:
            try:
                import pynvml
                pynvml.nvmlInit()
                self._nvml, self._nvml_ready = pynvml, True
            except Exception:           # no NVML on this machine: peer access alone decides
                self._nvml, self._nvml_ready = None, False

    def _nvlink(self, a: int, b: int) -> bool | None:
        """True / False from NVML, None when NVML cannot say."""
        if not self._nvml_ready:
            return None
        n = self._nvml
        try:
            ha, hb = self._handle(a), self._handle(b)
            return n.nvmlDeviceGetP2PStatus(ha, hb, n.NVML_P2P_CAPS_INDEX_NVLINK) == n.NVML_P2P_STATUS_OK
        except Exception:
            return None

    def _handle(self, cuda_index: int):
        """NVML handle of a CUDA device: by UUID where both sides know it (NVML numbers every GPU of the machine, CUDA
        only the visible ones), by index otherwise."""
        n = self._nvml
        by_uuid = getattr(n, "nvmlDeviceGetHandleByUUID", None)
        if by_uuid is not None:
            try:
                import torch
                uuid = str(torch.cuda.get_device_properties(cuda_index).uuid)
                return by_uuid(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
            except Exception:
                pass
        return n.nvmlDeviceGetHandleByIndex(cuda_index)

    def identity(self, device: DeviceId) -> DeviceIdentity | None:
        import torch
        if device.kind is not DeviceKind.CUDA or not torch.cuda.is_available() or device.index >= torch.cuda.device_count():
            return None
        p = torch.cuda.get_device_properties(device.index)
        return DeviceIdentity(str(getattr(p, "uuid", f"cuda-{device.index}")), "cuda", f"sm_{p.major}{p.minor}",
                              p.total_memory)

    def link(self, a: DeviceId, b: DeviceId) -> LinkClass:
        import torch
        if a == b:
            return LinkClass.SAME_DEVICE
        try:
            ok = torch.cuda.can_device_access_peer(a.index, b.index)
        except Exception:
            return LinkClass.UNREACHABLE
        if not ok:
            return LinkClass.HOST_BOUNCE
        nvlink = self._nvlink(a.index, b.index)
        return LinkClass.PEER_CAPABLE if nvlink is False else LinkClass.HIGH_BANDWIDTH


class BindErrorKind(enum.Enum):
    RANK_COUNT = "rank_count"
    REPEATED_DEVICE = "repeated_device"
    UNKNOWN_DEVICE = "unknown_device"
    ALIASED_DEVICE = "aliased_device"
    MIXED_BACKEND_FAMILY = "mixed_backend_family"
    MIXED_ARCHITECTURE = "mixed_architecture"
    UNREACHABLE_PEER = "unreachable_peer"
    INSUFFICIENT_LINK = "insufficient_link"


class BindError(ValueError):
    def __init__(self, kind: BindErrorKind, message: str):
        super().__init__(f"{kind.value}: {message}")
        self.kind = kind


@dataclass(frozen=True)
class CollectiveGroup:
    axis: Axis
    index: int
    ranks: tuple[int, ...]
    link: LinkClass

    def token(self) -> str:
        return f"{self.axis.value}:{self.index}"


@dataclass(frozen=True)
class DeviceMesh:
    spec: MeshSpec
    devices: tuple[DeviceId, ...]
    identities: tuple[DeviceIdentity, ...]
    groups: tuple[CollectiveGroup, ...]
    fingerprint: int        # topology fingerprint: identities + link classes
    mesh_id: int            # fingerprint + axis extents: what plans are hashed against

    def group_of(self, rank: int, axis: Axis) -> CollectiveGroup:
        for g in self.groups:
            if g.axis is axis and rank in g.ranks:
                return g
        raise KeyError((rank, axis))

    @staticmethod
    def bind(spec: MeshSpec, devices: Sequence[DeviceId], probe: TopologyProbe,
             minimum_link: LinkClass = LinkClass.NETWORK) -> "DeviceMesh":
        """Ordered guards; the first failing one names the misconfiguration."""
        devices = tuple(devices)
        if len(devices) != spec.world:
            raise BindError(BindErrorKind.RANK_COUNT, f"mesh world is {spec.world}, got {len(devices)} devices")
        seen: dict[DeviceId, int] = {}
        for r, d in enumerate(devices):
            if d in seen:
                raise BindError(BindErrorKind.REPEATED_DEVICE, f"{d} given for ranks {seen[d]} and {r}")
            seen[d] = r
        ids = []
        for r, d in enumerate(devices):
            ident = probe.identity(d)
            if ident is None:
                raise BindError(BindErrorKind.UNKNOWN_DEVICE, f"rank {r}: {d} names no installed device")
            ids.append(ident)
        by_pid: dict[str, int] = {}
        for r, ident in enumerate(ids):
            if ident.persistent_id in by_pid:
                raise BindError(BindErrorKind.ALIASED_DEVICE,
                                f"ranks {by_pid[ident.persistent_id]} and {r} are the same device {ident.persistent_id}")
            by_pid[ident.persistent_id] = r
        for r, ident in enumerate(ids):
            if ident.family != ids[0].family:
                raise BindError(BindErrorKind.MIXED_BACKEND_FAMILY, f"rank {r} is {ident.family}, rank 0 is {ids[0].family}")
        for r, ident in enumerate(ids):
            if ident.architecture != ids[0].architecture:
                raise BindError(BindErrorKind.MIXED_ARCHITECTURE,
                                f"rank {r} is {ident.architecture}, rank 0 is {ids[0].architecture}")
        groups: list[CollectiveGroup] = []
        for axis in (Axis.DATA, Axis.TENSOR, Axis.PIPELINE):
            for gi, ranks in enumerate(_axis_groups(spec, axis)):
                worst = LinkClass.SAME_DEVICE
                for i in ranks:
                    for j in ranks:
                        if i < j:
                            lk = probe.link(devices[i], devices[j])
                            if lk is LinkClass.UNREACHABLE:
                                raise BindError(BindErrorKind.UNREACHABLE_PEER,
                                                f"{axis.value} group {gi}: ranks {i} and {j} cannot reach each other")
                            if lk.weight > worst.weight:
                                worst = lk
                if worst.weight > minimum_link.weight:
                    raise BindError(BindErrorKind.INSUFFICIENT_LINK,
                                    f"{axis.value} group {gi} is connected by {worst.value}, need {minimum_link.value}")
                groups.append(CollectiveGroup(axis, gi, tuple(ranks), worst))
        fp = Digest().text("incin.topology.v1")
        for ident in ids:
            fp.text(ident.persistent_id).text(ident.family).text(ident.architecture)
        for g in groups:
            fp.text(g.token()).text(g.link.value)
        fingerprint = fp.finish()
        mid = Digest().text("incin.mesh.v1").number(fingerprint).number(spec.dp).number(spec.tp).number(spec.pp).finish()
        return DeviceMesh(spec, devices, tuple(ids), tuple(groups), fingerprint, mid)


def _axis_groups(spec: MeshSpec, axis: Axis) -> list[list[int]]:
    out = []
    if axis is Axis.TENSOR:
        for d in range(spec.dp):
            for p in range(spec.pp):
                out.append([spec.rank_of(d, p, t) for t in range(spec.tp)])
    elif axis is Axis.PIPELINE:
        for d in range(spec.dp):
            for t in range(spec.tp):
                out.append([spec.rank_of(d, p, t) for p in range(spec.pp)])
    else:
        for p in range(spec.pp):
            for t in range(spec.tp):
                out.append([spec.rank_of(d, p, t) for d in range(spec.dp)])
    return out
