"""Model / optimiser checkpoints in incin's tensor-name and dtype layout, with resharding.

Counterpart of crates/incin-core/src/nn/save.rs: ``save_checkpoint`` = ``manifest.json`` (version,
world_size, tensors{name, global_shape, dtype, placement_kind}) + ``model.safetensors`` (:302-328),
``slice_bytes_for_rank`` (:95-151) and ``load_resharded_checkpoint`` (one sharded axis per tensor, even
division, :332-435).  Name layout quirk reproduced on purpose: ``state_dict`` keys carry a trailing dot
(``"linear.weight."``, ``"0.bias."``; crates/incin/tests/serde_tests.rs:24,57) whereas
``named_parameters`` keys do not.  AdamW state uses ``m.<name>`` / ``v.<name>`` plus ``step_count``
(crates/incin-core/src/optim/mod.rs:127-195).  On top of that this build also stores the LR-scheduler
and RNG state the reference leaves out, under a separate ``trainer.json``.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass
from pathlib import Path

import torch

from ..core.dtype import DTypeId, from_torch, size_bytes, to_torch
from .limits import DEFAULT_LIMITS, ResourceLimits
from .safetensors import load_safetensors, save_safetensors

MANIFEST_VERSION = 1


def state_dict(module: torch.nn.Module) -> dict[str, torch.Tensor]:
    """incin-layout state dict: every key ends with a dot."""
    return {name + ".": p.detach() for name, p in module.state_dict().items()}


def load_state_dict(module: torch.nn.Module, sd: dict[str, torch.Tensor], strict: bool = True) -> None:
    plain = {(k[:-1] if k.endswith(".") else k): v for k, v in sd.items()}
    own = module.state_dict()
    missing = [k for k in own if k not in plain]
    unexpected = [k for k in plain if k not in own]
    if strict and (missing or unexpected):
        raise KeyError(f"state dict mismatch: missing {missing}, unexpected {unexpected}")
    with torch.no_grad():
        for k, v in plain.items():
            if k in own:
                if tuple(own[k].shape) != tuple(v.shape):
                    raise ValueError(f"{k}: checkpoint shape {tuple(v.shape)} != parameter shape {tuple(own[k].shape)}")
                own[k].copy_(v.to(own[k].dtype))


@dataclass
class TensorCheckpointMeta:
    name: str
    global_shape: list[int]
    dtype: str
    placement_kind: str           # "replicated" or "sharded:<axis>"


@dataclass
class GlobalCheckpointManifest:
    version: int
    world_size: int
    tensors: dict[str, TensorCheckpointMeta]

    def to_json(self) -> str:
        return json.dumps({"version": self.version, "world_size": self.world_size,
                           "tensors": {k: asdict(v) for k, v in sorted(self.tensors.items())}}, indent=1)

    @staticmethod
    def from_json(text: str) -> "GlobalCheckpointManifest":
        d = json.loads(text)
        return GlobalCheckpointManifest(d["version"], d["world_size"],
                                        {k: TensorCheckpointMeta(**v) for k, v in d["tensors"].items()})


def slice_bytes_for_rank(data: bytes, global_shape, dtype: DTypeId, shard_axis: int, rank: int,
                         world_size: int) -> tuple[bytes, list[int]]:
    """Rank's slice of a row-major tensor along ``shard_axis`` as raw bytes plus its local shape."""
    if shard_axis >= len(global_shape):
        raise ValueError(f"shard axis {shard_axis} out of bounds for shape {list(global_shape)}")
    gd = global_shape[shard_axis]
    if world_size == 0 or gd % world_size:
        raise ValueError(f"global dimension {gd} along axis {shard_axis} not divisible by world size {world_size}")
    if rank >= world_size:
        raise ValueError(f"rank {rank} out of bounds for world size {world_size}")
    local = gd // world_size
    shape = list(global_shape)
    shape[shard_axis] = local
    eb = size_bytes(dtype, 1)
    outer = 1
    for d in global_shape[:shard_axis]:
        outer *= d
    inner = 1
    for d in global_shape[shard_axis + 1:]:
        inner *= d
    shard_block, global_block = local * inner * eb, gd * inner * eb
    out = bytearray()
    for o in range(outer):
        lo = o * global_block + rank * shard_block
        if lo + shard_block > len(data):
            raise ValueError(f"byte slice {lo}..{lo + shard_block} outside a buffer of {len(data)} bytes")
        out += data[lo:lo + shard_block]
    return bytes(out), shape


def save_checkpoint(directory, module: torch.nn.Module, world_size: int = 1,
                    placements: dict[str, str] | None = None, optimizer=None, trainer_state: dict | None = None) -> None:
    """``placements[name] = "sharded:<axis>"`` records which tensors a tensor-parallel job splits; the file always
    holds GLOBAL tensors, so a checkpoint written at one world size loads at another."""
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    sd = state_dict(module)
    store = getattr(optimizer, "store", None)
    if store is not None:
        # flat optimiser: the module parameters are views of the low-precision shadow; the fp32 master weights are
        # the state to keep, under the same (trailing-dot) names
        for name, master in store.named_master():
            if name + "." in sd:
                sd[name + "."] = master.detach()
    placements = placements or {}
    man = GlobalCheckpointManifest(MANIFEST_VERSION, world_size, {})
    for k, t in sd.items():
        man.tensors[k] = TensorCheckpointMeta(k, list(t.shape), from_torch(t.dtype).value,
                                              placements.get(k.rstrip("."), "replicated"))
    save_safetensors({k: v for k, v in sd.items()}, d / "model.safetensors")
    if optimizer is not None:
        osd = optimizer.state_dict()
        step = osd.pop("step_count", 0)
        save_safetensors({k: v for k, v in osd.items()}, d / "optimizer.safetensors",
                         metadata={"step_count": str(step)})
    if trainer_state is not None:
        tmp = d / f"trainer.json.tmp{os.getpid()}"
        tmp.write_text(json.dumps(trainer_state))
        os.replace(tmp, d / "trainer.json")
    tmp = d / f"manifest.json.tmp{os.getpid()}"
    tmp.write_text(man.to_json())
    os.replace(tmp, d / "manifest.json")   # the manifest lands last: its presence marks a complete checkpoint


def load_checkpoint(directory, module: torch.nn.Module, optimizer=None, limits: ResourceLimits = DEFAULT_LIMITS,
                    threads: int = 0) -> dict:
    """``threads > 0`` reads the tensor files with that many native readers (see ``load_safetensors``)."""
    d = Path(directory)
    man = GlobalCheckpointManifest.from_json((d / "manifest.json").read_text())
    if man.version != MANIFEST_VERSION:
        raise ValueError(f"unsupported checkpoint manifest version {man.version}")
    sd = load_safetensors(d / "model.safetensors", limits, threads=threads)
    load_state_dict(module, sd)
    store = getattr(optimizer, "store", None)
    if store is not None:
        # the parameters just written are views of the shadow; the optimiser steps from the fp32 master, which
        # must receive the loaded values too (else the next step recomputes the shadow from stale masters)
        with torch.no_grad():
            for name, master in store.named_master():
                v = sd.get(name + ".", sd.get(name))
                if v is not None:
                    master.copy_(v.to(device=master.device, dtype=master.dtype).reshape(master.shape))
            store.sync_shadow_from_master()
    if optimizer is not None and (d / "optimizer.safetensors").exists():
        from .safetensors import load_metadata
        osd = load_safetensors(d / "optimizer.safetensors", limits, threads=threads)
        osd["step_count"] = int(load_metadata(d / "optimizer.safetensors").get("step_count", "0"))
        optimizer.load_state_dict(osd)
    tj = d / "trainer.json"
    return json.loads(tj.read_text()) if tj.exists() else {}


def load_resharded_checkpoint(directory, rank: int, world_size: int,
                              limits: ResourceLimits = DEFAULT_LIMITS, threads: int = 0) -> dict[str, torch.Tensor]:
    """Rank-local tensors for a job of ``world_size`` ranks, whatever world size wrote the checkpoint."""
    d = Path(directory)
    man = GlobalCheckpointManifest.from_json((d / "manifest.json").read_text())
    full = load_safetensors(d / "model.safetensors", limits, threads=threads)
    out = {}
    for name, meta in man.tensors.items():
        t = full[name]
        if meta.placement_kind.startswith("sharded:"):
            axis = int(meta.placement_kind.split(":")[1])
            dt = DTypeId(meta.dtype)
            raw, shape = slice_bytes_for_rank(t.contiguous().view(torch.uint8).numpy().tobytes(), meta.global_shape, dt,
                                              axis, rank, world_size)
            out[name] = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(to_torch(dt)).reshape(shape).clone()
        else:
            out[name] = t
    return out
