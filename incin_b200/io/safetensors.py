"""safetensors reader/writer (own implementation: 8-byte little-endian header length, JSON header,
raw little-endian tensor bytes) with atomic replace and resource limits.

Counterpart of ``save_safetensors`` / ``load_safetensors`` (crates/incin-core/src/nn/save.rs:237-298:
tmp file + rename; dtype map F32/F64/F16/BF16/I64/U32/U8 :184-198,253-267).
"""
from __future__ import annotations

import json
import os
import struct
from pathlib import Path

import torch

from .limits import DEFAULT_LIMITS, LimitError, ResourceLimits

_ST = {torch.float32: "F32", torch.float64: "F64", torch.float16: "F16", torch.bfloat16: "BF16", torch.int64: "I64",
       torch.uint32: "U32", torch.uint8: "U8", torch.int32: "I32", torch.bool: "BOOL"}
_TS = {v: k for k, v in _ST.items()}


def _bytes(t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous()
    return t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""   # reshape: 0-dim tensors too


def save_safetensors(tensors: dict[str, torch.Tensor], path, metadata: dict[str, str] | None = None) -> None:
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs, off = [], 0
    for name in sorted(tensors):
        t = tensors[name]
        if t.dtype not in _ST:
            raise TypeError(f"{name}: dtype {t.dtype} has no safetensors name")
        b = _bytes(t)
        header[name] = {"dtype": _ST[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    path = Path(path)
    tmp = path.with_name(path.name + f".tmp{os.getpid()}")
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)   # readers see the old file or the new one, never a torn one


def read_header(path, limits: ResourceLimits = DEFAULT_LIMITS) -> tuple[dict, int]:
    size = os.path.getsize(path)
    limits.check("file size", size, limits.max_file_bytes)
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise LimitError("file too short for a safetensors header")
        (n,) = struct.unpack("<Q", raw)
        limits.check("header size", n, min(limits.max_header_bytes, size - 8))
        try:
            header = json.loads(f.read(n))
        except (ValueError, UnicodeDecodeError) as e:
            raise LimitError(f"safetensors header is not valid JSON: {e}") from None
    if not isinstance(header, dict):
        raise LimitError("safetensors header is not an object")

    def _int(v) -> bool:
        return isinstance(v, int) and not isinstance(v, bool)
    limits.check("tensor count", len(header), limits.max_tensor_count)
    total = 0
    for name, meta in header.items():
        if name == "__metadata__":
            if not isinstance(meta, dict) or not all(isinstance(v, str) for v in meta.values()):
                raise LimitError("__metadata__ is not an object of strings")
            limits.check("metadata entries", len(meta), limits.max_metadata_entries)
            continue
        limits.check("name length", len(name.encode()), limits.max_name_bytes)
        # the header is untrusted: every entry must be {dtype: str, shape: [int >= 0], data_offsets: [int, int]}
        if not isinstance(meta, dict) or not isinstance(meta.get("dtype"), str):
            raise LimitError(f"{name}: entry is not an object with a dtype string")
        shape, offs = meta.get("shape"), meta.get("data_offsets")
        if not isinstance(shape, list) or not all(_int(d) and d >= 0 for d in shape):
            raise LimitError(f"{name}: shape is not a list of non-negative integers")
        if not isinstance(offs, list) or len(offs) != 2 or not all(_int(o) for o in offs):
            raise LimitError(f"{name}: data_offsets is not a pair of integers")
        limits.check("rank", len(meta["shape"]), limits.max_rank)
        for d in meta["shape"]:
            limits.check("dimension", d, limits.max_dimension)
        lo, hi = meta["data_offsets"]
        if not 0 <= lo <= hi <= size - 8 - n:
            raise LimitError(f"{name}: data offsets {lo}..{hi} outside the file")
        if meta["dtype"] not in _TS:
            raise LimitError(f"{name}: unknown dtype {meta['dtype']}")
        numel = 1
        for d in meta["shape"]:
            numel *= d
        if numel * torch.empty((), dtype=_TS[meta["dtype"]]).element_size() != hi - lo:
            raise LimitError(f"{name}: shape and byte range disagree")
        limits.check("tensor bytes", hi - lo, limits.max_tensor_bytes)
        total += hi - lo
    limits.check("total tensor bytes", total, limits.max_total_tensor_bytes)
    return header, 8 + n


def load_safetensors(path, limits: ResourceLimits = DEFAULT_LIMITS, names=None, *, threads: int = 0,
                     pin_memory: bool = False) -> dict[str, torch.Tensor]:
    """``threads > 0`` reads the tensor bytes with that many native readers straight into the result tensors
    (csrc/runtime/fileio.cpp; ``pin_memory`` makes those pinned, ready for an asynchronous copy to the device): the
    way to load multi-GB shards.  The header is validated against ``limits`` first in either case."""
    header, base = read_header(path, limits)
    out = {}
    if threads > 0:
        from ..runtime import read_ranges
        ranges = []
        for name, meta in header.items():
            if name == "__metadata__" or (names is not None and name not in names):
                continue
            lo, _ = meta["data_offsets"]
            t = torch.empty(meta["shape"], dtype=_TS[meta["dtype"]])
            if pin_memory and torch.cuda.is_available() and t.numel():
                t = t.pin_memory()
            out[name] = t
            ranges.append((base + lo, t))
        read_ranges(path, ranges, threads)
        return out
    with open(path, "rb") as f:
        for name, meta in header.items():
            if name == "__metadata__" or (names is not None and name not in names):
                continue
            lo, hi = meta["data_offsets"]
            f.seek(base + lo)
            buf = bytearray(f.read(hi - lo))
            t = torch.frombuffer(buf, dtype=torch.uint8).view(_TS[meta["dtype"]]) if hi > lo else \
                torch.empty(0, dtype=_TS[meta["dtype"]])
            out[name] = t.reshape(meta["shape"]).clone()
    return out


def load_metadata(path) -> dict[str, str]:
    return read_header(path)[0].get("__metadata__", {})
