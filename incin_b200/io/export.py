"""Exporters and file inspection: GGUF (F32 / F16 / Q8_0 tensors), MLX-style safetensors, ``inspect_file``.

Counterparts: crates/incin-core/src/io/gguf.rs:17-185, io/mlx.rs:10-34, io/inspect.rs:28.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass
from pathlib import Path

import torch

from ..ops.quant import quantize_q8_0
from .limits import DEFAULT_LIMITS, LimitError, ResourceLimits
from .safetensors import read_header, save_safetensors

GGUF_MAGIC = b"GGUF"
GGUF_VERSION = 3
GGML_F32, GGML_F16, GGML_Q8_0, GGML_BF16 = 0, 1, 8, 30
_ALIGN = 32


def _gstr(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def export_gguf(tensors: dict[str, torch.Tensor], path, *, quantize: str = "none", metadata: dict | None = None) -> None:
    """``quantize='q8_0'`` packs every 2-D tensor whose row length is a multiple of 32; the rest stay f32."""
    infos, blobs, off = [], [], 0
    for name in sorted(tensors):
        t = tensors[name].detach().cpu()
        if quantize == "q8_0" and t.dim() == 2 and t.shape[1] % 32 == 0:
            data, typ = quantize_q8_0(t).numpy().tobytes(), GGML_Q8_0
        elif t.dtype == torch.float16:
            data, typ = t.contiguous().view(torch.uint8).numpy().tobytes(), GGML_F16
        else:
            data, typ = t.float().contiguous().view(torch.uint8).numpy().tobytes(), GGML_F32
        infos.append((name, list(reversed(t.shape)), typ, off))   # GGML lists the innermost dimension first
        pad = (-len(data)) % _ALIGN
        blobs.append(data + b"\0" * pad)
        off += len(data) + pad
    kv = {"general.architecture": "incin", "general.alignment": _ALIGN}
    kv.update(metadata or {})
    head = GGUF_MAGIC + struct.pack("<IQQ", GGUF_VERSION, len(infos), len(kv))
    for k, v in kv.items():
        head += _gstr(k)
        if isinstance(v, int):
            head += struct.pack("<IQ", 10, v)      # GGUF_TYPE_UINT64
        else:
            head += struct.pack("<I", 8) + _gstr(str(v))   # GGUF_TYPE_STRING
    for name, dims, typ, o in infos:
        head += _gstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        head += struct.pack("<IQ", typ, o)
    head += b"\0" * ((-len(head)) % _ALIGN)
    with open(path, "wb") as f:
        f.write(head)
        for b in blobs:
            f.write(b)


def read_gguf_index(path, limits: ResourceLimits = DEFAULT_LIMITS) -> dict:
    """Header + tensor table of a GGUF file (enough to verify an export and to inspect foreign files)."""
    data = Path(path).read_bytes()
    limits.check("file size", len(data), limits.max_file_bytes)
    if data[:4] != GGUF_MAGIC:
        raise LimitError("not a GGUF file")
    pos = 4
    ver, n_t, n_kv = struct.unpack_from("<IQQ", data, pos)
    pos += 20
    limits.check("tensor count", n_t, limits.max_tensor_count)
    limits.check("metadata entries", n_kv, limits.max_metadata_entries)

    def rstr():
        nonlocal pos
        (n,) = struct.unpack_from("<Q", data, pos)
        limits.check("name length", n, limits.max_name_bytes)
        s = data[pos + 8:pos + 8 + n].decode()
        pos += 8 + n
        return s
    kv = {}
    for _ in range(n_kv):
        k = rstr()
        (typ,) = struct.unpack_from("<I", data, pos)
        pos += 4
        if typ == 10:
            (kv[k],) = struct.unpack_from("<Q", data, pos)
            pos += 8
        elif typ == 8:
            kv[k] = rstr()
        else:
            raise LimitError(f"unsupported GGUF metadata type {typ}")
    tensors = {}
    for _ in range(n_t):
        name = rstr()
        (nd,) = struct.unpack_from("<I", data, pos)
        pos += 4
        limits.check("rank", nd, limits.max_rank)
        dims = struct.unpack_from(f"<{nd}Q", data, pos)
        pos += 8 * nd
        typ, off = struct.unpack_from("<IQ", data, pos)
        pos += 12
        tensors[name] = {"shape": list(reversed(dims)), "type": typ, "offset": off}
    base = pos + ((-pos) % kv.get("general.alignment", _ALIGN))
    return {"version": ver, "metadata": kv, "tensors": tensors, "data_offset": base}


def export_mlx(tensors: dict[str, torch.Tensor], directory, config: dict | None = None) -> None:
    """MLX convention: ``weights.safetensors`` + ``config.json`` in one directory."""
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    save_safetensors({k: v for k, v in tensors.items()}, d / "weights.safetensors", metadata={"format": "mlx"})
    (d / "config.json").write_text(json.dumps(config or {}, indent=1))


@dataclass
class FileReport:
    format: str
    tensors: int
    parameters: int
    bytes: int
    dtypes: dict
    metadata: dict


def inspect_file(path, limits: ResourceLimits = DEFAULT_LIMITS) -> FileReport:
    p = Path(path)
    with open(p, "rb") as f:
        magic = f.read(4)
    if magic == GGUF_MAGIC:
        idx = read_gguf_index(p, limits)
        params = 0
        for t in idx["tensors"].values():
            n = 1
            for d in t["shape"]:
                n *= d
            params += n
        types: dict = {}
        for t in idx["tensors"].values():
            types[str(t["type"])] = types.get(str(t["type"]), 0) + 1
        return FileReport("gguf", len(idx["tensors"]), params, p.stat().st_size, types, idx["metadata"])
    header, _ = read_header(p, limits)
    meta = header.pop("__metadata__", {})
    params, dt = 0, {}
    for m in header.values():
        n = 1
        for d in m["shape"]:
            n *= d
        params += n
        dt[m["dtype"]] = dt.get(m["dtype"], 0) + 1
    return FileReport("safetensors", len(header), params, p.stat().st_size, dt, meta)
