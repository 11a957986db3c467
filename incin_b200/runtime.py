"""Python face of the native host runtime in ``csrc/runtime`` (part of ``libincin_host.so``).

* :func:`fnv1a64` / :class:`NativeDigest` — the streaming FNV-1a 64 digest behind plan hashes (``digest.cpp``);
  byte-for-byte the encoding of :class:`incin_b200.parallel.mesh.Digest`.
* :class:`NativeBatchLoader` — worker threads gather rows of in-memory tensors into batches, delivered in order through
  a bounded ring (``loader.cpp``); the batch sequence depends only on (seed, epoch, batch size), not on the number of
  workers.
* :func:`first_fit_arena` — arena planning by liveness (``memplan.cpp``), the planner of compiled plans.
* :func:`read_ranges` — parallel positional reads of byte ranges into host tensors (``fileio.cpp``), behind the
  threaded safetensors loader.
* :class:`NativeTelemetrySink` — JSON-lines events through a bounded queue and a background writer thread
  (``telemetry.cpp``), in the schema of :mod:`incin_b200.telemetry`.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _native as nat

_ready = False


def _lib():
    global _ready
    h = nat.host()
    if not _ready:
        u64, i64, vp, cp = C.c_uint64, C.c_int64, C.c_void_p, C.c_char_p
        h.incin_digest_init.restype = u64
        h.incin_digest_bytes.restype = u64
        h.incin_digest_bytes.argtypes = [u64, vp, i64]
        h.incin_digest_number.restype = u64
        h.incin_digest_number.argtypes = [u64, u64]
        h.incin_digest_field.restype = u64
        h.incin_digest_field.argtypes = [u64, vp, i64]
        h.incin_fnv1a64.restype = u64
        h.incin_fnv1a64.argtypes = [vp, i64]
        h.incin_loader_create.restype = i64
        h.incin_loader_create.argtypes = [vp, i64, vp, i64, i64, i64, C.c_int, C.c_int, u64, C.c_int, C.c_int]
        h.incin_loader_start.restype = i64
        h.incin_loader_start.argtypes = [i64, u64]
        h.incin_loader_next.restype = C.c_int
        h.incin_loader_next.argtypes = [i64, vp, vp, C.POINTER(i64)]
        h.incin_loader_order.restype = C.c_int
        h.incin_loader_order.argtypes = [i64, vp]
        h.incin_loader_destroy.restype = None
        h.incin_loader_destroy.argtypes = [i64]
        h.incin_memplan_first_fit.restype = i64
        h.incin_memplan_first_fit.argtypes = [i64, vp, vp, vp, vp, vp]
        h.incin_file_read_ranges.restype = C.c_int
        h.incin_file_read_ranges.argtypes = [cp, i64, vp, vp, vp, C.c_int]
        h.incin_telemetry_open.restype = i64
        h.incin_telemetry_open.argtypes = [cp, i64]
        h.incin_telemetry_scalar.restype = C.c_int
        h.incin_telemetry_scalar.argtypes = [i64, cp, C.c_double, i64]
        h.incin_telemetry_memory.restype = C.c_int
        h.incin_telemetry_memory.argtypes = [i64, C.c_int, i64, i64, i64]
        h.incin_telemetry_raw.restype = C.c_int
        h.incin_telemetry_raw.argtypes = [i64, cp]
        h.incin_telemetry_flush.restype = i64
        h.incin_telemetry_flush.argtypes = [i64]
        h.incin_telemetry_close.restype = i64
        h.incin_telemetry_close.argtypes = [i64]
        _ready = True
    return h


# ------------------------------------------------------------------------------------------------------ digest
def fnv1a64(data: bytes) -> int:
    return int(_lib().incin_fnv1a64(data, len(data)))


class NativeDigest:
    """Same interface and same results as :class:`incin_b200.parallel.mesh.Digest`, computed in native code."""

    def __init__(self, state: int | None = None):
        self.state = int(_lib().incin_digest_init()) if state is None else state

    def bytes(self, b: bytes) -> "NativeDigest":
        self.state = int(_lib().incin_digest_bytes(self.state, b, len(b)))
        return self

    def number(self, v: int) -> "NativeDigest":
        self.state = int(_lib().incin_digest_number(self.state, v & ((1 << 64) - 1)))
        return self

    def field(self, b: bytes) -> "NativeDigest":
        self.state = int(_lib().incin_digest_field(self.state, b, len(b)))
        return self

    def text(self, t: str) -> "NativeDigest":
        return self.field(t.encode())

    def finish(self) -> int:
        return self.state


# ------------------------------------------------------------------------------------------------------ loader
class NativeBatchLoader:
    """Batches of one or two CPU tensors (``inputs[N, ...]`` and optionally ``targets[N, ...]``) assembled by native
    worker threads.  Iterating runs one epoch; consecutive epochs use ``seed + epoch`` for the permutation.

    With ``pin=True`` the batches are written into a small ring of pinned tensors (``prefetch + 2`` of them) that is
    reused: a yielded batch stays valid until ``prefetch + 1`` further batches have been drawn, which is what a
    training loop that copies each batch to the device needs.  Without it every batch is a fresh tensor.
    """

    def __init__(self, inputs: torch.Tensor, targets: torch.Tensor | None = None, *, batch_size: int = 1,
                 shuffle: bool = False, drop_last: bool = False, seed: int = 0, workers: int = 2, prefetch: int = 4,
                 pin: bool = False):
        if inputs.device.type != "cpu" or (targets is not None and targets.device.type != "cpu"):
            raise ValueError("NativeBatchLoader gathers host tensors")
        if targets is not None and targets.shape[0] != inputs.shape[0]:
            raise ValueError("inputs and targets must have the same number of rows")
        if batch_size < 1:
            raise ValueError("batch_size must be >= 1")
        self.inputs = inputs.contiguous()
        self.targets = targets.contiguous() if targets is not None else None
        self.batch_size, self.shuffle, self.drop_last, self.seed = batch_size, shuffle, drop_last, seed
        self.workers, self.prefetch, self.pin = workers, prefetch, pin
        self.epoch = 0
        n = self.inputs.shape[0]
        row_a = self.inputs[0].numel() * self.inputs.element_size() if n else self.inputs.element_size()
        row_b = (self.targets[0].numel() * self.targets.element_size() if n else 1) if self.targets is not None else 0
        self._h = _lib().incin_loader_create(self.inputs.data_ptr(), max(row_a, 1),
                                             self.targets.data_ptr() if self.targets is not None else None, row_b, n,
                                             batch_size, int(shuffle), int(drop_last), seed, workers, prefetch + 1)
        if not self._h:
            raise ValueError("the native loader rejected its arguments")
        self._ring: list[tuple[torch.Tensor, torch.Tensor | None]] = []

    def __len__(self) -> int:
        n = self.inputs.shape[0]
        return n // self.batch_size if self.drop_last else (n + self.batch_size - 1) // self.batch_size

    def order(self) -> list[int]:
        """Row order of the epoch in progress (after iteration has started)."""
        out = torch.empty(self.inputs.shape[0], dtype=torch.int64)
        if _lib().incin_loader_order(self._h, out.data_ptr()) != 0:
            return []
        return out.tolist()

    def _buffers(self, k: int):
        shape_a = (self.batch_size, *self.inputs.shape[1:])
        shape_b = (self.batch_size, *self.targets.shape[1:]) if self.targets is not None else None
        if not self.pin:
            return (torch.empty(shape_a, dtype=self.inputs.dtype),
                    torch.empty(shape_b, dtype=self.targets.dtype) if shape_b else None)
        if not self._ring:
            for _ in range(self.prefetch + 2):
                self._ring.append((torch.empty(shape_a, dtype=self.inputs.dtype).pin_memory(),
                                   torch.empty(shape_b, dtype=self.targets.dtype).pin_memory() if shape_b else None))
        return self._ring[k % len(self._ring)]

    def __iter__(self):
        lib = _lib()
        n_batches = lib.incin_loader_start(self._h, self.epoch)
        self.epoch += 1
        rows = C.c_int64(0)
        for k in range(max(n_batches, 0)):
            a, b = self._buffers(k)
            rc = lib.incin_loader_next(self._h, a.data_ptr(), b.data_ptr() if b is not None else None, C.byref(rows))
            if rc != 1:
                raise RuntimeError(f"native loader stopped after {k} of {n_batches} batches (code {rc})")
            r = rows.value
            yield (a[:r], b[:r]) if b is not None else a[:r]

    def close(self) -> None:
        if getattr(self, "_h", 0):
            _lib().incin_loader_destroy(self._h)
            self._h = 0

    def __del__(self):
        try:
            self.close()
        except Exception:   # interpreter shutdown: the library may already be gone
            pass


# ------------------------------------------------------------------------------------------------------ memory plan
def first_fit_arena(sizes: list[int], first: list[int], last: list[int], skip: list[bool] | None = None
                    ) -> tuple[list[int], int]:
    """Offsets (``-1`` for skipped buffers) and arena size of the greedy first-fit plan (``memplan.cpp``)."""
    n = len(sizes)
    if not (len(first) == len(last) == n) or (skip is not None and len(skip) != n):
        raise ValueError("sizes, first, last (and skip) must have the same length")
    a = torch.tensor(sizes, dtype=torch.int64)
    f = torch.tensor(first, dtype=torch.int64)
    la = torch.tensor(last, dtype=torch.int64)
    sk = torch.tensor([1 if s else 0 for s in skip], dtype=torch.uint8) if skip is not None else None
    out = torch.empty(n, dtype=torch.int64)
    peak = _lib().incin_memplan_first_fit(n, a.data_ptr(), f.data_ptr(), la.data_ptr(),
                                          sk.data_ptr() if sk is not None else None, out.data_ptr())
    if peak < 0:
        raise ValueError("the native planner rejected its arguments")
    return out.tolist(), int(peak)


# ------------------------------------------------------------------------------------------------------ file reads
def read_ranges(path, ranges: list[tuple[int, torch.Tensor]], threads: int = 8) -> None:
    """Fill each (contiguous, host) tensor with the bytes of ``path`` starting at its offset, with ``threads`` native
    readers (``fileio.cpp``).  Raises ``OSError`` when the file cannot be opened or ends early."""
    n = len(ranges)
    if n == 0:
        return
    for _, t in ranges:
        if t.device.type != "cpu" or not t.is_contiguous():
            raise ValueError("destinations must be contiguous host tensors")
    offs = torch.tensor([o for o, _ in ranges], dtype=torch.int64)
    sizes = torch.tensor([t.numel() * t.element_size() for _, t in ranges], dtype=torch.int64)
    ptrs = (C.c_void_p * n)(*[t.data_ptr() if t.numel() else None for _, t in ranges])
    rc = _lib().incin_file_read_ranges(str(path).encode(), n, offs.data_ptr(), sizes.data_ptr(), ptrs, threads)
    if rc == 1:
        raise OSError(f"cannot open {path}")
    if rc == 2:
        raise OSError(f"{path}: read error or file shorter than its header says")
    if rc:
        raise ValueError("bad arguments to the native reader")


# ------------------------------------------------------------------------------------------------------ telemetry
class NativeTelemetrySink:
    """JSON-lines sink with a bounded queue and a writer thread.  ``send(line)`` makes it a transport of
    :class:`incin_b200.telemetry.Emitter`; ``scalar`` / ``memory`` format the event in native code."""

    def __init__(self, path, capacity: int = 4096):
        self.path = str(path)
        self._h = _lib().incin_telemetry_open(self.path.encode(), capacity)
        if not self._h:
            raise OSError(f"cannot open {self.path} for appending")

    def scalar(self, name: str, value: float, step: int) -> bool:
        return _lib().incin_telemetry_scalar(self._h, name.encode(), float(value), int(step)) == 1

    def memory(self, device: int, allocated: int, reserved: int, step: int) -> bool:
        return _lib().incin_telemetry_memory(self._h, device, allocated, reserved, step) == 1

    def send(self, line: str) -> None:
        _lib().incin_telemetry_raw(self._h, line.encode())

    def flush(self) -> int:
        """Block until everything queued is on disk; returns how many events were dropped so far."""
        return int(_lib().incin_telemetry_flush(self._h))

    def close(self) -> int:
        if not self._h:
            return 0
        h, self._h = self._h, 0
        return int(_lib().incin_telemetry_close(h))
