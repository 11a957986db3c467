"""Telemetry: schema-versioned events, a non-blocking emitter thread, JSONL file / local-socket transports,
per-run files under the XDG data directory, and a terminal viewer.

Counterpart of crates/incin-telemetry (events.rs:11-136; emitter.rs:40-140 — priority queue capped at 64,
bulk queue capped at 4096 with drop-oldest, one writer thread; transport/file.rs, transport/socket.rs;
run_dir.rs:18-69 with UUIDv7 run ids) and the hook in crates/incin-backends/src/telemetry.rs:25-71
(process-wide emitter; ``emit_scalar`` / ``emit_memory`` / ``emit_graph_snapshot``).
"""
from __future__ import annotations

import collections
import json
import os
import socket
import threading
import time
import uuid
from dataclasses import asdict, dataclass, field
from pathlib import Path

SCHEMA_VERSION = 1
PRIORITY_CAP = 64
BULK_CAP = 4096


@dataclass
class Event:
    kind: str                 # scalar | gradient_norm | weight_norm | memory | epoch | hyperparam | graph_snapshot | device_time
    name: str = ""
    value: float | None = None
    step: int | None = None
    payload: dict = field(default_factory=dict)
    ts: float = field(default_factory=time.time)
    v: int = SCHEMA_VERSION

    def to_json(self) -> str:
        d = {k: v for k, v in asdict(self).items() if v not in (None, {}, "")}
        return json.dumps(d, separators=(",", ":"))

    @staticmethod
    def from_json(line: str) -> "Event":
        d = json.loads(line)
        known = {"kind", "name", "value", "step", "payload", "ts", "v"}
        extra = {k: d[k] for k in d if k not in known}
        ev = Event(d.get("kind", "unknown"), d.get("name", ""), d.get("value"), d.get("step"), d.get("payload", {}),
                   d.get("ts", 0.0), d.get("v", SCHEMA_VERSION))
        if extra:                      # unknown fields of a newer schema are kept, not rejected
            ev.payload = dict(ev.payload, **extra)
        return ev


def uuid7() -> str:
    """Time-ordered UUID (version 7): 48-bit unix milliseconds, then random bits."""
    ms = int(time.time() * 1000)
    rnd = int.from_bytes(os.urandom(10), "big")
    v = (ms << 80) | (0x7 << 76) | ((rnd >> 68 & 0xFFF) << 64) | (0b10 << 62) | (rnd & ((1 << 62) - 1))
    return str(uuid.UUID(int=v & ((1 << 128) - 1)))


def run_dir() -> Path:
    base = os.environ.get("INCIN_RUN_DIR") or os.path.join(os.environ.get("XDG_DATA_HOME",
                                                           os.path.expanduser("~/.local/share")), "incin", "runs")
    p = Path(base)
    p.mkdir(parents=True, exist_ok=True)
    return p


class FileTransport:
    def __init__(self, path=None):
        self.path = Path(path) if path else run_dir() / f"{uuid7()}.jsonl"
        self._f = open(self.path, "a", buffering=1)

    def send(self, line: str) -> None:
        self._f.write(line + "\n")

    def close(self) -> None:
        self._f.close()


def native_transport(path=None, capacity: int = BULK_CAP):
    """A transport backed by the native sink (csrc/runtime/telemetry.cpp): ``send`` only queues the line, a C++ thread
    appends it to the file, and a full queue drops (and counts) instead of blocking the training loop."""
    from ..runtime import NativeTelemetrySink
    return NativeTelemetrySink(Path(path) if path else run_dir() / f"{uuid7()}.jsonl", capacity)


class SocketTransport:
    """Local IPC: a unix datagram-free stream socket a viewer listens on."""

    def __init__(self, path: str):
        self._s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        self._s.connect(path)

    def send(self, line: str) -> None:
        self._s.sendall(line.encode() + b"\n")

    def close(self) -> None:
        self._s.close()


class Emitter:
    """``emit`` never blocks the training loop: events go to bounded queues drained by one writer thread.
    Priority events (epoch, hyperparam) are never dropped in favour of bulk ones; when the bulk queue is full
    the OLDEST bulk event is dropped and counted."""

    def __init__(self, transport):
        self.transport = transport
        self._prio: collections.deque = collections.deque()
        self._bulk: collections.deque = collections.deque()
        self._cv = threading.Condition()
        self._stop = False
        self.dropped = 0
        self._t = threading.Thread(target=self._run, name="incin-telemetry", daemon=True)
        self._t.start()

    def emit(self, ev: Event, priority: bool = False) -> None:
        with self._cv:
            if priority:
                if len(self._prio) >= PRIORITY_CAP:
                    self._prio.popleft()
                    self.dropped += 1
                self._prio.append(ev)
            else:
                if len(self._bulk) >= BULK_CAP:
                    self._bulk.popleft()
                    self.dropped += 1
                self._bulk.append(ev)
            self._cv.notify()

    def _run(self) -> None:
        while True:
            with self._cv:
                while not self._prio and not self._bulk and not self._stop:
                    self._cv.wait(0.2)
                if self._stop and not self._prio and not self._bulk:
                    return
                ev = self._prio.popleft() if self._prio else self._bulk.popleft()
            try:
                self.transport.send(ev.to_json())
            except Exception:
                self.dropped += 1

    def close(self) -> None:
        with self._cv:
            self._stop = True
            self._cv.notify()
        self._t.join(timeout=5)
        self.transport.close()


_emitter: Emitter | None = None


def set_emitter(e: Emitter | None) -> None:
    global _emitter
    _emitter = e


def emitter() -> Emitter | None:
    return _emitter


def emit_scalar(name: str, value: float, step: int | None = None) -> None:
    if _emitter:
        _emitter.emit(Event("scalar", name, float(value), step))


def emit_memory(step: int | None = None) -> None:
    if not _emitter:
        return
    payload = {}
    try:
        import resource
        payload["rss_bytes"] = resource.getrusage(resource.RUSAGE_SELF).ru_maxrss * 1024
    except Exception:
        pass
    try:
        import torch
        if torch.cuda.is_available():
            payload["cuda_allocated"] = torch.cuda.memory_allocated()
            payload["cuda_reserved"] = torch.cuda.memory_reserved()
    except Exception:
        pass
    _emitter.emit(Event("memory", "memory", None, step, payload))


def emit_graph_snapshot(graph, step: int | None = None) -> None:
    if _emitter:
        _emitter.emit(Event("graph_snapshot", "graph", None, step, {"nodes": graph.to_list()}))


def emit_epoch(epoch: int, **payload) -> None:
    if _emitter:
        _emitter.emit(Event("epoch", "epoch", float(epoch), None, payload), priority=True)


def emit_hyperparam(name: str, value) -> None:
    if _emitter:
        _emitter.emit(Event("hyperparam", name, None, None, {"value": value}), priority=True)


def read_run(path) -> list[Event]:
    out = []
    for line in Path(path).read_text().splitlines():
        if line.strip():
            try:
                out.append(Event.from_json(line))
            except json.JSONDecodeError:
                continue   # a torn last line of a live run
    return out
