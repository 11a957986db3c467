"""Kernel-level tracing: NVTX ranges around the phases and ops of a step, and a per-step device-timed trace.

The reference has no profiler integration (its tracing is the op-graph recorder; timing exists only inside the
autotuner: crates/incin-backends/src/tuning.rs:438-475).  Two switches, both off by default and free when off:

* ``INCIN_NVTX=1`` (or :func:`enable` ``(nvtx=True)``): every native launch call leaves an NVTX mark with its name and
  :func:`op_range` / the training step's phases (zero-grad, forward, backward, optimiser) become NVTX ranges, so a
  timeline tool shows which launches belong to which phase.
* ``INCIN_TRACE=1`` (or ``enable(events=True)``): a CUDA event is recorded behind every native launch call of an eager
  step; :func:`end_step` turns them into ``(name, device milliseconds)`` rows — the time between consecutive events on
  the launching stream, i.e. the device time of that call's kernels when the stream is busy.  ``summary()`` groups
  them by name; ``to_jsonl`` appends one record per step.  (CUDA-graph replays enqueue nothing from Python: trace the
  eager steps, ``TrainStep(use_graph=False)``.)
"""
from __future__ import annotations

import contextlib
import json
import os
import time

_nvtx = os.environ.get("INCIN_NVTX") == "1"
_events = os.environ.get("INCIN_TRACE") == "1"
_rows: list[tuple[str, object]] = []       # (name, cuda event) of the current step
_start = None
_steps: list[list[tuple[str, float]]] = []


def enable(nvtx: bool | None = None, events: bool | None = None) -> None:
    global _nvtx, _events
    if nvtx is not None:
        _nvtx = bool(nvtx)
    if events is not None:
        _events = bool(events)
    _install()


def active() -> bool:
    return _nvtx or _events


def _install() -> None:
    """Point the native loader's launch hook at this module (or remove it when nothing is switched on)."""
    from .. import _native
    _native.LAUNCH_HOOK = on_launch if active() else None


def on_launch(what: str) -> None:
    """Called by the native loader after every launch call while tracing is on."""
    import torch
    if not torch.cuda.is_available():
        return
    if _nvtx:
        torch.cuda.nvtx.mark(what or "native")
    if _events and _start is not None and not torch.cuda.is_current_stream_capturing():
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        _rows.append((what or "native", ev))


@contextlib.contextmanager
def op_range(name: str):
    """NVTX range around a phase or an op (no-op unless NVTX tracing is on)."""
    if _nvtx:
        import torch
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


def begin_step() -> None:
    global _start
    if not _events:
        return
    import torch
    _rows.clear()
    _start = torch.cuda.Event(enable_timing=True)
    _start.record()


def end_step() -> list[tuple[str, float]]:
    """Synchronise and return this step's ``(name, ms)`` rows (empty when event tracing is off)."""
    global _start
    if not _events or _start is None:
        return []
    import torch
    torch.cuda.synchronize()
    out, prev = [], _start
    for name, ev in _rows:
        out.append((name, prev.elapsed_time(ev)))
        prev = ev
    _rows.clear()
    _start = None
    _steps.append(out)
    return out


def summary(rows: list[tuple[str, float]] | None = None) -> list[dict]:
    """Device time by launch name, largest first: ``[{name, calls, ms, share}]``."""
    rows = rows if rows is not None else (_steps[-1] if _steps else [])
    total = sum(ms for _, ms in rows) or 1.0
    agg: dict[str, list[float]] = {}
    for name, ms in rows:
        a = agg.setdefault(name, [0, 0.0])
        a[0] += 1
        a[1] += ms
    return sorted(({"name": n, "calls": int(c), "ms": round(ms, 4), "share": round(ms / total, 4)} for n, (c, ms) in agg.items()),
                  key=lambda r: -r["ms"])


def to_jsonl(path, rows: list[tuple[str, float]] | None = None, step: int | None = None) -> None:
    rows = rows if rows is not None else (_steps[-1] if _steps else [])
    with open(path, "a") as f:
        f.write(json.dumps({"t": time.time(), "step": step, "total_ms": round(sum(ms for _, ms in rows), 4),
                            "launches": len(rows), "by_name": summary(rows)}) + "\n")


if active():       # switched on through the environment
    try:
        _install()
    except Exception:   # the native loader is imported lazily elsewhere; enable() installs the hook then
        pass
