"""Terminal viewer for a run's JSONL (the role of incin-viz: loss / scalar / grad-norm / memory panels).
Plain text, no curses: ``python -m incin_b200 watch <run.jsonl>`` re-renders on an interval."""
from __future__ import annotations

import time

from . import read_run

_BARS = " ▁▂▃▄▅▆▇█"


def sparkline(values, width: int = 60) -> str:
    if not values:
        return ""
    if len(values) > width:
        step = len(values) / width
        values = [values[int(i * step)] for i in range(width)]
    lo, hi = min(values), max(values)
    span = (hi - lo) or 1.0
    return "".join(_BARS[int((v - lo) / span * (len(_BARS) - 1))] for v in values)


def render(path, width: int = 60) -> str:
    events = read_run(path)
    series: dict[str, list[float]] = {}
    mem, hyper, epochs = None, {}, 0
    for e in events:
        if e.kind in ("scalar", "gradient_norm", "weight_norm", "device_time") and e.value is not None:
            series.setdefault(f"{e.kind}/{e.name}" if e.kind != "scalar" else e.name, []).append(e.value)
        elif e.kind == "memory":
            mem = e.payload
        elif e.kind == "hyperparam":
            hyper[e.name] = e.payload.get("value")
        elif e.kind == "epoch":
            epochs = max(epochs, int(e.value or 0))
    lines = [f"run {path}  events={len(events)}  epochs={epochs}"]
    for name, vals in sorted(series.items()):
        lines.append(f"{name:24s} {sparkline(vals, width)}  last={vals[-1]:.5g} min={min(vals):.5g} n={len(vals)}")
    if mem:
        lines.append("memory  " + "  ".join(f"{k}={v / 2**20:.1f}MiB" for k, v in mem.items()))
    if hyper:
        lines.append("hyper   " + "  ".join(f"{k}={v}" for k, v in hyper.items()))
    return "\n".join(lines)


def watch(path, interval: float = 1.0, iterations: int | None = None) -> None:
    i = 0
    while iterations is None or i < iterations:
        print("\033[2J\033[H" + render(path), flush=True)
        time.sleep(interval)
        i += 1
