"""Terminal viewer of a run: panels, a plugin interface, a vim-style keymap and a live tail of the run's JSONL.

Counterpart of crates/incin-viz (``App`` with focus / layout / per-panel failure isolation: src/app.rs, src/dispatch.rs;
the tailing reader: src/transport_reader.rs; panels loss / scalar / norms / system / graph: src/panels/*.rs; flags and
keymap file: src/main.rs:53-157) and of crates/incin-viz-plugin-api (``Panel`` and ``Plugin``: src/lib.rs:58-75,
``Action`` and ``KeymapProvider``: src/keymap.rs).

The drawing surface is a character grid (:class:`Canvas`) that the terminal driver paints with ANSI escapes, so every
panel renders the same way into a string in a test, under ``--once`` and on a live terminal.

    python -m incin_b200 watch run.jsonl            live; h/j/k/l or Tab move the focus, t toggles the layout, q quits
    python -m incin_b200 watch run.jsonl --once     one frame on stdout

Plug-ins: ``INCIN_VIZ_PLUGINS=package.module:factory,...`` — each factory returns a :class:`Plugin` whose panels are
added after the built-in ones.  Key bindings: ``incin-viz.toml`` (``[keymap]`` table, ``action = "key"``) in the working
directory or ``--keymap FILE``.
"""
from __future__ import annotations

import enum
import importlib
import json
import os
import time
from dataclasses import dataclass
from pathlib import Path

from . import Event, read_run

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


# ---------------------------------------------------------------------------------------------------------------------
# plug-in interface
# ---------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Area:
    x: int
    y: int
    w: int
    h: int

    def inner(self) -> "Area":
        return Area(self.x + 1, self.y + 1, max(0, self.w - 2), max(0, self.h - 2))


class Canvas:
    """A ``width x height`` grid of characters with a bold mask; text is clipped to the area it is written into."""

    def __init__(self, width: int, height: int):
        self.width, self.height = width, height
        self.rows = [[" "] * width for _ in range(height)]
        self.bold = [[False] * width for _ in range(height)]

    def text(self, area: Area, col: int, row: int, s: str, bold: bool = False) -> None:
        y = area.y + row
        if not (0 <= row < area.h and 0 <= y < self.height):
            return
        for i, ch in enumerate(s):
            x = area.x + col + i
            if col + i >= area.w or x >= self.width:
                break
            if x >= 0 and col + i >= 0:
                self.rows[y][x] = ch
                self.bold[y][x] = bold

    def box(self, area: Area, title: str, focused: bool) -> None:
        if area.w < 2 or area.h < 2:
            return
        h, v = ("━", "┃") if focused else ("─", "│")
        tl, tr, bl, br = ("┏", "┓", "┗", "┛") if focused else ("┌", "┐", "└", "┘")
        self.text(area, 0, 0, tl + h * (area.w - 2) + tr, focused)
        self.text(area, 0, area.h - 1, bl + h * (area.w - 2) + br, focused)
        for r in range(1, area.h - 1):
            self.text(area, 0, r, v, focused)
            self.text(area, area.w - 1, r, v, focused)
        self.text(area, 2, 0, f" {title} "[: max(0, area.w - 4)], focused)

    def to_text(self) -> str:
        return "\n".join("".join(r).rstrip() for r in self.rows)

    def to_ansi(self) -> str:
        out = []
        for chars, bold in zip(self.rows, self.bold):
            line, on = [], False
            for ch, b in zip(chars, bold):
                if b != on:
                    line.append("\033[1m" if b else "\033[22m")
                    on = b
                line.append(ch)
            if on:
                line.append("\033[22m")
            out.append("".join(line))
        return "\r\n".join(out)


class Panel:
    """One tile of the viewer.  ``update`` sees every event of the run in order; ``render`` draws into the inner area
    of the panel's box; ``handle_key`` gets the keys that the keymap resolves to ``Action.PANEL_LOCAL`` while the panel
    has the focus and says whether it used the key."""
    id = "panel"
    title = "panel"

    def update(self, event: Event) -> None:
        raise NotImplementedError

    def render(self, canvas: Canvas, area: Area) -> None:
        raise NotImplementedError

    def handle_key(self, key: str) -> bool:
        return False

    def hover_text(self, col: int, row: int) -> str | None:
        return None

    def reset(self) -> None:
        pass


class Plugin:
    """A bundle of panels contributed by another package."""

    def panels(self) -> list[Panel]:
        return []


class Action(enum.Enum):
    QUIT = "quit"
    FOCUS_NEXT = "focus_next"
    FOCUS_PREV = "focus_prev"
    FOCUS_UP = "focus_up"
    FOCUS_DOWN = "focus_down"
    FOCUS_LEFT = "focus_left"
    FOCUS_RIGHT = "focus_right"
    RETRY_PANEL = "retry_panel"
    TOGGLE_LAYOUT = "toggle_layout"
    PANEL_LOCAL = "panel_local"


class Keymap:
    """Key -> action; unknown keys go to the focused panel.  The defaults are the vim keys plus Tab / Shift-Tab."""
    DEFAULT = {"q": Action.QUIT, "\x03": Action.QUIT, "\t": Action.FOCUS_NEXT, "\x1b[Z": Action.FOCUS_PREV,
               "k": Action.FOCUS_UP, "j": Action.FOCUS_DOWN, "h": Action.FOCUS_LEFT, "l": Action.FOCUS_RIGHT,
               "\x1b[A": Action.FOCUS_UP, "\x1b[B": Action.FOCUS_DOWN, "\x1b[D": Action.FOCUS_LEFT,
               "\x1b[C": Action.FOCUS_RIGHT, "r": Action.RETRY_PANEL, "t": Action.TOGGLE_LAYOUT}
    NAMED = {"tab": "\t", "backtab": "\x1b[Z", "up": "\x1b[A", "down": "\x1b[B", "left": "\x1b[D", "right": "\x1b[C",
             "esc": "\x1b", "enter": "\r", "space": " "}

    def __init__(self, bindings: dict[str, Action] | None = None):
        self.bindings = dict(self.DEFAULT if bindings is None else bindings)

    def resolve(self, key: str) -> Action:
        return self.bindings.get(key, Action.PANEL_LOCAL)

    @classmethod
    def from_toml(cls, path) -> "Keymap":
        """``[keymap]`` with ``action = "key"`` or ``action = ["key", ...]``; a rebound action loses its default keys.
        An unknown action name is an error: a typo must not silently leave the default in place."""
        import tomllib
        table = tomllib.loads(Path(path).read_text()).get("keymap", {})
        km = cls()
        for name, keys in table.items():
            try:
                action = Action(name)
            except ValueError:
                raise ValueError(f"{path}: unknown action '{name}' (known: {', '.join(a.value for a in Action)})") from None
            km.bindings = {k: a for k, a in km.bindings.items() if a is not action}
            for k in ([keys] if isinstance(keys, str) else keys):
                km.bindings[cls.NAMED.get(k.lower(), k)] = action
        return km


# ---------------------------------------------------------------------------------------------------------------------
# built-in panels
# ---------------------------------------------------------------------------------------------------------------------
def _chart(canvas: Canvas, area: Area, values: list[float], top: int = 0, height: int | None = None) -> None:
    """Column chart of ``values`` resampled to the area's width, eighth-block resolution."""
    height = area.h - top if height is None else height
    if height <= 0 or area.w <= 0 or not values:
        return
    w = area.w
    if len(values) != w and len(values) > 1:      # stretch or shrink to the tile's width
        step = len(values) / w
        values = [values[int(i * step)] for i in range(w)]
    lo, hi = min(values), max(values)
    span = (hi - lo) or 1.0
    for i, v in enumerate(values):
        level = (v - lo) / span * height * 8
        for r in range(height):
            fill = min(8, max(0, int(level - r * 8 + 0.5)))
            if r == 0:
                fill = max(fill, 1)
            if fill:
                canvas.text(area, i, top + height - 1 - r, _BARS[fill])


class LossPanel(Panel):
    """The ``loss`` scalar: chart, last / best value and a smoothed trend (exponential average, factor 0.9)."""
    id, title = "loss", "loss"

    def __init__(self):
        self.reset()

    def reset(self):
        self.values: list[float] = []
        self.steps: list[int] = []
        self.ema = None
        self.log = False

    def update(self, e):
        if e.kind == "scalar" and e.name == "loss" and e.value is not None:
            self.values.append(e.value)
            self.steps.append(e.step if e.step is not None else len(self.values))
            self.ema = e.value if self.ema is None else 0.9 * self.ema + 0.1 * e.value

    def handle_key(self, key):
        if key == "g":      # toggle a log scale
            self.log = not self.log
            return True
        return False

    def render(self, canvas, area):
        if not self.values:
            canvas.text(area, 0, 0, "waiting for a 'loss' scalar ...")
            return
        import math
        v = self.values
        canvas.text(area, 0, 0, f"step {self.steps[-1]}  last {v[-1]:.5g}  best {min(v):.5g}  ema {self.ema:.5g}"
                                f"{'  [log]' if self.log else ''}", bold=True)
        shown = [math.log10(max(x, 1e-12)) for x in v] if self.log else v
        _chart(canvas, area, shown, top=1)


class ScalarPanel(Panel):
    """Every other scalar and every device-time series: one sparkline row each; ``J`` / ``K`` scroll the list."""
    id, title = "scalars", "scalars"

    def __init__(self):
        self.reset()

    def reset(self):
        self.series: dict[str, list[float]] = {}
        self.scroll = 0

    def update(self, e):
        if e.value is None:
            return
        if e.kind == "scalar" and e.name != "loss":
            self.series.setdefault(e.name, []).append(e.value)
        elif e.kind == "device_time":
            self.series.setdefault("device_time/" + e.name, []).append(e.value)

    def handle_key(self, key):
        if key in ("J", "K"):
            self.scroll = max(0, min(max(0, len(self.series) - 1), self.scroll + (1 if key == "J" else -1)))
            return True
        return False

    def render(self, canvas, area):
        names = sorted(self.series)[self.scroll:]
        if not names:
            canvas.text(area, 0, 0, "no scalars yet")
        for r, name in enumerate(names[: area.h]):
            vals = self.series[name]
            label = f"{name[:22]:22s} {vals[-1]:>10.4g} "
            canvas.text(area, 0, r, label + sparkline(vals, max(4, area.w - len(label))))


class NormsPanel(Panel):
    """Gradient and weight norms by parameter (or ``global``): last value, ratio to the first, trend; the largest
    gradient norm on top.  A non-finite norm is flagged."""
    id, title = "norms", "grad / weight norms"

    def __init__(self):
        self.reset()

    def reset(self):
        self.grad: dict[str, list[float]] = {}
        self.weight: dict[str, list[float]] = {}

    def update(self, e):
        if e.value is None:
            return
        if e.kind == "gradient_norm":
            self.grad.setdefault(e.name or "global", []).append(e.value)
        elif e.kind == "weight_norm":
            self.weight.setdefault(e.name or "global", []).append(e.value)

    def render(self, canvas, area):
        names = sorted(set(self.grad) | set(self.weight), key=lambda n: -(self.grad.get(n) or [0.0])[-1])
        if not names:
            canvas.text(area, 0, 0, "no norms yet")
            return
        canvas.text(area, 0, 0, f"{'parameter':24s} {'|grad|':>10s} {'x first':>8s} {'|weight|':>10s}  trend", bold=True)
        for r, n in enumerate(names[: max(0, area.h - 1)]):
            g, w = self.grad.get(n, []), self.weight.get(n, [])
            gl = g[-1] if g else float("nan")
            bad = g and not (gl == gl and abs(gl) != float("inf"))
            ratio = (gl / g[0]) if g and g[0] else float("nan")
            row = f"{n[:24]:24s} {gl:>10.4g} {ratio:>8.3g} {(w[-1] if w else float('nan')):>10.4g}  "
            row += "NON-FINITE" if bad else sparkline([x for x in g if x == x], max(4, area.w - len(row)))
            canvas.text(area, 0, r + 1, row, bold=bool(bad))


class SystemPanel(Panel):
    """Memory (host and device), epochs, event rate and the run's hyper-parameters."""
    id, title = "system", "system"

    def __init__(self):
        self.reset()

    def reset(self):
        self.mem: dict[str, list[float]] = {}
        self.hyper: dict[str, object] = {}
        self.epochs, self.events = 0, 0
        self.first_ts = self.last_ts = None

    def update(self, e):
        self.events += 1
        if e.ts:
            self.first_ts = e.ts if self.first_ts is None else self.first_ts
            self.last_ts = e.ts
        if e.kind == "memory":
            for k, v in e.payload.items():
                if isinstance(v, (int, float)):
                    self.mem.setdefault(k, []).append(float(v))
        elif e.kind == "hyperparam":
            self.hyper[e.name] = e.payload.get("value")
        elif e.kind == "epoch":
            self.epochs = max(self.epochs, int(e.value or 0))

    def render(self, canvas, area):
        span = (self.last_ts - self.first_ts) if self.first_ts is not None else 0.0
        rate = f"{self.events / span:.1f}/s" if span > 0 else "-"
        canvas.text(area, 0, 0, f"events {self.events} ({rate})  epochs {self.epochs}  wall {span:.1f}s", bold=True)
        r = 1
        for k in sorted(self.mem):
            vals = self.mem[k]
            label = f"{k[:18]:18s} {vals[-1] / 2**20:>10.1f} MiB  peak {max(vals) / 2**20:>10.1f}  "
            canvas.text(area, 0, r, label + sparkline(vals, max(4, area.w - len(label))))
            r += 1
        for k in sorted(self.hyper):
            canvas.text(area, 0, r, f"{k[:18]:18s} {self.hyper[k]}")
            r += 1


class GraphPanel(Panel):
    """The last recorded op graph: op histogram and the node list in topological order with the inputs of each node;
    ``J`` / ``K`` scroll, ``G`` jumps to the end, ``0`` to the start."""
    id, title = "graph", "op graph"

    def __init__(self):
        self.reset()

    def reset(self):
        self.nodes: list[dict] = []
        self.step = None
        self.scroll = 0

    def update(self, e):
        if e.kind == "graph_snapshot":
            self.nodes = list(e.payload.get("nodes", []))
            self.step = e.step
            self.scroll = min(self.scroll, max(0, len(self.nodes) - 1))

    def handle_key(self, key):
        last = max(0, len(self.nodes) - 1)
        move = {"J": 1, "K": -1, "\x04": 10, "\x15": -10}.get(key)
        if move is not None:
            self.scroll = max(0, min(last, self.scroll + move))
        elif key == "G":
            self.scroll = last
        elif key == "0":
            self.scroll = 0
        else:
            return False
        return True

    def hover_text(self, col, row):
        i = self.scroll + row - 2
        return json.dumps(self.nodes[i], default=str) if row >= 2 and 0 <= i < len(self.nodes) else None

    def render(self, canvas, area):
        if not self.nodes:
            canvas.text(area, 0, 0, "no graph snapshot yet")
            return
        hist: dict[str, int] = {}
        for n in self.nodes:
            hist[n.get("op", "?")] = hist.get(n.get("op", "?"), 0) + 1
        top = sorted(hist.items(), key=lambda kv: -kv[1])[:6]
        canvas.text(area, 0, 0, f"{len(self.nodes)} nodes" + (f" @ step {self.step}" if self.step is not None else "")
                    + "  " + "  ".join(f"{k}x{v}" for k, v in top), bold=True)
        canvas.text(area, 0, 1, f"{'id':>5s}  {'op':18s} {'shape':22s} {'dtype':8s} inputs", bold=True)
        for r, n in enumerate(self.nodes[self.scroll: self.scroll + max(0, area.h - 2)]):
            shape = "x".join(map(str, n.get("shape", []))) or "scalar"
            ins = ",".join(f"%{i}" for i in n.get("inputs", []))
            canvas.text(area, 0, r + 2, f"{n.get('id', '?'):>5}  {str(n.get('op', '?'))[:18]:18s} {shape[:22]:22s} "
                                        f"{str(n.get('dtype', ''))[:8]:8s} {ins}")


def builtin_panels() -> list[Panel]:
    return [LossPanel(), ScalarPanel(), NormsPanel(), SystemPanel(), GraphPanel()]


def load_plugins(spec: str | None = None) -> list[Plugin]:
    """``module:factory`` entries, comma separated (default: ``INCIN_VIZ_PLUGINS``)."""
    spec = os.environ.get("INCIN_VIZ_PLUGINS", "") if spec is None else spec
    out = []
    for item in filter(None, (s.strip() for s in spec.split(","))):
        mod, _, attr = item.partition(":")
        obj = getattr(importlib.import_module(mod), attr or "plugin")
        plugin = obj() if callable(obj) and not isinstance(obj, Plugin) else obj
        if not hasattr(plugin, "panels"):
            raise TypeError(f"{item} is not a viz plug-in (no panels())")
        out.append(plugin)
    return out


# ---------------------------------------------------------------------------------------------------------------------
# application
# ---------------------------------------------------------------------------------------------------------------------
class RunTail:
    """Incremental reader of a growing JSONL file: remembers the byte offset, keeps a torn last line for the next
    poll and starts over when the file shrank (a new run under the same name)."""

    def __init__(self, path):
        self.path, self.offset, self._partial = Path(path), 0, b""
        self.restarted = False

    def poll(self) -> list[Event]:
        try:
            size = self.path.stat().st_size
        except FileNotFoundError:
            return []
        self.restarted = size < self.offset
        if self.restarted:
            self.offset, self._partial = 0, b""
        if size == self.offset:
            return []
        with open(self.path, "rb") as f:
            f.seek(self.offset)
            data = self._partial + f.read()
            self.offset = f.tell()
        lines = data.split(b"\n")
        self._partial = lines.pop()
        out = []
        for ln in lines:
            if ln.strip():
                try:
                    out.append(Event.from_json(ln.decode("utf-8", "replace")))
                except (json.JSONDecodeError, AttributeError):
                    continue
        return out


class App:
    """Owns the panels, the focus and the layout.  A panel whose ``update`` or ``render`` raises is fenced off: its tile
    shows the error, the other panels keep running, and ``retry_panel`` resets it and lets it back in."""

    def __init__(self, panels: list[Panel] | None = None, plugins: list[Plugin] | None = None, keymap: Keymap | None = None):
        self.panels = list(builtin_panels() if panels is None else panels)
        for pl in plugins or []:
            self.panels.extend(pl.panels())
        ids = [p.id for p in self.panels]
        if len(set(ids)) != len(ids):
            raise ValueError(f"duplicate panel id in {ids}")
        self.keymap = keymap or Keymap()
        self.focus, self.grid, self.running = 0, True, True
        self.failed: dict[str, str] = {}
        self.history: list[Event] = []
        self.status = ""

    # events
    def feed(self, events) -> None:
        for e in events:
            self.history.append(e)
            for p in self.panels:
                if p.id in self.failed:
                    continue
                try:
                    p.update(e)
                except Exception as ex:      # noqa: BLE001 — a panel's failure must not take the viewer down
                    self.failed[p.id] = f"update: {type(ex).__name__}: {ex}"

    def restart(self) -> None:
        self.history.clear()
        self.failed.clear()
        for p in self.panels:
            p.reset()

    # layout
    def columns(self) -> int:
        return 2 if self.grid and len(self.panels) > 1 else 1

    def areas(self, width: int, height: int) -> list[Area]:
        """Grid: two columns, rows of equal height, a lone last panel spans the row.  Stack: the focused panel gets
        the screen but for one title row per other panel."""
        n, body = len(self.panels), max(0, height - 1)
        if self.grid:
            cols = self.columns()
            rows = (n + cols - 1) // cols
            out = []
            for i in range(n):
                r, c = divmod(i, cols)
                y0, y1 = body * r // rows, body * (r + 1) // rows
                lone = i == n - 1 and c == 0 and cols == 2
                x0, x1 = (0, width) if lone else (width * c // cols, width * (c + 1) // cols)
                out.append(Area(x0, y0, x1 - x0, y1 - y0))
            return out
        out, y = [], 0
        big = max(2, body - 2 * (n - 1))
        for i in range(n):
            h = big if i == self.focus else 2
            out.append(Area(0, y, width, max(0, min(h, body - y))))
            y += h
        return out

    def render(self, width: int = 120, height: int = 40) -> Canvas:
        canvas = Canvas(width, height)
        for i, (p, a) in enumerate(zip(self.panels, self.areas(width, height))):
            if a.w < 4 or a.h < 2:
                continue
            err = self.failed.get(p.id)
            canvas.box(a, f"{p.title}{' [failed]' if err else ''}", i == self.focus)
            inner = a.inner()
            if err is None and inner.h > 0:
                scratch = Canvas(width, height)     # a panel that raises half-way leaves no partial drawing behind
                try:
                    p.render(scratch, inner)
                    for y in range(inner.y, min(height, inner.y + inner.h)):
                        canvas.rows[y][inner.x: inner.x + inner.w] = scratch.rows[y][inner.x: inner.x + inner.w]
                        canvas.bold[y][inner.x: inner.x + inner.w] = scratch.bold[y][inner.x: inner.x + inner.w]
                except Exception as ex:      # noqa: BLE001
                    err = self.failed[p.id] = f"render: {type(ex).__name__}: {ex}"
                    canvas.box(a, f"{p.title} [failed]", i == self.focus)
            if err is not None:
                canvas.text(inner, 0, 0, err)
                canvas.text(inner, 0, 1, "press r (retry_panel) with this panel focused to reset it")
        foot = Area(0, height - 1, width, 1)
        canvas.text(foot, 0, 0, (self.status or f"{len(self.history)} events  focus: {self.panels[self.focus].id}  "
                                 "h/j/k/l Tab move  t layout  r retry  q quit")[:width])
        return canvas

    # keys
    def _move(self, dx: int, dy: int) -> None:
        n, cols = len(self.panels), self.columns()
        r, c = divmod(self.focus, cols)
        r, c = r + dy, c + dx
        rows = (n + cols - 1) // cols
        if not (0 <= r < rows and 0 <= c < cols):
            return
        self.focus = min(n - 1, r * cols + c)

    def on_key(self, key: str) -> Action:
        action = self.keymap.resolve(key)
        n = len(self.panels)
        if action is Action.QUIT:
            self.running = False
        elif action is Action.FOCUS_NEXT:
            self.focus = (self.focus + 1) % n
        elif action is Action.FOCUS_PREV:
            self.focus = (self.focus - 1) % n
        elif action is Action.FOCUS_UP:
            self._move(0, -1)
        elif action is Action.FOCUS_DOWN:
            self._move(0, 1)
        elif action is Action.FOCUS_LEFT:
            self._move(-1, 0)
        elif action is Action.FOCUS_RIGHT:
            self._move(1, 0)
        elif action is Action.TOGGLE_LAYOUT:
            self.grid = not self.grid
        elif action is Action.RETRY_PANEL:
            p = self.panels[self.focus]
            if p.id in self.failed:      # reset, then replay the run so far into it
                del self.failed[p.id]
                try:
                    p.reset()
                    for e in self.history:
                        p.update(e)
                except Exception as ex:  # noqa: BLE001
                    self.failed[p.id] = f"update: {type(ex).__name__}: {ex}"
        else:
            p = self.panels[self.focus]
            if p.id not in self.failed:
                try:
                    p.handle_key(key)
                except Exception as ex:  # noqa: BLE001
                    self.failed[p.id] = f"key: {type(ex).__name__}: {ex}"
        return action


def default_keymap(path=None) -> Keymap:
    path = path or ("incin-viz.toml" if os.path.exists("incin-viz.toml") else None)
    return Keymap.from_toml(path) if path else Keymap()


def render(path, width: int = 120, height: int = 40) -> str:
    """One frame of the run as plain text (what ``watch --once`` prints)."""
    app = App(plugins=load_plugins())
    app.feed(read_run(path))
    app.status = f"run {path}  events={len(app.history)}"
    return app.render(width, height).to_text()


def _read_key(fd: int, timeout: float) -> str | None:
    """One key (escape sequences kept together) from a raw terminal, or None after ``timeout`` seconds."""
    import select
    if not select.select([fd], [], [], timeout)[0]:
        return None
    data = os.read(fd, 1)
    if data == b"\x1b":      # an escape sequence arrives in one burst; a lone Esc does not
        while select.select([fd], [], [], 0.01)[0] and len(data) < 8:
            data += os.read(fd, 1)
            if data[-1:].isalpha() or data[-1:] == b"~":
                break
    return data.decode("utf-8", "replace")


def watch(path, interval: float = 0.5, iterations: int | None = None, keymap: Keymap | None = None) -> None:
    """Live viewer.  On a terminal: raw mode, alternate screen, keys; otherwise (a pipe) frames are printed one after
    the other.  ``iterations`` bounds the number of frames."""
    import shutil
    import sys
    app = App(plugins=load_plugins(), keymap=keymap or default_keymap())
    tail = RunTail(path)
    tty = sys.stdin.isatty() and sys.stdout.isatty()
    restore = None
    if tty:
        import termios
        import tty as ttymod
        fd = sys.stdin.fileno()
        restore = termios.tcgetattr(fd)
        ttymod.setraw(fd)
        sys.stdout.write("\033[?1049h\033[?25l")
    try:
        i = 0
        while app.running and (iterations is None or i < iterations):
            events = tail.poll()
            if tail.restarted:
                app.restart()
            app.feed(events)
            size = shutil.get_terminal_size((120, 40))
            frame = app.render(size.columns, size.lines)
            if tty:
                sys.stdout.write("\033[H" + frame.to_ansi())
                sys.stdout.flush()
                deadline = time.monotonic() + interval
                while app.running and (left := deadline - time.monotonic()) > 0:
                    key = _read_key(sys.stdin.fileno(), left)
                    if key is None:
                        break
                    app.on_key(key)
                    sys.stdout.write("\033[H" + app.render(size.columns, size.lines).to_ansi())
                    sys.stdout.flush()
            else:
                print(frame.to_text(), flush=True)
                time.sleep(interval)
            i += 1
    finally:
        if restore is not None:
            import termios
            termios.tcsetattr(sys.stdin.fileno(), termios.TCSADRAIN, restore)
            sys.stdout.write("\033[?25h\033[?1049l")
            sys.stdout.flush()
