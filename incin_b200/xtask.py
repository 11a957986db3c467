"""Repository maintenance tasks: ledger, budgets, generated documents.

Counterpart of the reference's ``xtask`` crate (xtask/src/main.rs:15-30: ``ledger`` — the human-readable ledger table
and its machine-readable mirror must agree, dependencies exist and are acyclic, no task depends on a less mature tier,
complete tasks record evidence: xtask/src/ledger.rs:1-16; ``budgets`` — regression budgets; ``docs [--check]`` —
regenerate the generated tables or fail when they drifted).

    python -m incin_b200 xtask ledger [--write]     docs/plan/ledger.toml  <->  docs/components.md
    python -m incin_b200 xtask docs [--check]       capability matrix, Rust bindings, component table
    python -m incin_b200 xtask budgets BENCH.json   same as ``check``

The ledger's source of truth is the TOML file; the markdown table is its rendering, and a difference between the two
is an error rather than something a reader finds months later.
"""
from __future__ import annotations

import tomllib
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
LEDGER = "docs/plan/ledger.toml"
TABLE = "docs/components.md"
MATURITY = {"core": 0, "preview": 1, "exploratory": 2}
STATUSES = ("complete", "active", "blocked", "deferred", "planned")


def load_ledger(root: Path = ROOT) -> dict[str, dict]:
    return tomllib.loads((root / LEDGER).read_text())


def find_cycles(tasks: dict[str, dict]) -> list[list[str]]:
    """Dependency cycles, each reported once, as the list of ids along the cycle."""
    WHITE, GREY, BLACK = 0, 1, 2
    colour = {t: WHITE for t in tasks}
    cycles: list[list[str]] = []
    for start in sorted(tasks):
        if colour[start] != WHITE:
            continue
        colour[start] = GREY
        path, stack = [start], [iter(sorted(tasks[start].get("depends", [])))]
        while stack:
            nxt = next(stack[-1], None)
            if nxt is None:
                colour[path.pop()] = BLACK
                stack.pop()
            elif nxt in tasks:
                if colour[nxt] == GREY:
                    cycles.append(path[path.index(nxt):] + [nxt])
                elif colour[nxt] == WHITE:
                    colour[nxt] = GREY
                    path.append(nxt)
                    stack.append(iter(sorted(tasks[nxt].get("depends", []))))
    return cycles


def _key(task_id: str):
    head = task_id.rstrip("0123456789")
    return ("CBMK".find(head[:1]), head, int(task_id[len(head):] or 0))


def render_table(tasks: dict[str, dict]) -> str:
    lines = ["# Components", "",
             "Generated from `docs/plan/ledger.toml` by `python -m incin_b200 xtask ledger --write`; do not edit by hand.",
             "C = core library, B = backends and transports, M = tooling crates, K = device kernels.", "",
             "| id | tier | theme | status | depends on | files | tests | note |", "|---|---|---|---|---|---|---|---|"]
    for tid in sorted(tasks, key=_key):
        t = tasks[tid]
        cell = lambda xs: "<br>".join(f"`{x}`" for x in xs) or "—"   # noqa: E731
        lines.append(f"| {tid} | {t.get('tier', '')} | {t.get('theme', '')} | {t.get('status', '')} | "
                     f"{', '.join(t.get('depends', [])) or '—'} | {cell(t.get('files', []))} | {cell(t.get('tests', []))} | "
                     f"{t.get('note', '')} |")
    return "\n".join(lines) + "\n"


def check_ledger(root: Path = ROOT, tasks: dict[str, dict] | None = None, table: str | None = None) -> list[str]:
    """Every violation as one line; an empty list means the ledger is sound."""
    tasks = load_ledger(root) if tasks is None else tasks
    errors: list[str] = []
    if not tasks:
        return [f"{LEDGER}: no entries"]
    for tid, t in sorted(tasks.items(), key=lambda kv: _key(kv[0])):
        tier, status = t.get("tier"), t.get("status")
        if tier not in MATURITY:
            errors.append(f"{tid}: unknown tier `{tier}`")
        if status not in STATUSES:
            errors.append(f"{tid}: unknown status `{status}`")
        for dep in t.get("depends", []):
            if dep not in tasks:
                errors.append(f"{tid}: depends on unknown component {dep}")
            elif tier in MATURITY and tasks[dep].get("tier") in MATURITY and MATURITY[tasks[dep]["tier"]] > MATURITY[tier]:
                errors.append(f"{tid}: a {tier} component depends on {dep}, which is only {tasks[dep]['tier']}")
        for kind in ("files", "tests"):
            for f in t.get(kind, []):
                if not (root / f).exists():
                    errors.append(f"{tid}: {kind[:-1]} {f} does not exist")
        if status == "complete" and not (t.get("files") and t.get("tests")):
            errors.append(f"{tid}: marked complete without evidence (needs at least one file and one test)")
        if status in ("blocked", "deferred") and not t.get("note"):
            errors.append(f"{tid}: {status} without a note that says why")
    for cyc in find_cycles(tasks):
        errors.append("dependency cycle: " + " -> ".join(cyc))
    if table is None:
        p = root / TABLE
        table = p.read_text() if p.exists() else None
    if table is None:
        errors.append(f"{TABLE}: missing (run `python -m incin_b200 xtask ledger --write`)")
    elif table != render_table(tasks):
        errors.append(f"{TABLE}: differs from the rendering of {LEDGER} (run `python -m incin_b200 xtask ledger --write`)")
    return errors


def docs(check: bool, root: Path = ROOT) -> list[str]:
    """Regenerate (or, with ``check``, compare) every generated document: the capability matrix, the Rust ``-sys``
    bindings and the component table."""
    from . import ffi
    from .__main__ import CAPABILITIES_HEADER
    from .doctor import capability_report
    targets = {"docs/capabilities.md": CAPABILITIES_HEADER + capability_report(), "rust/incin-b200-sys/src/lib.rs": ffi.render_rust(),
               TABLE: render_table(load_ledger(root))}
    stale = []
    for rel, text in targets.items():
        p = root / rel
        if not p.exists() or p.read_text() != text:
            stale.append(rel)
            if not check:
                p.parent.mkdir(parents=True, exist_ok=True)
                p.write_text(text)
    return stale


def main(argv: list[str]) -> int:
    task = argv[0] if argv else None
    if task == "ledger":
        if "--write" in argv:
            (ROOT / TABLE).write_text(render_table(load_ledger()))
        errors = check_ledger()
        for e in errors:
            print("ledger: " + e)
        print(f"ledger: {len(load_ledger())} components, {len(errors)} problem(s)")
        return 1 if errors else 0
    if task == "docs":
        check = "--check" in argv
        stale = docs(check)
        for rel in stale:
            print(f"docs: {rel} {'is stale' if check else 'rewritten'}")
        return 1 if (check and stale) else 0
    if task == "budgets" and len(argv) > 1:
        from .budgets import check_bench
        ok, report = check_bench(argv[1], argv[2] if len(argv) > 2 else None)
        print(report)
        return 0 if ok else 1
    print("usage: python -m incin_b200 xtask {ledger [--write] | docs [--check] | budgets BENCH.json [BUDGETS.json]}")
    return 2
