"""Regression budgets: compare a benchmark result with the committed floor for its configuration.

Counterpart of the reference's ``xtask`` regression-budget check (xtask/src/main.rs:15-30 against
docs/plan/baselines/main.toml) and its README feature-table generator.  ``budgets.json`` beside this module holds,
per ``(metric config, n_gpus)``, the value a change must not fall below (higher-is-better metrics) after the allowed
slack; ``python -m incin_b200 check BENCH.json`` exits non-zero when a result violates its budget.
"""
from __future__ import annotations

import json
from pathlib import Path

DEFAULT = Path(__file__).with_name("budgets.json")


def load_budgets(path=None) -> dict:
    return json.loads(Path(path or DEFAULT).read_text())


def check_bench(bench_json, budgets_path=None) -> tuple[bool, str]:
    text = Path(bench_json).read_text().strip().splitlines()
    line = next((l for l in reversed(text) if l.lstrip().startswith("{")), None)
    if line is None:
        return False, "no JSON line in the benchmark output"
    res = json.loads(line)
    budgets = load_budgets(budgets_path)
    model = res.get("config", {}).get("model", "?")
    key = f"{model}/n{res.get('n_gpus', 1)}"
    b = budgets["entries"].get(key)
    if b is None:
        return True, f"{key}: no budget recorded (value {res.get('value')})"
    slack = budgets.get("slack", 0.05)
    floor = b["value"] * (1.0 - slack)
    higher = res.get("higher_is_better", True)
    ok = res["value"] >= floor if higher else res["value"] <= b["value"] * (1.0 + slack)
    return ok, (f"{key}: {res['value']:.1f} {res.get('unit', '')} vs budget {b['value']:.1f} "
                f"({'ok' if ok else 'REGRESSION'}; slack {slack:.0%}, recorded on {b.get('hardware', '?')})")


def feature_table() -> str:
    """The capability matrix for the README, generated from the registries."""
    from .core.spec import capability_table_markdown
    return capability_table_markdown()
