"""Command line (the role of ``cargo incin``: doctor | plan | tune | inspect | new | watch | capabilities | build).

    python -m incin_b200 doctor [--json]
    python -m incin_b200 plan --world 8 --params 1.1e9 --layers 22 --hidden 2048 --batch 16 --seq 2048 --shard 32
    python -m incin_b200 inspect model.safetensors
    python -m incin_b200 watch run.jsonl
    python -m incin_b200 new my_project
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

TEMPLATE = '''"""{name}: a minimal incin_b200 training script."""
import torch
from incin_b200 import nn
from incin_b200.data import DataLoader, TensorDataset
from incin_b200.optim import SGD, make_store
from incin_b200.train import Trainer

nn.manual_seed(0)
model = nn.seq(nn.Linear(784, 256), nn.ReLU(), nn.Linear(256, 10))
opt = SGD(make_store(model), lr=0.01)
x, y = torch.randn(640, 784), torch.randint(0, 10, (640,))
plan = Trainer.plan().epochs(2).build()
print(plan.explain())
losses = Trainer(plan).fit(model, opt, DataLoader(TensorDataset(x, y), 64),
                           lambda m, a, b: nn.cross_entropy_loss(m(a), b))
print("final loss", losses[-1])
'''


def _passthrough(a) -> int:
    """`run`, `test`, `bench`: the counterpart of the reference CLI's cargo pass-through with its diagnostic humaniser
    (crates/incin/src/bin/cargo-incin.rs:174-200): the wrapped program runs unchanged, shape errors come out explained."""
    import subprocess
    from .diagnostics import explain
    if a.cmd == "run":
        import runpy
        import traceback
        old_argv = sys.argv
        sys.argv = [a.script, *a.args]
        try:
            runpy.run_path(a.script, run_name="__main__")
            return 0
        except SystemExit as e:
            return int(e.code or 0) if not isinstance(e.code, str) else 1
        except Exception as e:   # noqa: BLE001 - the point is to report whatever the script raised
            traceback.print_exc()
            d = explain(str(e))
            if d is not None:
                print(d, file=sys.stderr)
            return 1
        finally:
            sys.argv = old_argv
    if a.cmd == "bench":
        bench = Path(__file__).resolve().parent.parent / "bench.py"
        if not bench.exists():
            print(f"{bench} not found (bench runs from a source tree)", file=sys.stderr)
            return 1
        return subprocess.call([sys.executable, str(bench), *a.args])
    proc = subprocess.Popen([sys.executable, "-m", "pytest", *a.args], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                            text=True)
    for line in proc.stdout:
        sys.stdout.write(line)
        if line.startswith("E "):
            d = explain(line)
            if d is not None:
                sys.stdout.write("".join(f"E   {ln}\n" for ln in str(d).splitlines()))
    return proc.wait()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="incin_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    d = sub.add_parser("doctor"); d.add_argument("--json", action="store_true")
    sub.add_parser("capabilities")
    f = sub.add_parser("ffi"); f.add_argument("--write", action="store_true", help="rewrite rust/incin-b200-sys/src/lib.rs")
    c = sub.add_parser("check"); c.add_argument("bench_json"); c.add_argument("--budgets", default=None)
    sub.add_parser("build")
    sub.add_parser("tune")
    p = sub.add_parser("plan")
    p.add_argument("--world", type=int, default=8); p.add_argument("--params", type=float, default=1.1e9)
    p.add_argument("--layers", type=int, default=22); p.add_argument("--hidden", type=int, default=2048)
    p.add_argument("--batch", type=int, default=16); p.add_argument("--seq", type=int, default=2048)
    p.add_argument("--shard", type=int, default=32); p.add_argument("--objective", default="step_time")
    i = sub.add_parser("inspect"); i.add_argument("path")
    w = sub.add_parser("watch"); w.add_argument("path"); w.add_argument("--once", action="store_true")
    n = sub.add_parser("new"); n.add_argument("name")
    t = sub.add_parser("translate", help="explain a pasted shape error (arguments, or standard input when there are none)")
    t.add_argument("message", nargs="*")
    t.add_argument("--raw", action="store_true", help="print the message unchanged")
    t.add_argument("--explain", action="store_true", help="add the rule of the operation family")
    sub.add_parser("run", help="run SCRIPT [ARGS...]; a shape error ends with its explanation")
    sub.add_parser("test", help="pytest pass-through; error lines get their explanation appended")
    sub.add_parser("bench", help="run bench.py of the source tree with the given flags")
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] in ("run", "test", "bench"):      # everything after the command belongs to the wrapped program
        import types
        if argv[0] == "run" and len(argv) < 2:
            ap.error("run needs a script")
        return _passthrough(types.SimpleNamespace(cmd=argv[0], script=argv[1] if argv[0] == "run" else None,
                                                  args=argv[2:] if argv[0] == "run" else argv[1:]))
    a = ap.parse_args(argv)
    if a.cmd == "doctor":
        from .doctor import doctor
        rep = doctor()
        print(rep.to_json() if a.json else rep.to_text())
        return 0 if rep.healthy else 1
    if a.cmd == "capabilities":
        from .doctor import capability_report
        print(capability_report())
    elif a.cmd == "ffi":
        from . import ffi
        text = ffi.render_rust()
        if a.write:
            out = Path(__file__).resolve().parent.parent / "rust" / "incin-b200-sys" / "src" / "lib.rs"
            out.write_text(text)
            print(f"wrote {out}")
        else:
            print(text)
    elif a.cmd == "check":
        from .budgets import check_bench
        ok, report = check_bench(a.bench_json, a.budgets)
        print(report)
        return 0 if ok else 1
    elif a.cmd == "build":
        from . import build
        print(build())
    elif a.cmd == "tune":
        from .doctor import tune_report
        print(tune_report())
    elif a.cmd == "plan":
        from .doctor import plan_report
        print(plan_report(a.world, params=int(a.params), layers=a.layers, hidden=a.hidden, batch=a.batch, seq=a.seq,
                          shard_extent=a.shard, objective=a.objective))
    elif a.cmd == "inspect":
        from .io import inspect_file
        print(inspect_file(a.path))
    elif a.cmd == "watch":
        from .telemetry.viz import render, watch
        if a.once:
            print(render(a.path))
        else:
            watch(a.path)
    elif a.cmd == "translate":
        from .diagnostics import translate
        text = " ".join(a.message) if a.message else sys.stdin.read()
        print(text.rstrip() if a.raw else translate(text, with_rule=a.explain))
    elif a.cmd == "new":
        d = Path(a.name)
        if d.exists():
            print(f"{d} already exists", file=sys.stderr)
            return 1
        d.mkdir(parents=True)
        (d / "train.py").write_text(TEMPLATE.format(name=a.name))
        print(f"created {d}/train.py")
    return 0


if __name__ == "__main__":
    sys.exit(main())
