"""Per-launch device times of one eager GPT-2 training step, from the per-step CUDA-event trace.

    python -m incin_b200.benchmarks.step_trace [--model gpt2-small] [--batch 8] [--seq 1024] [--steps 3]

Unlike a profiler's launch list (serialised, cold caches) the trace times the launches inside a running step: events sit
back to back on the launching stream, so a row is the device time of that call's kernels with warm caches (plus any gap
the host left before the next launch: the eager step is launch-bound in places, which is what the CUDA-graph replay of
the same step removes).  Rows are grouped by native call name; the last line compares the eager step with its replay.
"""
from __future__ import annotations

import argparse
import json

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gpt2-small", choices=["gpt2-small", "gpt2-tiny"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=3)
    args = ap.parse_args()
    from incin_b200.engine import TrainStep
    from incin_b200.models.gpt2 import GPT2, GPT2Config
    from incin_b200.optim import AdamW, ParamStore
    from incin_b200.telemetry import trace
    cfg = GPT2Config.small() if args.model == "gpt2-small" else GPT2Config.tiny()
    T = min(args.seq, cfg.max_seq)
    dev = torch.device("cuda", torch.cuda.current_device())
    model = GPT2(cfg, seed=0).to(dev)
    step = TrainStep(model, AdamW(ParamStore(model.named_parameters()), lr=3e-4), use_graph=False)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (args.batch, T), generator=g).to(dev)
    tgt = torch.randint(0, cfg.vocab_size, (args.batch, T), generator=g).to(dev)
    for _ in range(3):
        step(tok, tgt)
    trace.enable(events=True)
    rows = []
    for _ in range(args.steps):
        trace.begin_step()
        step(tok, tgt)
        rows = trace.end_step()
    trace.enable(events=False)
    total = sum(ms for _, ms in rows)
    for r in trace.summary(rows):
        print(json.dumps(r))
    replay = TrainStep(model, AdamW(ParamStore(model.named_parameters()), lr=3e-4), use_graph=True)
    for _ in range(4):
        replay(tok, tgt)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        replay(tok, tgt)
    e1.record()
    torch.cuda.synchronize()
    print(json.dumps({"eager_step_ms": round(total, 3), "native_calls": len(rows),
                      "graph_replay_step_ms": round(e0.elapsed_time(e1) / 10, 3), "graph": replay.graph is not None}))


if __name__ == "__main__":
    main()
