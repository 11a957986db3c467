"""Tensor-parallel / 2-D mesh training throughput (tokens/s), device-timed, max over ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \\
        -m incin_b200.benchmarks.tp_bench --model llama-1b --tp 8 --batch 16 --seq 2048 --steps 5 --warmup 3
    ... --model llama-3b --tp 4 --dp 2 --batch 2 --seq 4096      (batch = sequences per data-parallel replica)
    ... --collectives nccl                                         (baseline arm: NCCL all-gather / reduce-scatter)

Synthetic data (uniform token ids), random-init N(0, 0.02) weights, bf16 compute with fp32 master weights, AdamW.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def run(model_name: str, tp: int, dp: int, batch: int, seq: int, steps: int = 5, warmup: int = 3,
        collectives: str = "fused", use_graph: bool = True, layers: int = 0, ctx=None) -> dict | None:
    """One measurement inside an initialised process group of ``tp * dp`` ranks (one GPU each, current device set).
    Returns the result row on rank 0, None elsewhere.  Everything it allocates is released before it returns.
    ``ctx``: a rendezvous context of the job; the fused arm then runs under the plan contract (the step's collectives
    are agreed on before any peer mapping is opened, handles travel over the context's control channel, every fused
    launch is checked against the plan)."""
    dev = torch.device("cuda", torch.cuda.current_device())
    rank, world = dist.get_rank(), dist.get_world_size()
    assert world == tp * dp, f"world {world} != tp {tp} x dp {dp}"
    from incin_b200.engine import TrainStep
    from incin_b200.models.llama import LlamaConfig
    from incin_b200.models.llama_tp import LlamaTP, TPOptimizer
    from incin_b200.ops import gemm as G
    from incin_b200.parallel.mesh import mesh
    from incin_b200.parallel.tp import TensorParallel

    cfg = {"llama-1b": LlamaConfig.llama_1b, "llama-3b": LlamaConfig.llama_3b, "llama-tiny": LlamaConfig.tiny}[model_name]()
    if layers:
        cfg.n_layer = layers
    spec = mesh(dp=dp, tp=tp)
    d, _, t = spec.coords(rank)
    tp_group = dp_group = None
    if dp > 1:
        tp_groups = [dist.new_group([spec.rank_of(dd, 0, tt) for tt in range(tp)]) for dd in range(dp)]
        dp_groups = [dist.new_group([spec.rank_of(dd, 0, tt) for dd in range(dp)]) for tt in range(tp)]
        tp_group, dp_group = tp_groups[d], dp_groups[t]
    B, T = batch, seq
    Ml = B * T // tp
    session = plan = tp_ranks = dp_ranks = None
    if ctx is not None and collectives == "fused":
        from incin_b200.models.llama_tp import tensor_parallel_plan
        from incin_b200.parallel.session import bind_session
        session = bind_session(ctx, spec)
        plan = tensor_parallel_plan(cfg, session.mesh, rank, B * T)
        tp_ranks = [spec.rank_of(d, 0, tt) for tt in range(tp)]
        dp_ranks = [spec.rank_of(dd, 0, t) for dd in range(dp)]
    tpc = TensorParallel(dev, tp_group, max_rows_per_rank=Ml, max_cols=cfg.d_model, mode=collectives, session=session,
                         plan=plan, ranks=tp_ranks)
    torch.manual_seed(0)
    model = LlamaTP(cfg, tp, t)
    with torch.no_grad():       # random-init N(0, 0.02) directly on the shards (no full model on the host)
        g = torch.Generator().manual_seed(1000 + t)
        for name, p in model.named_parameters():
            if p.dim() >= 2:
                if name in ("embed", "lm_head"):
                    p.normal_(0.0, cfg.init_std, generator=torch.Generator().manual_seed(7 + (name == "lm_head")))
                else:
                    p.normal_(0.0, cfg.init_std, generator=g)
    model = model.to(dev)
    model.tp = tpc
    opt = TPOptimizer(model, tpc, dev, lr=3e-4, dp_group=dp_group, world_group=None, session=session, dp_ranks=dp_ranks)
    step = TrainStep(model, opt, use_graph=use_graph and collectives == "fused")
    gen = torch.Generator().manual_seed(99 + d)
    tok = torch.randint(0, cfg.vocab_size, (B, T), generator=gen).to(dev)
    tgt = torch.randint(0, cfg.vocab_size, (B, T), generator=gen).to(dev)
    losses = []
    for _ in range(max(warmup, 3)):
        losses.append(float(step(tok, tgt)))
    G.check_status(dev)
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        loss = step(tok, tgt)
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    lt = loss.detach().clone()
    dist.all_reduce(lt)
    G.check_status(dev)
    row = None
    if rank == 0:
        ms_step = float(ms) / steps
        tokens = B * T * dp
        flops = cfg.flops_per_token(T) * tokens / world / (ms_step / 1e3)
        row = {"metric": "train tokens/sec", "model": model_name, "layers": cfg.n_layer, "tp": tp, "dp": dp,
               "collectives": collectives, "global_batch": B * dp, "seq_len": T, "value": tokens / (ms_step / 1e3),
               "ms_per_step": ms_step, "n_gpus": world, "steps": steps, "model_tflops_per_gpu": flops / 1e12,
               "cuda_graph": step.graph is not None, "loss_first": losses[0] * tp, "loss_last": float(lt) / dp,
               "plan_validated_launches": (session.launches if session is not None else 0),
               "dtype": "bf16", "data": "synthetic"}
    del step, opt, model, tpc, tok, tgt, loss
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return row


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-1b", choices=["llama-1b", "llama-3b", "llama-tiny"])
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--collectives", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0 = the model's own)")
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    row = run(args.model, args.tp, args.dp, args.batch, args.seq, args.steps, args.warmup, args.collectives,
              use_graph=not args.no_graph, layers=args.layers)
    if row is not None:
        print(json.dumps(row), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
