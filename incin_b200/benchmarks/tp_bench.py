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
    rank, world = dist.get_rank(), dist.get_world_size()
    assert world == args.tp * args.dp, f"world {world} != tp {args.tp} x dp {args.dp}"
    from incin_b200.engine import TrainStep
    from incin_b200.models.llama import LlamaConfig
    from incin_b200.models.llama_tp import LlamaTP, TPOptimizer
    from incin_b200.ops import gemm as G
    from incin_b200.parallel.mesh import mesh
    from incin_b200.parallel.tp import TensorParallel

    cfg = {"llama-1b": LlamaConfig.llama_1b, "llama-3b": LlamaConfig.llama_3b, "llama-tiny": LlamaConfig.tiny}[args.model]()
    if args.layers:
        cfg.n_layer = args.layers
    spec = mesh(dp=args.dp, tp=args.tp)
    d, _, t = spec.coords(rank)
    tp_groups = [dist.new_group([spec.rank_of(dd, 0, tt) for tt in range(args.tp)]) for dd in range(args.dp)]
    dp_groups = [dist.new_group([spec.rank_of(dd, 0, tt) for dd in range(args.dp)]) for tt in range(args.tp)]
    tp_group = tp_groups[d] if args.dp > 1 else None
    dp_group = dp_groups[t] if args.dp > 1 else None
    B, T = args.batch, args.seq
    Ml = B * T // args.tp
    tpc = TensorParallel(dev, tp_group, max_rows_per_rank=Ml, max_cols=cfg.d_model, mode=args.collectives)
    torch.manual_seed(0)
    model = LlamaTP(cfg, args.tp, t)
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
    opt = TPOptimizer(model, tpc, dev, lr=3e-4, dp_group=dp_group, world_group=None)
    step = TrainStep(model, opt, use_graph=not args.no_graph and args.collectives == "fused")
    gen = torch.Generator().manual_seed(99 + d)
    tok = torch.randint(0, cfg.vocab_size, (B, T), generator=gen).to(dev)
    tgt = torch.randint(0, cfg.vocab_size, (B, T), generator=gen).to(dev)
    losses = []
    for _ in range(max(args.warmup, 3)):
        losses.append(float(step(tok, tgt)))
    G.check_status(dev)
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step(tok, tgt)
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    lt = loss.clone()
    dist.all_reduce(lt)
    G.check_status(dev)
    if rank == 0:
        ms_step = float(ms) / args.steps
        tokens = B * T * args.dp
        flops = cfg.flops_per_token(T) * tokens / world / (ms_step / 1e3)
        print(json.dumps({"metric": "train tokens/sec", "model": args.model, "layers": cfg.n_layer, "tp": args.tp,
                          "dp": args.dp, "collectives": args.collectives, "global_batch": B * args.dp, "seq_len": T,
                          "value": tokens / (ms_step / 1e3), "ms_per_step": ms_step, "n_gpus": world,
                          "model_tflops_per_gpu": flops / 1e12, "cuda_graph": step.graph is not None,
                          "loss_first": losses[0], "loss_last": float(lt) / args.dp, "dtype": "bf16",
                          "data": "synthetic"}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
