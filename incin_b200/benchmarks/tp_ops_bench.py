"""Per-op benchmark of the fused tensor-parallel kernels against the NCCL collective + local GEMM pair.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29500 \\
        -m incin_b200.benchmarks.tp_ops_bench --rows 16384 --hidden 2048 --shard-cols 384,1408 --copy-ctas 8,16,32

For each shape it times (CUDA events, max over ranks, input larger than L2):
  all-gather -> GEMM   x_shard [rows, hidden]  @ W[cols, hidden]^T   -> [tp*rows, cols]
  GEMM -> reduce-scatter  a [tp*rows, cols] @ W[hidden, cols]^T      -> [rows, hidden]
and prints one JSON line per measurement with the bytes that had to cross NVLink per GPU and the resulting GB/s,
next to the roofline time max(FLOPs / GEMM peak, link bytes / 770 GB/s).

    python -m incin_b200.benchmarks.tp_ops_bench --loopback 2 --rows 16384 --shard-cols 384 --copy-ctas 32 --iters 3

``--loopback N`` runs the same two fused launches in ONE process on one GPU as rank 0 of an N-rank group whose "peer"
buffers are local allocations: the kernel code paths (copy CTAs or copy warps, flags, tile order) are the ones a real
group runs, which makes them measurable with a profiler that must not wrap a multi-rank command.  Times are then a
measure of the kernel's own copy machinery against local memory, not of NVLink.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _time(fn, iters, dev):
    for _ in range(3):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], dtype=torch.float64, device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms)


def loopback(args) -> None:
    from incin_b200.ops import gemm as G
    dev = torch.device("cuda", torch.cuda.current_device())
    world, Ml, H = args.loopback, args.rows, args.hidden
    M = Ml * world

    def timed(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.iters

    shards = [(torch.randn(Ml, H, device=dev) * 0.1).bfloat16() for _ in range(world)]
    for cols in [int(c) for c in args.shard_cols.split(",")]:
        w_col = (torch.randn(cols, H, device=dev) * 0.02).bfloat16()
        w_row = (torch.randn(H, cols, device=dev) * 0.02).bfloat16()
        a = (torch.randn(M, cols, device=dev) * 0.1).bfloat16()
        gathered = torch.zeros(M, H, dtype=torch.bfloat16, device=dev)
        gathered[:Ml].copy_(shards[0])                  # rank 0's own rows are in place, as in the real op
        out = torch.empty(M, cols, dtype=torch.bfloat16, device=dev)
        slots = [torch.zeros(world, Ml, H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        stage = torch.empty(M, H, dtype=torch.bfloat16, device=dev)
        src = [0] + [s.data_ptr() for s in shards[1:]]
        for cc in [int(c) for c in args.copy_ctas.split(",")]:
            def ag():
                flags = torch.zeros(M // 128, dtype=torch.int32, device=dev)
                G.gemm(gathered, w_col, out, M=M, N=cols, K=H, lda=H, ldb=H, ldc=cols,
                       gather={"world": world, "rank": 0, "rows_per_rank": Ml, "src": src, "flags": flags, "copy_ctas": cc or 32})

            def rs():
                ready = torch.zeros(M // 128, dtype=torch.int32, device=dev)
                G.gemm(a, w_row, stage, M=M, N=H, K=cols, lda=cols, ldb=cols, ldc=H,
                       scatter={"world": world, "rank": 0, "rows_per_rank": Ml, "dst": [t.data_ptr() for t in slots],
                                "slot_stride": Ml * H, "ready": ready, "copy_ctas": cc or 32})
            t_ag, t_rs = timed(ag), timed(rs)
            G.check_status(dev)
            ok = torch.equal(gathered, torch.cat(shards, 0))
            moved = (world - 1) * Ml * H * 2
            for op, ms in (("all_gather_gemm", t_ag), ("gemm_reduce_scatter", t_rs)):
                print(json.dumps({"loopback": world, "rows_per_rank": Ml, "hidden": H, "shard_cols": cols, "copy_ctas": cc or 32,
                                  "op": op, "ms": ms, "copied_gbs": moved / ms / 1e6, "gathered_ok": ok}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--loopback", type=int, default=0, help="emulate rank 0 of this many ranks on one GPU with local peers")
    ap.add_argument("--rows", type=int, default=16384, help="rows per rank")
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--shard-cols", default="384,1408")
    ap.add_argument("--copy-ctas", default="0")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--gemm-peak-tflops", type=float, default=1400.0)
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if args.loopback:
        loopback(args)
        return
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from incin_b200.ops import gemm as G
    from incin_b200.parallel.tp import TensorParallel

    Ml, H = args.rows, args.hidden
    M = Ml * world
    torch.manual_seed(rank)
    x = (torch.randn(Ml, H, device=dev) * 0.1).bfloat16()
    link = (world - 1) / world * M * H * 2
    for cols in [int(c) for c in args.shard_cols.split(",")]:
        w_col = (torch.randn(cols, H, device=dev) * 0.02).bfloat16()
        w_row = (torch.randn(H, cols, device=dev) * 0.02).bfloat16()
        a = (torch.randn(M, cols, device=dev) * 0.1).bfloat16()
        flops = 2.0 * M * H * cols
        roof = max(flops / (args.gemm_peak_tflops * 1e12), link / 770e9) * 1e3
        # a count, 0 (the per-call model) or "tune" (measured under the collective tuning contract, then timed)
        arms = [("nccl", 0)] + [("fused", c if c == "tune" else int(c)) for c in args.copy_ctas.split(",")]
        ref = {}
        for mode, cc in arms:
            tuned = cc == "tune"
            tp = TensorParallel(dev, None, max_rows_per_rank=Ml, max_cols=max(H, cols), mode=mode, copy_ctas=0 if tuned else cc)
            if tuned:
                tp.tune_copy_ctas("gather", x, w_col)
                tp.tune_copy_ctas("scatter", a, w_row)
            ag = _time(lambda: tp.gather_gemm(x, w_col), args.iters, dev)
            rs = _time(lambda: tp.gemm_scatter(a, w_row), args.iters, dev)
            G.check_status(dev)
            # the fused kernels must reproduce the collective + GEMM pair (same bf16 inputs, fp32 accumulation)
            o_ag = tp.gather_gemm(x, w_col)[0].float()
            o_rs = tp.gemm_scatter(a, w_row).float()
            if mode == "nccl":
                ref = {"ag": o_ag, "rs": o_rs}
            else:
                e_ag = float((o_ag - ref["ag"]).abs().max())
                e_rs = float((o_rs - ref["rs"]).abs().max() / ref["rs"].abs().max())
                assert e_ag == 0.0 and e_rs < 2e-2, (e_ag, e_rs)
            if rank == 0:
                base = {"tp": world, "rows_per_rank": Ml, "hidden": H, "shard_cols": cols, "mode": mode,
                        "copy_ctas": (sorted(tp._tuned.items()) if tuned else tp.copy_ctas) if mode == "fused" else None,
                        "link_mb_per_gpu": link / 2 ** 20,
                        "roofline_ms": roof}
                print(json.dumps({**base, "op": "all_gather_gemm", "ms": ag, "link_gbs": link / ag / 1e6,
                                  "of_roofline": roof / ag}), flush=True)
                if rs is not None:
                    print(json.dumps({**base, "op": "gemm_reduce_scatter", "ms": rs, "link_gbs": link / rs / 1e6,
                                      "of_roofline": roof / rs}), flush=True)
            del tp
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
