"""Worker for the multi-GPU collective test (torch.distributed.run, one rank per GPU): the stand-alone peer-memory
collectives against torch.distributed results, a pipeline channel round trip, a two-stage pipeline step against the
unsplit model, and a bounded wait that runs out (a flag nobody sets) reporting through the status word."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from incin_b200 import _native as nat
    from incin_b200.ops import gemm as G
    from incin_b200.parallel.collectives import PeerCollectives, PipelineChannel
    from incin_b200.parallel.pp import PeerEdge, PipelineStage, StageIO
    from incin_b200.parallel.strategies import PipelineSchedule
    out = {"world": world}
    pc = PeerCollectives(dev, max_bytes=8 << 20)
    torch.manual_seed(100 + rank)
    for dtype in (torch.float32, torch.bfloat16):
        x = torch.randn(world * 64, 96, device=dev).to(dtype)
        for it in range(2):      # twice: staging-buffer reuse across calls
            ag = pc.all_gather(x)
            ref = torch.empty(world * x.shape[0], 96, dtype=dtype, device=dev)
            dist.all_gather_into_tensor(ref, x)
            out[f"ag_{dtype}_{it}"] = bool(torch.equal(ag, ref))
            for op, rop in (("sum", dist.ReduceOp.SUM), ("max", dist.ReduceOp.MAX), ("mean", dist.ReduceOp.AVG)):
                ar = pc.all_reduce(x, op)
                ref = x.float().clone()
                dist.all_reduce(ref, rop)
                tol = 1e-5 if dtype == torch.float32 else 3e-2
                out[f"ar_{op}_{dtype}_{it}"] = bool(torch.allclose(ar.float(), ref, rtol=tol, atol=tol))
                gathered = [torch.empty_like(ar) for _ in range(world)]
                dist.all_gather(gathered, ar)
                out[f"ar_{op}_{dtype}_{it}_bitwise_equal_on_all_ranks"] = all(torch.equal(g, ar) for g in gathered)
            rs = pc.reduce_scatter(x, "sum")
            ref = torch.empty(64, 96, dtype=torch.float32, device=dev)
            dist.reduce_scatter_tensor(ref, x.float())
            out[f"rs_{dtype}_{it}"] = bool(torch.allclose(rs.float(), ref, rtol=3e-2, atol=3e-2))
            a2a = pc.all_to_all(x)
            ref = torch.empty_like(x)
            dist.all_to_all_single(ref, x)
            out[f"a2a_{dtype}_{it}"] = bool(torch.equal(a2a, ref))
    G.check_status(dev)

    # pipeline channel: rank 0 -> rank 1, more messages than slots (the receiver drains between sends)
    ch = PipelineChannel(dev, 0, 1, 64 * 128 * 2, depth=2)
    ok = True
    for k in range(5):
        msg = torch.full((64, 128), float(k + 1), dtype=torch.bfloat16, device=dev)
        if rank == 0:
            ch.send(msg)
        elif rank == 1:
            got = ch.recv((64, 128), torch.bfloat16)
            ok = ok and bool(torch.equal(got, msg))
        torch.cuda.synchronize()
        dist.barrier()          # slot reuse is separated by the schedule in real use; here by a host barrier
    out["channel"] = ok
    G.check_status(dev)

    # two-stage pipeline over the first two ranks vs the unsplit model
    if world >= 2:
        torch.manual_seed(0)
        layers = [torch.nn.Sequential(torch.nn.Linear(32, 32), torch.nn.Tanh()).to(dev) for _ in range(2)]
        full = torch.nn.Sequential(*layers)
        xs = [torch.randn(8, 32, device=dev) for _ in range(4)]
        ts = [torch.randn(8, 32, device=dev) for _ in range(4)]
        ref = sum(torch.nn.functional.mse_loss(full(a), b) for a, b in zip(xs, ts)) / 4
        ref.backward()
        fwd = PipelineChannel(dev, 0, 1, 8 * 32 * 4, depth=4)
        bwd = PipelineChannel(dev, 1, 0, 8 * 32 * 4, depth=4)
        if rank < 2:
            want = [p.grad.clone() for p in layers[rank].parameters()]
            full.zero_grad()
            io = StageIO(fwd_in=PeerEdge(fwd) if rank == 1 else None, fwd_out=PeerEdge(fwd) if rank == 0 else None,
                         bwd_in=PeerEdge(bwd) if rank == 0 else None, bwd_out=PeerEdge(bwd) if rank == 1 else None)
            st = PipelineStage(layers[rank], rank, 2, io, (8, 32), torch.float32, dev, PipelineSchedule.ONE_F_ONE_B)
            losses = st.step(xs, lambda y, m: torch.nn.functional.mse_loss(y, ts[m]), microbatches=4)
            torch.cuda.synchronize()
            err = max(float((p.grad - g).abs().max()) for p, g in zip(layers[rank].parameters(), want))
            out["pipeline_grad_err"] = err
            out["pipeline"] = err < 1e-5 and (rank == 0 or abs(float(torch.stack(losses).mean()) - float(ref)) < 1e-5)
        G.check_status(dev)
        dist.barrier()

    # a wait that runs out: nobody sets this flag; the kernel gives up after 50 ms and the host reads the status
    if rank == 0:
        flag = torch.zeros(64, dtype=torch.int32, device=dev)
        nat.check(nat.cuda().incin_p2p_wait(flag.data_ptr(), 1, G.status_word(dev).data_ptr(), 50, nat.stream_ptr()), "p2p_wait")
        try:
            G.check_status(dev)
            out["timeout_reported"] = False
        except nat.NativeError:
            out["timeout_reported"] = True
        z = torch.ones(4, device=dev).sum().item()      # the context is still usable
        out["context_alive"] = z == 4.0
    dist.barrier()
    everyone = [None] * world
    dist.all_gather_object(everyone, out)
    if rank == 0:       # one line, printed by one process: lines of several ranks can interleave
        print("COLL_RESULT " + json.dumps(everyone), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
