"""Pipeline-parallel stage runner on CPU ranks (gloo): every schedule / checkpoint mode must reproduce the gradients
and the loss of the unsplit model."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

WORLD, MICRO = 3, 6


def _worker(rank, port, sched, ckpt, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        from incin_b200.parallel.pp import DistEdge, PipelineStage, StageIO
        from incin_b200.parallel.strategies import ActivationCheckpoint, PipelineSchedule
        torch.manual_seed(0)
        layers = [torch.nn.Sequential(torch.nn.Linear(16, 16), torch.nn.Tanh()) for _ in range(WORLD)]
        full = torch.nn.Sequential(*layers)
        xs = [torch.randn(4, 16) for _ in range(MICRO)]
        ts = [torch.randn(4, 16) for _ in range(MICRO)]
        ref = sum(torch.nn.functional.mse_loss(full(x), t) for x, t in zip(xs, ts)) / MICRO
        ref.backward()
        want = [p.grad.clone() for p in layers[rank].parameters()]
        full.zero_grad()
        io = StageIO(fwd_in=DistEdge(rank - 1, rank) if rank > 0 else None,
                     fwd_out=DistEdge(rank, rank + 1) if rank < WORLD - 1 else None,
                     bwd_in=DistEdge(rank + 1, rank) if rank < WORLD - 1 else None,
                     bwd_out=DistEdge(rank, rank - 1) if rank > 0 else None)
        stage = PipelineStage(layers[rank], rank, WORLD, io, (4, 16), torch.float32, "cpu", PipelineSchedule(sched),
                              ActivationCheckpoint(ckpt))
        losses = stage.step(xs, lambda y, m: torch.nn.functional.mse_loss(y, ts[m]), microbatches=MICRO)
        err = max(float((p.grad - g).abs().max()) for p, g in zip(layers[rank].parameters(), want))
        loss = float(torch.stack(losses).mean()) if losses else None
        q.put((rank, err, loss, float(ref.detach())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("sched,ckpt", [("gpipe", "keep"), ("1f1b", "keep"), ("1f1b", "recompute")])
def test_pipeline_matches_unsplit_model(sched, ckpt):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29640 + hash((sched, ckpt)) % 50
    procs = [ctx.Process(target=_worker, args=(r, port, sched, ckpt, q)) for r in range(WORLD)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in range(WORLD))
    for p in procs:
        p.join(30)
    for rank, err, loss, ref in results:
        assert err < 1e-6, (rank, err)
        if rank == WORLD - 1:
            assert abs(loss - ref) < 1e-6
