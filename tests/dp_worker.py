"""Worker for the multi-GPU data-parallel test (launched by torch.distributed.run, one rank per GPU).

Trains GPT-2 (tiny) for a few steps with each gradient reducer from the same initial weights and
different data per rank, and checks that (a) every rank ends with bit-identical parameters, (b) the
fused peer-memory reducers agree with the NCCL all-reduce baseline, and (c) no device-side wait timed out.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run(kind: str, use_graph: bool, steps: int = 5, session=None):
    from incin_b200.engine import TrainStep
    from incin_b200.models.gpt2 import GPT2, GPT2Config
    from incin_b200.optim import AdamW, ParamStore
    from incin_b200.parallel import dp as DP
    rank = dist.get_rank()
    device = torch.device("cuda", torch.cuda.current_device())
    cfg = GPT2Config.tiny()
    model = GPT2(cfg, seed=0).to(device)
    reducer, allocator, desc = DP.make_reducer(kind, device, session=session)
    if isinstance(reducer, DP.FusedReducer):
        reducer.bucket_elems = 1 << 16  # several buckets even for the tiny model
    store = ParamStore(model.named_parameters(), allocator=allocator)
    opt = AdamW(store, lr=1e-3, weight_decay=0.1)
    reducer.attach(store, opt)
    step = TrainStep(model, opt, use_graph=use_graph, reducer=reducer)
    g = torch.Generator().manual_seed(100 + rank)
    losses = []
    tok = torch.randint(0, cfg.vocab_size, (2, 128), generator=g).to(device)  # one fixed batch per rank
    tgt = torch.randint(0, cfg.vocab_size, (2, 128), generator=g).to(device)
    for i in range(steps):
        losses.append(float(step(tok, tgt)))
    torch.cuda.synchronize()
    return store.shadow.float().clone(), losses, desc


def run_trainer(steps: int = 5, session=None):
    """The same training through the public ``Trainer`` API on a plan of every GPU of the job."""
    from incin_b200.core.device import DeviceSet
    from incin_b200.models.gpt2 import GPT2, GPT2Config
    from incin_b200.optim import AdamW, ParamStore
    from incin_b200.parallel import dp as DP
    from incin_b200.train import Trainer
    rank, world = dist.get_rank(), dist.get_world_size()
    device = torch.device("cuda", torch.cuda.current_device())
    plan = Trainer.plan().devices(DeviceSet.cuda(range(world))).epochs(1).build()
    assert plan.is_multi_device and "collectives-required" in [d.code for d in plan.decisions]
    cfg = GPT2Config.tiny()
    model = GPT2(cfg, seed=0).to(device)
    reducer, allocator, _ = DP.make_reducer("auto", device, session=session)
    store = ParamStore(model.named_parameters(), allocator=allocator)
    opt = AdamW(store, lr=1e-3, weight_decay=0.1)
    reducer.attach(store, opt)
    g = torch.Generator().manual_seed(100 + rank)
    tok = torch.randint(0, cfg.vocab_size, (2, 128), generator=g).pin_memory()
    tgt = torch.randint(0, cfg.vocab_size, (2, 128), generator=g).pin_memory()
    seen = []
    losses = Trainer(plan).fit(model, opt, [(tok, tgt)] * steps, on_step=lambda n, v: seen.append(n))
    torch.cuda.synchronize()
    assert seen == list(range(1, steps + 1))
    return store.shadow.float().clone(), list(losses)


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from incin_b200.ops import gemm as G
    rank, world = dist.get_rank(), dist.get_world_size()
    out = {"world": world}
    ref, ref_losses, _ = run("nccl", False)
    ok = True
    # the fused arms run under the repo's own control plane: plan agreed before the peer mappings exist, IPC handles
    # over the rendezvous channel, every bucket launch checked against the plan cursor
    from incin_b200.parallel.context import DistributedContext
    from incin_b200.parallel.mesh import mesh
    from incin_b200.parallel.session import bind_session
    session = bind_session(DistributedContext.from_env(), mesh(dp=world))
    for kind, graph in (("fused-tail", False), ("fused", False), ("fused", True)):
        before = session.launches
        w, losses, desc = run(kind, graph, session=session)
        ok = ok and session.launches > before
        G.check_status()
        gathered = [torch.empty_like(w) for _ in range(world)]
        dist.all_gather(gathered, w)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        err = (w - ref).abs().max().item()
        out[f"{kind}{'-graph' if graph else ''}"] = {"ranks_identical": same, "max_abs_diff_vs_nccl": err,
                                                     "loss_first": losses[0], "loss_last": losses[-1]}
        ok = ok and same and err < 2e-2 and losses[-1] < losses[0]
    w, losses = run_trainer(session=session)
    err = (w - ref).abs().max().item()
    out["trainer_fit"] = {"max_abs_diff_vs_nccl": err, "loss_first": losses[0], "loss_last": losses[-1]}
    ok = ok and err < 2e-2 and len(losses) == 5 and max(abs(a - b) for a, b in zip(losses, ref_losses)) < 5e-2
    out["plan_validated_launches"] = session.launches
    out["multimem"] = bool(os.environ.get("INCIN_TEST_EXPECT_MULTIMEM") == "1")
    if out["multimem"]:      # the launcher asked for the NVSwitch multicast variant: make sure that is what ran
        from incin_b200.parallel.symm import MulticastBuffer
        ok = ok and MulticastBuffer.available()
    out["ok"] = ok
    if rank == 0:
        print("DP_RESULT " + json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
