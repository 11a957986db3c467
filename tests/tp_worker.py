"""Worker for the multi-GPU tensor-parallel test (torch.distributed.run, one rank per GPU).

Checks the two fused kernels against plain math (all-gather -> GEMM, GEMM -> reduce-scatter), then trains a tiny
Llama tensor-parallel and compares loss and parameters with the same model trained on one GPU."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from incin_b200.engine import TrainStep
    from incin_b200.models.llama import Llama, LlamaConfig
    from incin_b200.models.llama_tp import LlamaTP, TPOptimizer
    from incin_b200.ops import gemm as G
    from incin_b200.optim import AdamW, make_store
    from incin_b200.parallel.tp import TensorParallel
    out = {"world": world}

    # ---- kernel level
    Ml, Kd, N = 256, 320, 448
    tp = TensorParallel(dev, max_rows_per_rank=Ml, max_cols=max(Kd, N, 512))
    g = torch.Generator().manual_seed(7)
    x_full = (torch.randn(world * Ml, Kd, generator=g)).to(torch.bfloat16).to(dev)
    w = (torch.randn(N, Kd, generator=g) * 0.1).to(torch.bfloat16).to(dev)
    for it in range(3):   # repeated: exercises buffer parities and barrier epochs
        y, gathered = tp.gather_gemm(x_full[rank * Ml:(rank + 1) * Ml].contiguous(), w)
        G.check_status()
        out[f"ag_gemm_{it}"] = max(rel(y, x_full.float() @ w.float().t()), rel(gathered, x_full))
    a = (torch.randn(world * Ml, Kd, generator=torch.Generator().manual_seed(100 + rank))).to(torch.bfloat16).to(dev)
    res = torch.randn(Ml, N, generator=g).to(torch.bfloat16).to(dev)
    for it in range(3):
        ys = tp.gemm_scatter(a, w, residual=res)
        G.check_status()
        part = (a.float() @ w.float().t())
        dist.all_reduce(part)
        out[f"gemm_rs_{it}"] = rel(ys, part[rank * Ml:(rank + 1) * Ml] + res.float())

    # ---- the copy-CTA count of a shape, measured under the collective tuning contract (same candidates on every
    # rank, median of the max over ranks, unanimous commit); the committed count is then what the op launches with
    committed = tp.tune_copy_ctas("gather", x_full[rank * Ml:(rank + 1) * Ml].contiguous(), w, candidates=(4, 8), samples=2)
    out["tuned_gather"] = {"candidate": committed.candidate, "world": committed.world, "picked": tp._tuned[("gather", Ml, Kd, N)]}
    y2, _ = tp.gather_gemm(x_full[rank * Ml:(rank + 1) * Ml].contiguous(), w)
    out["ag_gemm_tuned"] = rel(y2, x_full.float() @ w.float().t())
    tp.tune_copy_ctas("scatter", a, w, candidates=(4, 8), samples=2)
    out["tuned_scatter_picked"] = tp._tuned[("scatter", Ml, Kd, N)]
    G.check_status()

    # ---- model level
    # the first model runs under the repo's own control plane (plan agreed before any peer mapping, handles over the
    # rendezvous channel, every fused launch checked against the plan cursor); the second on the torch.distributed plumbing
    from incin_b200.models.llama_tp import tensor_parallel_plan
    from incin_b200.parallel.context import DistributedContext
    from incin_b200.parallel.mesh import mesh
    from incin_b200.parallel.session import bind_session
    session = bind_session(DistributedContext.from_env(), mesh(tp=world))
    for name, kvh in (("sharded_kv", 2), ("shared_kv", 1)):
        cfg = LlamaConfig(vocab_size=512, n_layer=2, d_model=256, n_head=4, n_kv_head=kvh, head_dim=64, d_ffn=512)
        B, T = 4, 128
        sess = session if name == "sharded_kv" else None
        tpm = TensorParallel(dev, max_rows_per_rank=B * T // world, max_cols=cfg.d_model, session=sess,
                             plan=tensor_parallel_plan(cfg, session.mesh, rank, B * T) if sess else None,
                             ranks=list(range(world)) if sess else None)
        if sess is not None:
            # the same measurement with the reports and votes travelling over the session's control channel
            xs = torch.randn(B * T // world, cfg.d_model, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(dev)
            ws = (torch.randn(384, cfg.d_model, generator=torch.Generator().manual_seed(6)) * 0.1).to(torch.bfloat16).to(dev)
            c2 = tpm.tune_copy_ctas("gather", xs, ws, candidates=(4, 8), samples=2)
            out["tuned_over_session"] = c2.world == world and tpm._tuned[("gather", B * T // world, cfg.d_model, 384)] in (4, 8)
        gg = torch.Generator().manual_seed(3)
        tok = torch.randint(0, cfg.vocab_size, (B, T), generator=gg).to(dev)
        tgt = torch.randint(0, cfg.vocab_size, (B, T), generator=gg).to(dev)
        ref = Llama(cfg, seed=0).to(dev)
        ref_opt = AdamW(make_store(ref), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
        ref_step = TrainStep(ref, ref_opt, use_graph=False)
        m = LlamaTP.from_seed(cfg, world, rank, seed=0).to(dev)
        m.tp = tpm
        opt = TPOptimizer(m, tpm, dev, lr=1e-3, session=sess)
        step = TrainStep(m, opt, use_graph=False)
        lr_, lt_ = [], []
        for _ in range(4):
            lr_.append(float(ref_step(tok, tgt)))
            l = step(tok, tgt).clone()
            dist.all_reduce(l)
            lt_.append(float(l))
        G.check_status()
        full_q = dict(ref.named_parameters())["blocks.1.qkv_w"][: cfg.n_head * 64]
        mine = dict(m.named_parameters())["blocks.1.q_w"]
        hq = cfg.n_head // world * 64
        if sess is not None:
            out["plan_validated_launches"] = sess.launches
            out["plan_completed_each_step"] = bool(tpm.lane.complete)
        out[name] = {"loss_ref": lr_, "loss_tp": lt_, "q_w_diff": rel(mine, full_q[rank * hq:(rank + 1) * hq]),
                     "embed_diff": rel(m.embed, ref.embed)}
    ok = all(v < 2e-2 for k, v in out.items() if k.startswith(("ag_", "gemm_")))
    for name in ("sharded_kv", "shared_kv"):
        r = out[name]
        ok = ok and all(abs(a - b) < 5e-2 for a, b in zip(r["loss_ref"], r["loss_tp"])) and r["loss_tp"][-1] < r["loss_tp"][0]
        ok = ok and r["q_w_diff"] < 5e-2 and r["embed_diff"] < 5e-2
    ok = ok and out.get("plan_validated_launches", 0) >= 4 * 8 * 2 and out.get("plan_completed_each_step", False)
    ok = ok and out.get("tuned_over_session", False)
    ok = ok and out["tuned_gather"]["picked"] in (4, 8) and out["tuned_gather"]["world"] == world and out["tuned_scatter_picked"] in (4, 8)
    out["ok"] = ok
    if rank == 0:
        print("TP_RESULT " + json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


def mesh2d():
    """dp x tp = 2 x 2 with ONE K/V head (both tensor-parallel ranks hold it): the sharded gradients are summed over the
    K/V pair and then reduced over the data axis, through two mappings of the same buffer.  Compared with the same
    model trained on one GPU on the concatenated batch."""
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rank, world = dist.get_rank(), dist.get_world_size()
    from incin_b200.engine import TrainStep
    from incin_b200.models.llama import Llama, LlamaConfig
    from incin_b200.models.llama_tp import LlamaTP, TPOptimizer, tensor_parallel_plan
    from incin_b200.ops import gemm as G
    from incin_b200.optim import AdamW, make_store
    from incin_b200.parallel.context import DistributedContext
    from incin_b200.parallel.mesh import mesh
    from incin_b200.parallel.session import bind_session
    from incin_b200.parallel.tp import TensorParallel
    tp, dp = 2, world // 2
    spec = mesh(dp=dp, tp=tp)
    d, _, t = spec.coords(rank)
    tp_groups = [dist.new_group([spec.rank_of(dd, 0, tt) for tt in range(tp)]) for dd in range(dp)]
    dp_groups = [dist.new_group([spec.rank_of(dd, 0, tt) for dd in range(dp)]) for tt in range(tp)]
    tp_ranks = [spec.rank_of(d, 0, tt) for tt in range(tp)]
    dp_ranks = [spec.rank_of(dd, 0, t) for dd in range(dp)]
    out = {"world": world}
    for name, use_session in (("session", True), ("torch", False)):
        session = bind_session(DistributedContext.from_env(), spec) if use_session else None
        cfg = LlamaConfig(vocab_size=512, n_layer=2, d_model=256, n_head=4, n_kv_head=1, head_dim=64, d_ffn=512)
        B, T = 4, 128
        tpm = TensorParallel(dev, tp_groups[d], max_rows_per_rank=B * T // tp, max_cols=cfg.d_model, session=session,
                             plan=tensor_parallel_plan(cfg, session.mesh, rank, B * T) if session else None,
                             ranks=tp_ranks if session else None)
        gg = torch.Generator().manual_seed(3)
        tok_all = torch.randint(0, cfg.vocab_size, (dp * B, T), generator=gg).to(dev)
        tgt_all = torch.randint(0, cfg.vocab_size, (dp * B, T), generator=gg).to(dev)
        tok, tgt = tok_all[d * B:(d + 1) * B].contiguous(), tgt_all[d * B:(d + 1) * B].contiguous()
        ref = Llama(cfg, seed=0).to(dev)
        ref_step = TrainStep(ref, AdamW(make_store(ref), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1), use_graph=False)
        m = LlamaTP.from_seed(cfg, tp, t, seed=0).to(dev)
        m.tp = tpm
        opt = TPOptimizer(m, tpm, dev, lr=1e-3, dp_group=dp_groups[t], world_group=None, session=session, dp_ranks=dp_ranks)
        step = TrainStep(m, opt, use_graph=False)
        lr_, lt_ = [], []
        for _ in range(4):
            lr_.append(float(ref_step(tok_all, tgt_all)))
            l = step(tok, tgt).clone()
            dist.all_reduce(l)
            lt_.append(float(l) / dp)
        G.check_status()
        kv_ref = dict(ref.named_parameters())["blocks.1.qkv_w"][cfg.n_head * 64:]
        out[name] = {"loss_ref": lr_, "loss_tp": lt_, "kv_w_diff": rel(dict(m.named_parameters())["blocks.1.kv_w"], kv_ref),
                     "embed_diff": rel(m.embed, ref.embed)}
        del step, opt, m, tpm, ref_step, ref
    ok = True
    for name in ("session", "torch"):
        r = out[name]
        ok = ok and all(abs(a - b) < 5e-2 for a, b in zip(r["loss_ref"], r["loss_tp"])) and r["loss_tp"][-1] < r["loss_tp"][0]
        ok = ok and r["kv_w_diff"] < 5e-2 and r["embed_diff"] < 5e-2
    out["ok"] = ok
    if rank == 0:
        print("TP_RESULT " + json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    mesh2d() if sys.argv[1:] == ["mesh2d"] else main()
