"""Distributed layer without a cluster: fake topology probes, the in-process reference transport, and
real child processes on 127.0.0.1 for the rendezvous (missing peer, wrong run id, peer abort, divergent
plan) — the reference's own strategy (crates/incin/tests/rendezvous.rs, incin-core/tests/mesh_bind.rs)."""
import multiprocessing as mp
import socket

import pytest
import torch

from incin_b200.core import Cuda, DTypeId
from incin_b200.parallel import mesh as M
from incin_b200.parallel import placement as P
from incin_b200.parallel import plan as PL
from incin_b200.parallel import strategies as S
from incin_b200.parallel.planner import HybridPlanner, HybridWorkload, MemoryLimit, PlanObjective
from incin_b200.parallel.transport import ReferenceTransport, TransportError


class FakeMachine:
    def __init__(self, n=8, arch=None, alias=None, link=M.LinkClass.HIGH_BANDWIDTH):
        self.n, self.arch, self.alias, self.lk = n, arch or {}, alias or {}, link

    def identity(self, d):
        if d.index >= self.n:
            return None
        return M.DeviceIdentity(self.alias.get(d.index, f"GPU-{d.index}"), "cuda", self.arch.get(d.index, "sm_100"))

    def link(self, a, b):
        return self.lk


def _mesh(dp=1, tp=1, pp=1, probe=None):
    spec = M.mesh(dp, tp, pp)
    return M.DeviceMesh.bind(spec, [Cuda(i) for i in range(spec.world)], probe or FakeMachine())


def test_rank_formula_and_groups():
    spec = M.mesh(dp=2, tp=2, pp=2)
    for r in range(8):
        d, p, t = spec.coords(r)
        assert spec.rank_of(d, p, t) == r == d * 4 + p * 2 + t
    m = _mesh(2, 2, 2)
    assert m.group_of(5, M.Axis.TENSOR).ranks == (4, 5)
    assert m.group_of(5, M.Axis.DATA).ranks == (1, 5)
    assert m.group_of(5, M.Axis.PIPELINE).ranks == (5, 7)


@pytest.mark.parametrize("kind,kwargs,devs", [
    (M.BindErrorKind.RANK_COUNT, {}, [Cuda(0)]),
    (M.BindErrorKind.REPEATED_DEVICE, {}, [Cuda(0), Cuda(0)]),
    (M.BindErrorKind.UNKNOWN_DEVICE, {"n": 1}, [Cuda(0), Cuda(1)]),
    (M.BindErrorKind.ALIASED_DEVICE, {"alias": {1: "GPU-0"}}, [Cuda(0), Cuda(1)]),
    (M.BindErrorKind.MIXED_ARCHITECTURE, {"arch": {1: "sm_90"}}, [Cuda(0), Cuda(1)]),
    (M.BindErrorKind.UNREACHABLE_PEER, {"link": M.LinkClass.UNREACHABLE}, [Cuda(0), Cuda(1)]),
])
def test_bind_guards(kind, kwargs, devs):
    with pytest.raises(M.BindError) as e:
        M.DeviceMesh.bind(M.mesh(dp=2), devs, FakeMachine(**kwargs))
    assert e.value.kind is kind


def test_bind_minimum_link_and_stable_ids():
    with pytest.raises(M.BindError) as e:
        M.DeviceMesh.bind(M.mesh(tp=2), [Cuda(0), Cuda(1)], FakeMachine(link=M.LinkClass.HOST_BOUNCE),
                          minimum_link=M.LinkClass.HIGH_BANDWIDTH)
    assert e.value.kind is M.BindErrorKind.INSUFFICIENT_LINK
    assert _mesh(2, 4).mesh_id == _mesh(2, 4).mesh_id != _mesh(4, 2).mesh_id
    assert M.Digest().bytes(b"hello").finish() == 0xA430D84680AABD0B  # FNV-1a 64 test vector


def test_transition_table():
    T = P.PlacementTransition
    assert P.validate_transition(P.Replicated(), P.Sharded(0)) is T.LOCAL_SHARD
    assert P.validate_transition(P.Sharded(1), P.Replicated()) is T.ALL_GATHER
    assert P.validate_transition(P.Partial(), P.Replicated()) is T.ALL_REDUCE
    assert P.validate_transition(P.Partial(), P.Sharded(0)) is T.REDUCE_SCATTER
    assert P.validate_transition(P.Local, P.Local) is T.IDENTITY
    for bad in ((P.Local, P.Replicated()), (P.Replicated(), P.Partial()), (P.Sharded(0), P.Partial()),
                (P.Sharded(0), P.Sharded(1))):
        with pytest.raises(P.PlacementError):
            P.validate_transition(*bad)
    assert P.validate_shard((16, 2048, 5632), P.Sharded(2), M.mesh(tp=8)) == (16, 2048, 704)
    with pytest.raises(P.PlacementError):
        P.validate_shard((16, 2048, 5633), P.Sharded(2), M.mesh(tp=8))
    assert P.matmul_placement(P.Replicated(), P.Sharded(1)).kind is P.PlacementKind.SHARDED
    assert P.matmul_placement(P.Sharded(1), P.Sharded(0)).kind is P.PlacementKind.PARTIAL
    assert P.reduce_sharded_axis(P.Sharded(1), 1, P.Reduction.SUM).kind is P.PlacementKind.PARTIAL


def test_plan_hash_is_order_and_content_sensitive():
    m = _mesh(dp=2)
    def build(sizes):
        b = S.DataParallelPlanBuilder(m)
        for i, n in enumerate(sizes):
            b.push(i, n)
        return b.finish()
    a, b, c = build([100, 200]), build([100, 200]), build([200, 100])
    assert a.hash == b.hash != c.hash
    assert a.descriptors[1].depends_on == 0 and a.summary().collectives == 2
    agreed = PL.preflight(2, [(a.mesh_id, a.hash, 2)] * 2, a)
    cur = PL.PlanCursor(agreed)
    cur.next(tag=0, kind=PL.CollectiveKind.all_reduce(P.Reduction.MEAN), elements=100, dtype=DTypeId.F32)
    with pytest.raises(PL.PlanError):
        cur.next(tag=1, kind=PL.CollectiveKind.all_reduce(P.Reduction.MEAN), elements=999, dtype=DTypeId.F32)
    with pytest.raises(PL.PreflightError):
        PL.preflight(2, [(a.mesh_id, a.hash, 2), (c.mesh_id, c.hash, 2)], a)
    bld = PL.CollectivePlanBuilder(m)
    with pytest.raises(PL.PlanError):  # all-gather cannot realise Partial -> Replicated
        bld.push(0, M.Axis.DATA, PL.CollectiveKind.all_gather(), 10, DTypeId.F32, P.Partial(mesh_axis=M.Axis.DATA),
                 P.Replicated())
    assert PL.CollectiveKind.all_gather().adjoint().op is PL.CollectiveOp.REDUCE_SCATTER
    assert PL.CollectiveKind.send_recv(0, 1).adjoint() == PL.CollectiveKind.send_recv(1, 0)


def test_tp_and_pp_builders():
    m = _mesh(dp=1, tp=4, pp=2)
    tp = S.TensorParallelPlanBuilder(m)
    tp.push_column(3, (16, 2048, 5632), 2)
    tp.push_row(4, (16, 2048, 2048))
    tp.push_row_scatter(5, (16, 2048, 2048), 1)
    plan = tp.finish()
    assert [d.tag for d in plan.descriptors] == [(3 << 2) | 0, (4 << 2) | 1, (5 << 2) | 3]
    assert plan.descriptors[0].output_elements == 16 * 2048 * 5632
    assert plan.descriptors[2].output_elements == 16 * 2048 * 2048 // 4
    pp, tl = S.PipelinePlanBuilder(m).build(S.PipelineSchedule.ONE_F_ONE_B, 4, 1000)
    assert len(pp.descriptors) == 8 and pp.descriptors[0].tag == S.pp_tag(0, 0, S.PipelineTransfer.FORWARD_ACTIVATION)
    assert S.transfer_order(S.PipelineSchedule.GPIPE, 2) == [
        (S.PipelineTransfer.FORWARD_ACTIVATION, 0), (S.PipelineTransfer.FORWARD_ACTIVATION, 1),
        (S.PipelineTransfer.BACKWARD_GRADIENT, 1), (S.PipelineTransfer.BACKWARD_GRADIENT, 0)]
    g = S.build_timeline(S.PipelineSchedule.GPIPE, 4, 8)
    f = S.build_timeline(S.PipelineSchedule.ONE_F_ONE_B, 4, 8)
    assert max(f.peak_live_activations) == 4 < max(g.peak_live_activations) == 8
    assert f.bubble_slots == g.bubble_slots == 24


def test_hybrid_planner():
    wl = HybridWorkload(batch_size=16, seq_len=2048, parameter_elements=1_100_000_000, layers=22, hidden=2048,
                        flops_per_token=6 * 1.1e9, tensor_shard_extent=32, microbatches=2)
    pl = HybridPlanner(8)
    assert any(m.dp == 2 and m.tp == 4 for m in pl.candidates())
    best = pl.plan(wl)
    assert best.feasible and best.mesh.world == 8
    small = pl.plan(wl, PlanObjective.MINIMIZE_MEMORY)
    assert small.memory_bytes <= best.memory_bytes
    with pytest.raises(ValueError):
        pl.plan(wl, limit=MemoryLimit(1 << 20))
    front = pl.frontier(wl)
    assert all(e.feasible for e in front) and len(front) >= 1


# ------------------------------------------------------------------------------------------ reference transport
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.int64])
def test_reference_transport_matches_single_device_math(dtype):
    w, n = 4, 24
    tr = ReferenceTransport(w)
    g = torch.Generator().manual_seed(0)
    bufs = [(torch.randn(n, generator=g) * 4).to(dtype) for _ in range(w)]
    stacked = torch.stack([b.double() for b in bufs])
    out = tr.all_reduce(bufs, P.Reduction.SUM)
    ref = stacked.sum(0)
    assert all(torch.allclose(o.double(), ref, rtol=2e-2, atol=1e-1) for o in out)
    assert torch.equal(out[0], out[3])
    ag = tr.all_gather(bufs)
    assert torch.equal(ag[2], torch.cat(bufs))
    rs = tr.reduce_scatter(bufs, P.Reduction.MAX)
    assert torch.allclose(rs[1].double(), stacked.max(0).values[6:12])
    a2a = tr.all_to_all(bufs)
    assert torch.equal(a2a[1].view(w, -1)[3], bufs[3].view(w, -1)[1])
    sr = tr.send_recv(bufs, 0, 2)
    assert torch.equal(sr[2], bufs[0]) and torch.equal(sr[1], bufs[1])


def test_reference_transport_checks():
    tr = ReferenceTransport(2)
    big = torch.tensor([2 ** 62], dtype=torch.int64)
    with pytest.raises(TransportError, match="overflow"):
        tr.all_reduce([big, big], P.Reduction.SUM)
    with pytest.raises(TransportError):
        tr.all_reduce([torch.zeros(3)], P.Reduction.SUM)
    with pytest.raises(TransportError):
        tr.reduce_scatter([torch.zeros(3), torch.zeros(3)])
    mean = tr.all_reduce([torch.tensor([1.0, 3.0]), torch.tensor([3.0, 5.0])], P.Reduction.MEAN)
    assert mean[0].tolist() == [2.0, 4.0]


# ------------------------------------------------------------------------------------------ rendezvous (child processes)
def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, run_id, scenario, q):
    from incin_b200.parallel.context import ContextFailure, DistributedContext, RendezvousConfig, RendezvousError
    try:
        ctx = DistributedContext.rendezvous(RendezvousConfig(rank, world, f"127.0.0.1:{port}", run_id, rank, 4000))
    except RendezvousError as e:
        q.put((rank, "connect_failed", e.failure.name))
        return
    try:
        if scenario == "ok":
            blobs = ctx.allgather_bytes(bytes([rank]) * 8)
            ctx.shutdown(4000)
            q.put((rank, "ok", [b[0] for b in blobs], ctx.state.name))
        elif scenario == "abort":
            if rank == 1:
                ctx.abort(ContextFailure.DEVICE_TIMEOUT)   # e.g. a bounded device wait gave up on this rank
                q.put((rank, "aborted", ctx.state.name))
            else:
                msg = ctx.wait_for_peer(4000)
                q.put((rank, "saw", msg[0] if msg else None, ctx.state.name))
        elif scenario == "plan":
            from incin_b200.core import Cuda
            from incin_b200.parallel import mesh as M, plan as PL, strategies as S
            class Probe:
                def identity(self, d): return M.DeviceIdentity(f"GPU-{d.index}", "cuda", "sm_100")
                def link(self, a, b): return M.LinkClass.HIGH_BANDWIDTH
            m = M.DeviceMesh.bind(M.mesh(dp=world), [Cuda(i) for i in range(world)], Probe())
            b = S.DataParallelPlanBuilder(m, rank)
            b.push(0, 1000 + (rank == 1))    # rank 1 diverges
            try:
                ctx.preflight(b.finish())
                q.put((rank, "agreed"))
            except PL.PreflightError:
                q.put((rank, "rejected", ctx.state.name))
        elif scenario in ("tp_plan", "tp_plan_same"):
            # the tensor-parallel group under the plan contract: rank 1 plans a different model width.  The plan must
            # be rejected before a single peer-mapped buffer is created or opened.
            import incin_b200.parallel.tp as TP
            from incin_b200.core import Cuda
            from incin_b200.models.llama import LlamaConfig
            from incin_b200.models.llama_tp import tensor_parallel_plan
            from incin_b200.parallel import mesh as M, plan as PL
            from incin_b200.parallel.session import CollectiveSession
            class Probe:
                def identity(self, d): return M.DeviceIdentity(f"GPU-{d.index}", "cuda", "sm_100")
                def link(self, a, b): return M.LinkClass.HIGH_BANDWIDTH
            m = M.DeviceMesh.bind(M.mesh(tp=world), [Cuda(i) for i in range(world)], Probe())
            cfg = LlamaConfig.tiny()
            if scenario == "tp_plan" and rank == 1:
                cfg.d_model *= 2
            opened = []
            class RecordingBuffer:                       # stands in for the peer-mapped allocation
                def __init__(self, nbytes, device): opened.append(("alloc", nbytes))
                def exchange(self, *a, **k): opened.append(("exchange",)); return self
            TP.SymmetricBuffer = RecordingBuffer
            session = CollectiveSession(ctx, m)
            try:
                TP.TensorParallel("cpu", None, max_rows_per_rank=128, max_cols=cfg.d_model, session=session,
                                  plan=tensor_parallel_plan(cfg, m, rank, 256), ranks=list(range(world)))
                q.put((rank, "constructed", len(opened)))
            except PL.PreflightError:
                q.put((rank, "rejected", len(opened), ctx.state.name))
            except Exception as e:      # past the preflight the CPU stand-in cannot go on (no device library): expected
                q.put((rank, "agreed_then", type(e).__name__, len(opened) > 0))
        elif scenario in ("nccl_connect", "nccl_connect_diverge"):
            # the library communicator comes up from the context: topology, preflight, then the bootstrap address
            import torch
            import torch.distributed as dist
            from incin_b200.core import Cuda
            from incin_b200.parallel import mesh as M, plan as PL, strategies as S
            from incin_b200.parallel.transport import NcclTransport
            class Probe:
                def identity(self, d): return M.DeviceIdentity(f"GPU-{d.index}", "cuda", "sm_100")
                def link(self, a, b): return M.LinkClass.HIGH_BANDWIDTH
            m = M.DeviceMesh.bind(M.mesh(dp=world), [Cuda(i) for i in range(world)], Probe())
            b = S.DataParallelPlanBuilder(m, rank)
            b.push(0, 8 + (scenario == "nccl_connect_diverge" and rank == 1))
            try:
                tr = NcclTransport.connect_context(ctx, b.finish(), device=torch.device("cpu"))
            except PL.PreflightError:
                q.put((rank, "rejected", dist.is_initialized(), ctx.state.name))
            else:
                t = tr.all_reduce(torch.full((8,), float(rank + 1)), PL.Reduction.MEAN, tag=0)    # the planned gradient mean
                ok_plan = True
                try:
                    tr.all_reduce(torch.zeros(8), PL.Reduction.MEAN, tag=1)     # not in the agreed plan
                    ok_plan = False
                except PL.PlanError:
                    pass
                q.put((rank, "connected", t.tolist()[0], ok_plan, len(tr.topology), ctx.state.name))
                dist.destroy_process_group()
        elif scenario == "vanish":
            if rank == 1:
                import os
                os._exit(0)   # dies without a word: the socket closes
            try:
                ctx.wait_for_peer(4000)
                q.put((rank, "no_error", ctx.state.name))
            except RendezvousError as e:
                q.put((rank, "peer_lost", e.failure.name, ctx.state.name))
    finally:
        ctx.close()


def _run(world, scenario, run_ids=None, skip=()):
    ctxm = mp.get_context("spawn")
    q, port = ctxm.Queue(), _free_port()
    procs = []
    for r in range(world):
        if r in skip:
            continue
        p = ctxm.Process(target=_rank_main, args=(r, world, port, (run_ids or {}).get(r, "run-A"), scenario, q))
        p.start()
        procs.append(p)
    out = {}
    for _ in range(len(procs) - (1 if scenario == "vanish" else 0)):   # the vanishing rank reports nothing
        item = q.get(timeout=60)
        out[item[0]] = item[1:]
    for p in procs:
        p.join(timeout=10)
    return out


def test_rendezvous_allgather_and_shutdown_three_ranks():
    out = _run(3, "ok")
    assert all(out[r] == ("ok", [0, 1, 2], "SHUTDOWN") for r in range(3))


def test_rendezvous_missing_peer_times_out():
    out = _run(2, "ok", skip=(1,))
    assert out[0] == ("connect_failed", "TIMEOUT")


def test_rendezvous_run_id_mismatch_is_rejected():
    out = _run(2, "ok", run_ids={1: "run-B"})
    assert out[1] == ("connect_failed", "RUN_ID_MISMATCH")
    assert out[0][0] == "connect_failed"   # the root never got its peer and gave up at the deadline


def test_peer_abort_fails_the_others():
    out = _run(2, "abort")
    assert out[1] == ("aborted", "FAILED")
    assert out[0] == ("saw", 5, "FAILED")   # kind 5 = Abort


def test_vanished_peer_is_detected_on_the_host():
    out = _run(2, "vanish", skip=())
    assert out[0][0] == "peer_lost" and out[0][-1] == "FAILED"


def test_divergent_plan_rejected_before_any_communicator():
    out = _run(2, "plan")
    assert out[0][0] == "rejected" and out[1][0] == "rejected" and out[0][1] == "FAILED"


def test_divergent_tensor_parallel_plan_is_rejected_before_any_peer_mapping():
    out = _run(2, "tp_plan")
    assert out[0] == ("rejected", 0, "FAILED") and out[1] == ("rejected", 0, "FAILED")     # nothing allocated or opened
    same = _run(2, "tp_plan_same")
    assert all(v[0] in ("constructed", "agreed_then") for v in same.values())              # equal plans pass the preflight


def test_library_communicator_is_bootstrapped_from_the_context():
    out = _run(2, "nccl_connect")
    # mean of (rank + 1) over two ranks; the launch outside the plan is refused and fails the context
    assert out[0] == ("connected", 1.5, True, 2, "FAILED") and out[1] == ("connected", 1.5, True, 2, "FAILED")
    bad = _run(2, "nccl_connect_diverge")
    assert all(v == ("rejected", False, "FAILED") for v in bad.values())      # no communicator was ever created


def test_plan_lane_checks_every_launch_and_placements_pick_the_kernel():
    from incin_b200.core import Cuda
    from incin_b200.models.llama import LlamaConfig
    from incin_b200.models.llama_tp import tensor_parallel_plan
    from incin_b200.parallel import mesh as M, plan as PL
    from incin_b200.parallel.dp import bucket_ranges, reducer_plan
    from incin_b200.parallel.placement import Partial, PlacementError, Reduction, Replicated, Sharded
    from incin_b200.parallel.session import CollectiveSession
    from incin_b200.parallel.strategies import TensorParallelCollective as TC, tp_tag
    from incin_b200.parallel.tp import parallel_linear

    class Probe:
        def identity(self, d): return M.DeviceIdentity(f"GPU-{d.index}", "cuda", "sm_100")
        def link(self, a, b): return M.LinkClass.HIGH_BANDWIDTH
    m = M.DeviceMesh.bind(M.mesh(tp=4), [Cuda(i) for i in range(4)], Probe())
    cfg = LlamaConfig.tiny()
    tokens = 512
    plan = tensor_parallel_plan(cfg, m, 0, tokens)
    assert len(plan.descriptors) == 8 * cfg.n_layer
    lane = CollectiveSession(None, m).agree(plan)                 # single process: agreement is local
    shard, full = tokens // 4 * cfg.d_model, tokens * cfg.d_model
    lane.launch(tag=tp_tag(0, TC.COLUMN_OUTPUT_GATHER), kind=PL.CollectiveKind.all_gather(), elements=shard)
    lane.launch(tag=tp_tag(2, TC.ROW_OUTPUT_SCATTER), kind=PL.CollectiveKind.reduce_scatter(Reduction.SUM), elements=full)
    with pytest.raises(PL.PlanError):                              # out of order: the gate/up gather comes next
        lane.launch(tag=tp_tag(6, TC.ROW_OUTPUT_SCATTER), kind=PL.CollectiveKind.reduce_scatter(Reduction.SUM), elements=full)
    lane.begin_step()
    with pytest.raises(PL.PlanError):                              # right tag, wrong element count
        lane.launch(tag=tp_tag(0, TC.COLUMN_OUTPUT_GATHER), kind=PL.CollectiveKind.all_gather(), elements=shard + 1)
    # the backward half is the adjoint sequence in reverse layer order
    back = plan.descriptors[4 * cfg.n_layer]
    assert back.tag == tp_tag(2 * (4 * (cfg.n_layer - 1) + 3) + 1, TC.COLUMN_OUTPUT_GATHER)
    # data-parallel reducer plan: one chained all-reduce(mean) per bucket
    entries = [("a", None, 0, 100), ("b", None, 128, 300), ("c", None, 448, 64)]
    assert bucket_ranges(entries, 512, 0) == [(0, 512)] and bucket_ranges(entries, 512, 120) == [(0, 128), (128, 448), (448, 512)]
    dpm = M.DeviceMesh.bind(M.mesh(dp=4), [Cuda(i) for i in range(4)], Probe())
    rp = reducer_plan(dpm, 0, [(0, 128), (128, 448)])
    assert [d.input_elements for d in rp.descriptors] == [128, 320] and rp.descriptors[1].depends_on == 0
    # placements decide the kernel; illegal transitions are refused with the reason, before any tensor is touched
    with pytest.raises(PlacementError):
        parallel_linear(None, None, (None,), src=Replicated(), dst=Partial(Reduction.SUM))
    with pytest.raises(PlacementError):
        parallel_linear(None, None, (None,), src=Sharded(1), dst=Replicated())          # only token rows are gathered
    with pytest.raises(PlacementError):
        parallel_linear(None, None, (None, None), src=Partial(Reduction.SUM), dst=Sharded(0))


def test_copy_cta_heuristic_balances_copy_link_and_gemm():
    """The number of copy CTAs of a fused launch: enough of them to keep up with the link when the GEMM is light, fewer
    when the GEMM needs the SMs, fewer for the pushing reduce-scatter than for the pulling all-gather, and the explicit
    settings win over the model."""
    import incin_b200.parallel.tp as TP
    pick = TP.TensorParallel._copy_ctas
    class Stub:
        copy_ctas = 0
        COPY_CTA_GBS, COPY_CTA_GBS_PUSH = TP.TensorParallel.COPY_CTA_GBS, TP.TensorParallel.COPY_CTA_GBS_PUSH
        LINK_GBS, GEMM_TFLOPS = TP.TensorParallel.LINK_GBS, TP.TensorParallel.GEMM_TFLOPS
    s = Stub()
    link = 112e6                                        # tp = 8, 32768 tokens, hidden 2048: bytes in per GPU
    light, heavy = 2.0 * 32768 * 384 * 2048, 2.0 * 32768 * 1408 * 2048 * 4
    c_light, c_heavy = pick(s, link, link, light), pick(s, link, link, heavy)
    assert 24 <= c_light <= 48 and c_heavy < c_light and c_heavy >= 4
    assert pick(s, link, link, light, push=True) < c_light
    assert pick(s, link / 8, link / 8, light) <= c_light          # fewer bytes never ask for more copy CTAs
    s.copy_ctas = 12
    assert pick(s, link, link, light) == 12
    s.copy_ctas = 0
    import os
    old = os.environ.get("INCIN_TP_COPY")
    os.environ["INCIN_TP_COPY"] = "warps"
    try:
        assert pick(s, link, link, light) < 0                      # copy warps: minus the ring's operand stages
    finally:
        if old is None:
            del os.environ["INCIN_TP_COPY"]
        else:
            os.environ["INCIN_TP_COPY"] = old


def test_cuda_topology_probe_reads_link_classes_from_nvml(monkeypatch):
    """NVLink-connected pairs are HIGH_BANDWIDTH, PCIe-only peers PEER_CAPABLE, no peer access HOST_BOUNCE; NVML is only
    queried (a stand-in module plays it here) and its absence falls back to peer access alone."""
    import types
    from incin_b200.core import Cuda
    from incin_b200.parallel import mesh as M
    calls = []
    fake = types.SimpleNamespace(NVML_P2P_CAPS_INDEX_NVLINK=2, NVML_P2P_STATUS_OK=0,
                                 nvmlDeviceGetHandleByIndex=lambda i: ("h", i))

    def status(ha, hb, cap):
        calls.append((ha[1], hb[1], cap))
        return 0 if {ha[1], hb[1]} == {0, 1} else 5          # only GPUs 0 and 1 share NVLink
    fake.nvmlDeviceGetP2PStatus = status
    monkeypatch.setattr(torch.cuda, "can_device_access_peer", lambda a, b: (a, b) != (0, 3) and (a, b) != (3, 0))
    probe = M.CudaTopologyProbe(nvml=fake)
    assert probe.link(Cuda(0), Cuda(0)) is M.LinkClass.SAME_DEVICE
    assert probe.link(Cuda(0), Cuda(1)) is M.LinkClass.HIGH_BANDWIDTH
    assert probe.link(Cuda(0), Cuda(2)) is M.LinkClass.PEER_CAPABLE
    assert probe.link(Cuda(0), Cuda(3)) is M.LinkClass.HOST_BOUNCE
    assert all(cap == 2 for _, _, cap in calls) and (0, 3, 2) not in calls        # no NVML query without peer access
    broken = types.SimpleNamespace(nvmlDeviceGetHandleByIndex=lambda i: (_ for _ in ()).throw(RuntimeError("nvml down")))
    assert M.CudaTopologyProbe(nvml=broken).link(Cuda(0), Cuda(2)) is M.LinkClass.HIGH_BANDWIDTH   # NVML cannot say
