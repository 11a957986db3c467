"""End-to-end: GPT-2 (tiny) forward/backward/optimiser on CUDA against the fp32 CPU backend."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu

from _tol import check_close  # noqa: E402


def _setup(impl):
    from incin_b200.models.gpt2 import GPT2, GPT2Config
    from incin_b200.ops import functional as F
    F.set_attention_impl(impl)
    cfg = GPT2Config.tiny()
    cpu = GPT2(cfg, seed=0)
    gpu = copy.deepcopy(cpu).cuda()
    g = torch.Generator().manual_seed(1)
    tok = torch.randint(0, cfg.vocab_size, (4, 128), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (4, 128), generator=g)
    return cfg, cpu, gpu, tok, tgt


@pytest.mark.parametrize("impl", ["composed", "auto"])
def test_loss_and_grads_match_cpu(impl):
    from incin_b200.optim import ParamStore
    cfg, cpu, gpu, tok, tgt = _setup(impl)
    store = ParamStore(gpu.named_parameters())
    loss_c = cpu(tok, tgt)
    loss_c.backward()
    store.zero_grad()
    loss_g = gpu(tok.cuda(), tgt.cuda())
    loss_g.backward()
    assert abs(loss_g.item() - loss_c.item()) < 3e-2
    ref = dict(cpu.named_parameters())
    for name, p, o, k in store.entries:
        g_gpu = p.main_grad.float().cpu()
        g_cpu = ref[name].grad
        denom = g_cpu.abs().max().item() + 1e-6
        assert (g_gpu - g_cpu).abs().max().item() <= 6e-2 * denom + 2e-4, name
        # a whole model in bf16 against fp32: the direction of every parameter gradient must still agree, and no
        # element may be off by more than a tenth of the gradient's RMS plus a tenth of its own size
        check_close(g_gpu, g_cpu, rtol=1e-1, atol_rms=1e-1, min_cos=0.995, what=f"grad {name}")


@pytest.mark.parametrize("use_graph", [False, True])
def test_training_reduces_loss(use_graph):
    from incin_b200.engine import TrainStep
    from incin_b200.ops import gemm as G
    from incin_b200.optim import AdamW, ParamStore
    cfg, cpu, gpu, tok, tgt = _setup("auto")
    opt = AdamW(ParamStore(gpu.named_parameters()), lr=1e-3)
    step = TrainStep(gpu, opt, use_graph=use_graph)
    tok, tgt = tok.cuda(), tgt.cuda()
    losses = [step(tok, tgt).item() for _ in range(12)]
    assert losses[-1] < losses[0] - 1.0, losses
    if use_graph:
        assert step.graph is not None, "CUDA graph capture of the training step failed"
    G.check_status()


def test_step_pipeline_matches_sequential_steps():
    """Feeding pinned host batches through StepPipeline (copy stream, lagged loss read) gives the losses of the same
    steps run one by one with device inputs and a blocking read."""
    from incin_b200.engine import StepPipeline, TrainStep
    from incin_b200.optim import AdamW, ParamStore
    cfg, cpu, gpu_a, tok, tgt = _setup("auto")
    gpu_b = copy.deepcopy(gpu_a)
    g = torch.Generator().manual_seed(7)
    batches = [(torch.randint(0, cfg.vocab_size, (4, 128), generator=g).pin_memory(),
                torch.randint(0, cfg.vocab_size, (4, 128), generator=g).pin_memory()) for _ in range(8)]
    step_a = TrainStep(gpu_a, AdamW(ParamStore(gpu_a.named_parameters()), lr=1e-3))
    ref = [step_a(t.cuda(), y.cuda()).item() for t, y in batches]
    step_b = TrainStep(gpu_b, AdamW(ParamStore(gpu_b.named_parameters()), lr=1e-3))
    pipe = StepPipeline(step_b)
    got = []
    for i, (t, y) in enumerate(batches):
        pipe.submit(t, y)
        if i:
            got.append(pipe.pop())
    got += pipe.drain()
    assert pipe.outstanding == 0 and len(got) == len(ref)
    assert max(abs(a - b) for a, b in zip(got, ref)) < 2e-2, (got, ref)
    with pytest.raises(RuntimeError):
        pipe.pop()


def test_steady_state_step_makes_no_device_allocation():
    """After warm-up, neither an eager nor a graph-replayed training step asks the driver for memory: the caching
    allocator's count of device allocations, its reserved bytes and the device's free memory do not move."""
    from incin_b200.engine import TrainStep
    from incin_b200.optim import AdamW, ParamStore
    for use_graph in (False, True):
        cfg, cpu, gpu, tok, tgt = _setup("auto")
        step = TrainStep(gpu, AdamW(ParamStore(gpu.named_parameters()), lr=1e-3), use_graph=use_graph)
        tok, tgt = tok.cuda(), tgt.cuda()
        for _ in range(5):
            step(tok, tgt)
        torch.cuda.synchronize()
        s0 = torch.cuda.memory_stats()
        free0, _ = torch.cuda.mem_get_info()
        for _ in range(6):
            step(tok, tgt)
        torch.cuda.synchronize()
        s1 = torch.cuda.memory_stats()
        free1, _ = torch.cuda.mem_get_info()
        assert s1["num_device_alloc"] == s0["num_device_alloc"], (use_graph, s0["num_device_alloc"], s1["num_device_alloc"])
        assert s1["reserved_bytes.all.current"] == s0["reserved_bytes.all.current"]
        assert free1 == free0, (use_graph, free0, free1)


def test_device_trace_rows_cover_the_eager_step():
    """The per-step trace records one row per native launch call of an eager step; the rows' device times add up to
    the step's own device time (events sit on the launching stream back to back)."""
    from incin_b200 import _native
    from incin_b200.engine import TrainStep
    from incin_b200.optim import AdamW, ParamStore
    from incin_b200.telemetry import trace
    cfg, cpu, gpu, tok, tgt = _setup("auto")
    step = TrainStep(gpu, AdamW(ParamStore(gpu.named_parameters()), lr=1e-3), use_graph=False)
    tok, tgt = tok.cuda(), tgt.cuda()
    for _ in range(3):
        step(tok, tgt)
    trace.enable(nvtx=True, events=True)
    try:
        calls0 = _native.LAUNCH_CALLS
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        trace.begin_step()
        step(tok, tgt)
        e1.record()
        rows = trace.end_step()
        calls = _native.LAUNCH_CALLS - calls0
    finally:
        trace.enable(nvtx=False, events=False)
    assert _native.LAUNCH_HOOK is None
    assert len(rows) == calls and calls > 10
    total = sum(ms for _, ms in rows)
    assert 0 < total <= e0.elapsed_time(e1) * 1.05
    top = trace.summary(rows)
    assert abs(sum(r["share"] for r in top) - 1.0) < 1e-2 and top[0]["ms"] >= top[-1]["ms"]
    assert trace.end_step() == []      # tracing off again: free
