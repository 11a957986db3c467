"""Native host runtime (csrc/runtime: digest, batch loader, telemetry sink) against its Python counterparts."""
import json
import random

import pytest
import torch


def test_native_digest_equals_the_python_digest():
    from incin_b200.parallel.mesh import Digest
    from incin_b200.runtime import NativeDigest, fnv1a64
    rng = random.Random(5)
    assert fnv1a64(b"") == Digest().finish() == 0xCBF29CE484222325
    assert fnv1a64(b"a") == 0xAF63DC4C8601EC8C                       # published FNV-1a 64 test vector
    for _ in range(50):
        a, b = Digest(), NativeDigest()
        for _ in range(rng.randint(1, 12)):
            kind = rng.choice("bntf")
            if kind == "b":
                blob = bytes(rng.randrange(256) for _ in range(rng.randint(0, 40)))
                a.bytes(blob), b.bytes(blob)
            elif kind == "n":
                v = rng.choice([0, 1, (1 << 64) - 1, rng.getrandbits(64), -1])
                a.number(v), b.number(v)
            elif kind == "t":
                t = "".join(rng.choice("abcxyz/.é") for _ in range(rng.randint(0, 16)))
                a.text(t), b.text(t)
            else:
                blob = bytes(rng.randrange(256) for _ in range(rng.randint(0, 9)))
                a.field(blob), b.field(blob)
        assert a.finish() == b.finish()


def _reference_order(n, seed, epoch):
    """The permutation the native loader documents: Fisher-Yates driven by splitmix64 of seed + epoch."""
    mask = (1 << 64) - 1
    state = (seed + epoch) & mask
    order = list(range(n))

    def nxt():
        nonlocal state
        state = (state + 0x9E3779B97F4A7C15) & mask
        z = state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        return z ^ (z >> 31)
    for i in range(n - 1, 0, -1):
        j = nxt() % (i + 1)
        order[i], order[j] = order[j], order[i]
    return order


@pytest.mark.parametrize("workers", [1, 3, 8])
def test_native_loader_order_is_seeded_and_independent_of_workers(workers):
    from incin_b200.runtime import NativeBatchLoader
    n = 103
    x = torch.arange(n * 6, dtype=torch.float32).reshape(n, 2, 3)
    y = torch.arange(n, dtype=torch.int64)
    ld = NativeBatchLoader(x, y, batch_size=16, shuffle=True, seed=11, workers=workers, prefetch=2)
    assert len(ld) == 7
    for epoch in range(2):
        batches = list(ld)
        got = torch.cat([b[1] for b in batches]).tolist()
        assert got == _reference_order(n, 11, epoch) == ld.order()
        assert [b[0].shape[0] for b in batches] == [16] * 6 + [7]
        for xb, yb in batches:                      # rows of the two arrays stay aligned
            assert torch.equal(xb, x[yb])
    ld.close()
    plain = NativeBatchLoader(x, batch_size=25, drop_last=True, workers=workers)
    rows = torch.cat(list(plain))
    assert len(plain) == 4 and torch.equal(rows, x[:100])
    plain.close()
    with pytest.raises(ValueError):
        NativeBatchLoader(x, y[:5], batch_size=4)


def test_native_loader_abandoned_epoch_and_restart():
    from incin_b200.runtime import NativeBatchLoader
    x = torch.arange(64, dtype=torch.int32).reshape(64, 1)
    ld = NativeBatchLoader(x, batch_size=4, workers=4, prefetch=1)
    it = iter(ld)
    first = next(it).clone()
    assert first.flatten().tolist() == [0, 1, 2, 3]
    del it                                           # workers are parked on a full ring; the next epoch restarts them
    assert torch.equal(torch.cat(list(ld)), x)
    ld.close()


def test_native_telemetry_sink_writes_schema_lines_and_counts_drops(tmp_path):
    from incin_b200.runtime import NativeTelemetrySink
    from incin_b200.telemetry import Event
    path = tmp_path / "run.jsonl"
    sink = NativeTelemetrySink(path, capacity=1024)
    for step in range(200):
        assert sink.scalar('loss "train"', 1.0 / (step + 1), step)
    assert sink.memory(0, 123, 456, 7)
    sink.send(Event("epoch", payload={"steps": 200}).to_json())
    assert sink.scalar("nan", float("nan"), 1)
    assert sink.flush() == 0
    lines = path.read_text().splitlines()
    assert len(lines) == 203
    evs = [Event.from_json(ln) for ln in lines]
    assert evs[0].kind == "scalar" and evs[0].name == 'loss "train"' and evs[0].value == 1.0 and evs[0].step == 0
    assert abs(evs[199].value - 1.0 / 200) < 1e-12 and evs[0].ts > 1.6e9
    mem = json.loads(lines[200])
    assert mem["kind"] == "memory" and mem["allocated"] == 123 and mem["reserved"] == 456
    assert evs[201].kind == "epoch" and evs[201].payload == {"steps": 200}
    assert json.loads(lines[202])["value"] is None          # non-finite values become null
    assert sink.close() == 0
    # a tiny queue drops the newest events instead of blocking, and says so when the file is closed
    tight = NativeTelemetrySink(tmp_path / "tight.jsonl", capacity=2)
    results = [tight.scalar("x", float(i), i) for i in range(20000)]
    dropped = tight.close()
    assert dropped == results.count(False)
    tail = (tmp_path / "tight.jsonl").read_text().splitlines()
    assert len(tail) == results.count(True) + (1 if dropped else 0)
    if dropped:
        assert json.loads(tail[-1]) == {"v": 1, "kind": "dropped", "count": dropped}


def test_dataloader_native_path_and_emitter_over_the_native_sink(tmp_path):
    from incin_b200 import telemetry
    from incin_b200.data import DataLoader, TensorDataset
    x = torch.arange(40, dtype=torch.float32).reshape(20, 2)
    y = torch.arange(20)
    ld = DataLoader(TensorDataset(x, y), batch_size=6, shuffle=True, seed=3, workers=2, native=True)
    assert ld.native and len(ld) == 4
    e0 = [b for b in ld]
    e1 = [b for b in ld]
    assert sorted(torch.cat([b[1] for b in e0]).tolist()) == list(range(20))
    assert torch.cat([b[1] for b in e0]).tolist() != torch.cat([b[1] for b in e1]).tolist()   # a new permutation per epoch
    assert all(torch.equal(xb, x[yb]) for xb, yb in e0)
    assert torch.cat([b[1] for b in e0]).tolist() == _reference_order(20, 3, 1)   # DataLoader counts epochs from 1
    single = DataLoader(TensorDataset(x), batch_size=8, native=True)
    assert [b[0].shape[0] for b in single] == [8, 8, 4]
    assert not DataLoader(TensorDataset(x, y), batch_size=4).native                  # opt-in
    # the Emitter's queueing on top of the native file sink
    tr = telemetry.native_transport(tmp_path / "e.jsonl")
    em = telemetry.Emitter(tr)
    telemetry.set_emitter(em)
    try:
        for i in range(10):
            telemetry.emit_scalar("loss", float(i), i)
    finally:
        telemetry.set_emitter(None)
        em.close()
    evs = telemetry.read_run(tmp_path / "e.jsonl")
    assert [e.step for e in evs if e.kind == "scalar"] == list(range(10))


def test_native_arena_planner_equals_the_python_planner(monkeypatch):
    """Random lifetimes: the native first fit and the Python loop place every buffer at the same offset; no two
    buffers that are alive together overlap."""
    import incin_b200.graph as G
    from incin_b200.runtime import first_fit_arena
    rng = random.Random(9)
    for _ in range(40):
        n = rng.randint(1, 40)
        sizes = [256 * rng.randint(0, 20) for _ in range(n)]
        first = list(range(n))
        last = [i + rng.randint(0, 12) for i in range(n)]
        skip = [rng.random() < 0.15 for _ in range(n)]
        offs, peak = first_fit_arena(sizes, first, last, skip)
        placed, ref, ref_peak = [], [], 0          # the Python algorithm of plan_memory, on plain lists
        for i in range(n):
            if skip[i]:
                ref.append(-1)
                continue
            busy = sorted((o, s) for o, s, pf, pl in placed if not (pl < first[i] or pf > last[i]))
            off = 0
            for o, s in busy:
                if off + sizes[i] <= o:
                    break
                off = max(off, o + s)
            ref.append(off)
            placed.append((off, sizes[i], first[i], last[i]))
            ref_peak = max(ref_peak, off + sizes[i])
        assert offs == ref and peak == ref_peak
        for i in range(n):
            for j in range(i):
                if skip[i] or skip[j] or last[j] < first[i] or first[j] > last[i] or not sizes[i] or not sizes[j]:
                    continue
                assert offs[i] + sizes[i] <= offs[j] or offs[j] + sizes[j] <= offs[i]
    # plan_memory gives the same plan through either path
    def fn(a, b):
        c = a + b
        d = torch.relu(c)
        e = d * b
        return (e + c).sum()
    g = G.trace(fn, torch.randn(8, 8), torch.randn(8, 8))
    native = G.plan_memory(g)
    monkeypatch.setenv("INCIN_NATIVE_MEMPLAN", "0")
    python = G.plan_memory(g)
    assert native.offsets == python.offsets and native.peak_bytes == python.peak_bytes
    with pytest.raises(ValueError):
        first_fit_arena([1], [0, 1], [0])


def test_threaded_safetensors_load_equals_the_plain_one(tmp_path):
    from incin_b200.io.safetensors import load_safetensors, save_safetensors
    g = torch.Generator().manual_seed(2)
    tensors = {
        "a.weight": torch.randn(300, 257, generator=g),
        "a.bias": torch.randn(257, generator=g).to(torch.bfloat16),
        "ids": torch.randint(0, 1000, (4097,), generator=g),
        "half": torch.randn(3, 5, 7, generator=g).to(torch.float16),
        "mask": torch.randint(0, 2, (33,), generator=g).to(torch.uint8),
        "empty": torch.empty(0, 4),
        "scalar": torch.tensor(3.5),
    }
    path = tmp_path / "m.safetensors"
    save_safetensors(tensors, path, metadata={"step": "7"})
    plain = load_safetensors(path)
    for threads in (1, 4):
        fast = load_safetensors(path, threads=threads)
        assert fast.keys() == plain.keys() == tensors.keys()
        for k in tensors:
            assert fast[k].dtype == tensors[k].dtype and fast[k].shape == tensors[k].shape
            assert torch.equal(fast[k], plain[k]) and torch.equal(fast[k], tensors[k])
    only = load_safetensors(path, names={"ids"}, threads=2)
    assert list(only) == ["ids"] and torch.equal(only["ids"], tensors["ids"])
    # a file that ends before its last tensor does is an error, not a tensor of garbage
    from incin_b200.runtime import read_ranges
    with pytest.raises(OSError):
        read_ranges(path, [(path.stat().st_size - 8, torch.empty(16, dtype=torch.uint8))], 2)
    with pytest.raises(OSError):
        read_ranges(tmp_path / "missing.bin", [(0, torch.empty(4, dtype=torch.uint8))], 1)
