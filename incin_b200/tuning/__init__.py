"""Autotuning: candidate generation, device-timed measurement, single-flight permits, an in-memory LRU and a
persistent checksummed cache keyed by stable hardware/software identities, and the policy service that decides
when tuning may run.

Counterpart of crates/incin-backends/src/tuning.rs (:35-475: candidates, 2 warm-ups + 7 CUDA-event samples,
``TuningPermit``), tuning/cache.rs (bounded, checksummed, file-locked), tuning/identity.rs (GPU UUID, sm_XY,
driver, NVRTC version and options), tuning/service.rs (Disabled / Heuristic / CoordinatedWarmup /
ProfileGuided), tuning/signature.rs (pruning) and tuning/telemetry.rs (explain records).
"""
from __future__ import annotations

import collections
import enum
import fcntl
import hashlib
import json
import os
import statistics
import threading
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Callable, Sequence

LRU_BOUND = 1024
DISK_BOUND = 4096
WARMUPS, SAMPLES = 2, 7


class TuningPolicy(enum.Enum):
    DISABLED = "disabled"                  # always the heuristic, never measure, never read the cache
    HEURISTIC = "heuristic"                # cached result if present, else the heuristic; never measure
    COORDINATED_WARMUP = "coordinated_warmup"  # measure during warm-up steps only, one tuner per key
    PROFILE_GUIDED = "profile_guided"      # measure whenever a key is missing


@dataclass(frozen=True)
class Identity:
    """Everything that invalidates a measurement when it changes."""
    gpu_uuid: str
    arch: str
    driver: str
    compiler: str
    options: str = ""

    def token(self) -> str:
        return hashlib.sha256("|".join((self.gpu_uuid, self.arch, self.driver, self.compiler, self.options)).encode()).hexdigest()[:24]

    @staticmethod
    def current() -> "Identity":
        try:
            import torch
            if torch.cuda.is_available():
                p = torch.cuda.get_device_properties(torch.cuda.current_device())
                return Identity(str(getattr(p, "uuid", "gpu")), f"sm_{p.major}{p.minor}",
                                str(torch.version.cuda), "nvcc-12.9/nvrtc", "-O3 --use_fast_math sm_100a")
        except Exception:
            pass
        return Identity("no-gpu", "cpu", "none", "none")


@dataclass(frozen=True)
class Candidate:
    name: str
    params: tuple    # hashable (key, value) pairs

    def as_dict(self) -> dict:
        return dict(self.params)


def candidates(**grid) -> list[Candidate]:
    """Cartesian product of parameter lists, e.g. ``candidates(block=[128,256,512], vec=[1,2,4])``."""
    out = [()]
    for k, vals in grid.items():
        out = [c + ((k, v),) for c in out for v in vals]
    return [Candidate(",".join(f"{k}={v}" for k, v in c), c) for c in out]


def prune(cands: Sequence[Candidate], signature: dict, rules: Sequence[Callable[[dict, dict], bool]]) -> list[Candidate]:
    """Signature pruning: drop candidates a rule proves pointless for this problem signature before timing them."""
    return [c for c in cands if all(r(c.as_dict(), signature) for r in rules)]


def time_cuda(fn: Callable[[], None], warmups: int = WARMUPS, samples: int = SAMPLES) -> float:
    """Median milliseconds of ``fn`` measured with CUDA events on the current stream."""
    import torch
    for _ in range(warmups):
        fn()
    ts = []
    for _ in range(samples):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


@dataclass
class TuningRecord:
    key: str
    identity: str
    best: dict
    best_ms: float
    tried: list = field(default_factory=list)     # [(candidate name, ms)] — the "explain" evidence
    source: str = "measured"


def _checksum(payload: str) -> str:
    return hashlib.sha256(payload.encode()).hexdigest()[:16]


class PersistentCache:
    """One JSON-lines file, each line ``{"sum": checksum, "rec": record}``; corrupt lines are skipped, the file is
    rewritten under an exclusive lock, and only the newest ``DISK_BOUND`` records are kept."""

    def __init__(self, path=None):
        base = Path(os.environ.get("INCIN_AUTOTUNE_CACHE_DIR", os.path.expanduser("~/.cache/incin/autotune")))
        base.mkdir(parents=True, exist_ok=True)
        self.path = Path(path) if path else base / "tuning.jsonl"

    def load(self) -> dict[str, TuningRecord]:
        out: dict[str, TuningRecord] = {}
        if not self.path.exists():
            return out
        for line in self.path.read_text().splitlines():
            try:
                d = json.loads(line)
                body = json.dumps(d["rec"], sort_keys=True)
                if _checksum(body) != d["sum"]:
                    continue
                r = TuningRecord(**d["rec"])
                out[r.identity + "/" + r.key] = r
            except Exception:
                continue
        return out

    def store(self, rec: TuningRecord) -> None:
        with open(str(self.path) + ".lock", "w") as lk:
            fcntl.flock(lk, fcntl.LOCK_EX)
            recs = self.load()
            recs[rec.identity + "/" + rec.key] = rec
            keep = list(recs.values())[-DISK_BOUND:]
            tmp = self.path.with_suffix(f".tmp{os.getpid()}")
            with open(tmp, "w") as f:
                for r in keep:
                    body = json.dumps(asdict(r), sort_keys=True)
                    f.write(json.dumps({"sum": _checksum(body), "rec": json.loads(body)}) + "\n")
            os.replace(tmp, self.path)
            fcntl.flock(lk, fcntl.LOCK_UN)


class TuningPermit:
    """Single flight: the first caller for a key tunes, concurrent callers wait for its result."""

    def __init__(self):
        self._lock = threading.Lock()
        self._inflight: dict[str, threading.Event] = {}

    def acquire(self, key: str) -> tuple[bool, threading.Event]:
        with self._lock:
            ev = self._inflight.get(key)
            if ev is None:
                ev = threading.Event()
                self._inflight[key] = ev
                return True, ev
            return False, ev

    def release(self, key: str) -> None:
        with self._lock:
            ev = self._inflight.pop(key, None)
        if ev:
            ev.set()


class TuningService:
    def __init__(self, policy: TuningPolicy = TuningPolicy.HEURISTIC, cache: PersistentCache | None = None,
                 identity: Identity | None = None):
        self.policy, self.disk = policy, cache
        self.identity = identity or Identity.current()
        self.lru: "collections.OrderedDict[str, TuningRecord]" = collections.OrderedDict()
        self.permit = TuningPermit()
        self.warmup = True
        self.log: list[TuningRecord] = []
        self._disk_loaded = False

    def end_warmup(self) -> None:
        self.warmup = False

    def _remember(self, rec: TuningRecord) -> None:
        self.lru[rec.key] = rec
        self.lru.move_to_end(rec.key)
        while len(self.lru) > LRU_BOUND:
            self.lru.popitem(last=False)

    def lookup(self, key: str) -> TuningRecord | None:
        if key in self.lru:
            self.lru.move_to_end(key)
            return self.lru[key]
        if self.disk is not None and not self._disk_loaded:
            for k, r in self.disk.load().items():
                if r.identity == self.identity.token():
                    self._remember(r)
            self._disk_loaded = True
        return self.lru.get(key)

    def choose(self, key: str, cands: Sequence[Candidate], heuristic: Callable[[], dict],
               measure: Callable[[dict], float] | None = None) -> dict:
        """Parameters to use for ``key``.  ``measure(params) -> ms`` is only called when the policy allows it."""
        if self.policy is TuningPolicy.DISABLED:
            return heuristic()
        rec = self.lookup(key)
        if rec is not None:
            return rec.best
        may_measure = measure is not None and (self.policy is TuningPolicy.PROFILE_GUIDED or
                                                (self.policy is TuningPolicy.COORDINATED_WARMUP and self.warmup))
        if not may_measure or not cands:
            return heuristic()
        leader, ev = self.permit.acquire(key)
        if not leader:
            ev.wait(timeout=60)
            rec = self.lookup(key)
            return rec.best if rec else heuristic()
        try:
            tried = []
            for c in cands:
                try:
                    tried.append((c.name, float(measure(c.as_dict())), c.as_dict()))
                except Exception:
                    continue   # a candidate that cannot launch is simply not chosen
            if not tried:
                return heuristic()
            name, ms, best = min(tried, key=lambda t: t[1])
            rec = TuningRecord(key, self.identity.token(), best, ms, [(n, t) for n, t, _ in tried])
            self._remember(rec)
            self.log.append(rec)
            if self.disk is not None:
                self.disk.store(rec)
            try:
                from .. import telemetry
                telemetry.emit_scalar(f"tune/{key}", ms)
            except Exception:
                pass
            return best
        finally:
            self.permit.release(key)

    def explain(self) -> str:
        return "\n".join(f"{r.key}: {r.best} {r.best_ms:.4f} ms  (tried " + ", ".join(f"{n}={t:.4f}" for n, t in r.tried) + ")"
                         for r in self.log)


_service = TuningService(TuningPolicy(os.environ.get("INCIN_AUTOTUNE", "heuristic")))


def service() -> TuningService:
    return _service


def set_service(s: TuningService) -> None:
    global _service
    _service = s
