"""Collective tuning contract: candidates, per-rank sample reports, median-of-max scoring and a unanimous commit.

Counterpart of crates/incin-backends/src/dist/tuning.rs (:25-932).  As there, the candidate vocabulary of NCCL
(algorithm Ring/Tree, protocol Simple/LL/LL128, channels) is recorded but NOT forced onto NCCL; what the
contract really tunes here are the knobs of the fused peer-memory kernels: grid size (CTAs), bucket size and
whether the reduction overlaps backward.  Every rank must measure the same candidates; a candidate's score is
the median over samples of the MAX over ranks (a collective is as slow as its slowest rank); the winner is
committed only if every rank votes for the same candidate.
"""
from __future__ import annotations

import enum
import statistics
from dataclasses import dataclass


class CollectiveAlgorithm(enum.Enum):
    RING = "ring"
    TREE = "tree"
    ONE_SHOT_P2P = "one_shot_p2p"      # every rank reads all peers (fused kernels; NVSwitch makes it uniform)
    TWO_SHOT_P2P = "two_shot_p2p"      # reduce-scatter then all-gather through peer memory


class CollectiveProtocol(enum.Enum):
    SIMPLE = "simple"
    LL = "ll"
    LL128 = "ll128"


@dataclass(frozen=True)
class CollectiveCandidate:
    algorithm: CollectiveAlgorithm
    protocol: CollectiveProtocol = CollectiveProtocol.SIMPLE
    channels: int = 32          # CTAs of the fused kernel
    chunk_bytes: int = 64 << 20  # bucket size
    stream_priority: int = 0
    overlap_chunks: int = 1
    workspace_bytes: int = 0

    def token(self) -> str:
        return f"{self.algorithm.value}/{self.protocol.value}/c{self.channels}/b{self.chunk_bytes}/o{self.overlap_chunks}"


@dataclass(frozen=True)
class SampleReport:
    rank: int
    candidate: str
    samples_ns: tuple[int, ...]


class TuningDisagreement(RuntimeError):
    pass


def score(reports: list[SampleReport]) -> dict[str, float]:
    """candidate -> median over sample index of the max over ranks."""
    by: dict[str, list[SampleReport]] = {}
    for r in reports:
        by.setdefault(r.candidate, []).append(r)
    out = {}
    for cand, rs in by.items():
        n = min(len(r.samples_ns) for r in rs)
        if n == 0:
            continue
        out[cand] = statistics.median(max(r.samples_ns[i] for r in rs) for i in range(n))
    return out


@dataclass(frozen=True)
class CommitVote:
    rank: int
    candidate: str


@dataclass(frozen=True)
class CommittedCollectiveTuning:
    candidate: str
    score_ns: float
    world: int


def commit(world: int, reports: list[SampleReport], votes: list[CommitVote]) -> CommittedCollectiveTuning:
    ranks = {r.rank for r in reports}
    if ranks != set(range(world)):
        raise TuningDisagreement(f"sample reports from ranks {sorted(ranks)}, expected 0..{world - 1}")
    sc = score(reports)
    if not sc:
        raise TuningDisagreement("no candidate has samples from every rank")
    if len(votes) != world or {v.rank for v in votes} != set(range(world)):
        raise TuningDisagreement("one vote per rank is required")
    chosen = {v.candidate for v in votes}
    if len(chosen) != 1:
        raise TuningDisagreement(f"ranks voted for different candidates: {sorted(chosen)}")
    cand = chosen.pop()
    if cand not in sc:
        raise TuningDisagreement(f"voted candidate {cand} was not measured by every rank")
    return CommittedCollectiveTuning(cand, sc[cand], world)


def local_vote(rank: int, reports: list[SampleReport]) -> CommitVote:
    sc = score(reports)
    return CommitVote(rank, min(sc, key=sc.get))
