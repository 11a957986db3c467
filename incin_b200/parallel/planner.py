"""Hybrid parallelism planner: analytical memory / communication / step-time model over candidate
(dp, tp, pp) factorizations of the world, Pareto frontier, and objective-driven choice.

Counterpart of ``HybridPlanner`` in crates/incin-core/src/dist/plan.rs:956-2184 (HybridWorkload,
MemoryLimit, PlanObjective {MinimizeStepTime, MinimizeMemory, MinimizeCommunication}, link weights,
Pareto frontier).  The reference chooses ONE of DP/TP/PP for exactly two ranks; this planner also
considers product meshes (e.g. dp=2 x tp=4) because the execution layer here runs them, and its link
model is NVSwitch: every peer at full bandwidth, so collective cost depends on bytes and rank count only.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass

from .mesh import LinkClass, MeshSpec
from .strategies import ActivationCheckpoint, PipelineSchedule, build_timeline


class PlanObjective(enum.Enum):
    MINIMIZE_STEP_TIME = "step_time"
    MINIMIZE_MEMORY = "memory"
    MINIMIZE_COMMUNICATION = "communication"


@dataclass(frozen=True)
class HybridWorkload:
    batch_size: int                       # global batch (sequences)
    seq_len: int
    parameter_elements: int
    layers: int
    hidden: int                           # d_model: activation width moved by TP / PP collectives
    flops_per_token: float                # training FLOPs per token (fwd + bwd)
    tensor_shard_extent: int              # extent TP shards (heads / FFN width): must divide by tp
    microbatches: int = 1
    optimizer_state_copies: int = 2       # Adam: m and v
    activation_bytes_per_token_layer: int = 34 * 2  # ~34 * hidden bf16 values per token per layer, / hidden
    device_capacity_bytes: int = 180 * (1 << 30)


@dataclass(frozen=True)
class MemoryLimit:
    bytes_per_device: int


@dataclass(frozen=True)
class PlanEstimate:
    mesh: MeshSpec
    memory_bytes: int
    comm_bytes: int            # bytes each rank moves over NVLink per step
    step_seconds: float
    bubble_fraction: float
    feasible: bool
    reason: str = ""

    def explain(self) -> str:
        return (f"dp={self.mesh.dp} tp={self.mesh.tp} pp={self.mesh.pp}: {self.memory_bytes / 2**30:.1f} GiB/device, "
                f"{self.comm_bytes / 2**20:.1f} MiB comm/step, {self.step_seconds * 1e3:.2f} ms/step"
                + ("" if self.feasible else f" [infeasible: {self.reason}]"))


class HybridPlanner:
    def __init__(self, world: int, link: LinkClass = LinkClass.HIGH_BANDWIDTH, *, tflops: float = 1400.0,
                 link_gbs: float = 770.0):
        self.world, self.link = world, link
        self.flops = tflops * 1e12
        # a slower link class scales effective bandwidth by the planner weights (HB=2 is the reference point)
        self.bw = link_gbs * 1e9 * LinkClass.HIGH_BANDWIDTH.weight / link.weight

    def candidates(self) -> list[MeshSpec]:
        out = []
        w = self.world
        for dp in range(1, w + 1):
            if w % dp:
                continue
            rest = w // dp
            for tp in range(1, rest + 1):
                if rest % tp:
                    continue
                out.append(MeshSpec(dp, tp, rest // tp))
        return out

    def estimate(self, m: MeshSpec, wl: HybridWorkload, limit: MemoryLimit | None = None,
                 schedule: PipelineSchedule = PipelineSchedule.ONE_F_ONE_B) -> PlanEstimate:
        cap = (limit.bytes_per_device if limit else wl.device_capacity_bytes)
        reason = ""
        if wl.tensor_shard_extent % m.tp:
            reason = f"tp={m.tp} does not divide the sharded extent {wl.tensor_shard_extent}"
        elif wl.batch_size % (m.dp * wl.microbatches if m.pp > 1 else m.dp):
            reason = f"batch {wl.batch_size} does not split over dp={m.dp}" + (f" x {wl.microbatches} microbatches" if m.pp > 1 else "")
        elif wl.layers % m.pp:
            reason = f"pp={m.pp} does not divide {wl.layers} layers"
        params_local = wl.parameter_elements // (m.tp * m.pp)
        # bf16 shadow + fp32 grads + (fp32 master + optimizer copies) sharded over dp by the fused reducer
        state = params_local * (2 + 4) + params_local * 4 * (1 + wl.optimizer_state_copies) // m.dp
        tokens_local = wl.batch_size * wl.seq_len // m.dp
        mb = wl.microbatches if m.pp > 1 else 1
        tl = build_timeline(schedule, m.pp, mb) if m.pp > 1 else None
        live_mb = max(tl.peak_live_activations) if tl else 1
        act = (tokens_local // mb) * live_mb * (wl.layers // m.pp) * wl.activation_bytes_per_token_layer * wl.hidden // m.tp
        memory = state + act
        # communication per rank per step
        comm = 0.0
        if m.dp > 1:
            comm += 2.0 * (m.dp - 1) / m.dp * params_local * 4          # reduce-scatter fp32 grads + all-gather (bf16 ~ half)
        if m.tp > 1:
            per_layer = 4 * tokens_local * wl.hidden * 2                # AG + RS forward, and again backward
            comm += per_layer * (wl.layers // m.pp) * (m.tp - 1) / m.tp
        if m.pp > 1:
            comm += 2 * tokens_local * wl.hidden * 2                    # activation forward + gradient backward
        compute = wl.flops_per_token * wl.batch_size * wl.seq_len / self.world / self.flops
        bubble = tl.bubble_fraction if tl else 0.0
        step = compute / max(1e-9, (1.0 - bubble)) + comm / self.bw * (0.35 if m.tp == 1 else 0.6)  # part overlaps
        feasible = not reason and memory <= cap
        if not reason and memory > cap:
            reason = f"{memory / 2**30:.1f} GiB exceeds {cap / 2**30:.1f} GiB"
        return PlanEstimate(m, int(memory), int(comm), step, bubble, feasible, reason)

    def frontier(self, wl: HybridWorkload, limit: MemoryLimit | None = None) -> list[PlanEstimate]:
        ests = [e for e in (self.estimate(m, wl, limit) for m in self.candidates()) if e.feasible]
        out = []
        for e in ests:
            dominated = any(o is not e and o.memory_bytes <= e.memory_bytes and o.comm_bytes <= e.comm_bytes
                            and o.step_seconds <= e.step_seconds and
                            (o.memory_bytes, o.comm_bytes, o.step_seconds) != (e.memory_bytes, e.comm_bytes, e.step_seconds)
                            for o in ests)
            if not dominated:
                out.append(e)
        return out

    def plan(self, wl: HybridWorkload, objective: PlanObjective = PlanObjective.MINIMIZE_STEP_TIME,
             limit: MemoryLimit | None = None) -> PlanEstimate:
        front = self.frontier(wl, limit)
        if not front:
            all_ = [self.estimate(m, wl, limit) for m in self.candidates()]
            raise ValueError("no feasible parallel plan: " + "; ".join(e.explain() for e in all_))
        key = {PlanObjective.MINIMIZE_STEP_TIME: lambda e: (e.step_seconds, e.memory_bytes),
               PlanObjective.MINIMIZE_MEMORY: lambda e: (e.memory_bytes, e.step_seconds),
               PlanObjective.MINIMIZE_COMMUNICATION: lambda e: (e.comm_bytes, e.step_seconds)}[objective]
        return min(front, key=key)
