"""Pipeline-parallel execution of one stage: GPipe and 1F1B over micro-batches, with optional activation recompute.

Counterpart of ``TwoRankPipeline`` / ``PipelinePlanBuilder`` and the NCCL send/recv launches that carry
``ForwardActivation`` / ``BackwardGradient`` transfers (crates/incin-core/src/dist/pipeline.rs;
crates/incin-backends/src/transport/nccl.rs:801-894, 1889-1935).  The reference plans and moves the tensors; the
order each stage works through comes from the same clocked timeline the planner uses
(:func:`incin_b200.parallel.strategies.build_timeline`), so what runs is exactly what was planned.

Transfers go through an ``Edge`` object with ``send(tensor)`` / ``recv(shape, dtype)``:

* :class:`PeerEdge`   the GPU path: :class:`~incin_b200.parallel.collectives.PipelineChannel` (copy into the next
  stage's memory over NVLink + signal; the receiver's wait is bounded and reports through the device status word);
* :class:`DistEdge`   ``torch.distributed`` send/recv (gloo on CPU for the host-side tests, NCCL as a baseline).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from .strategies import ActivationCheckpoint, PipelineSchedule, build_timeline


class DistEdge:
    def __init__(self, src: int, dst: int, group=None):
        self.src, self.dst, self.group = src, dst, group
        self._pending: list = []

    def send(self, x: torch.Tensor) -> None:
        # non-blocking: neighbouring stages may both be sending (activation one way, gradient the other)
        x = x.contiguous()
        self._pending.append((dist.isend(x, self.dst, group=self.group), x))

    def flush(self) -> None:
        for work, _ in self._pending:
            work.wait()
        self._pending = []

    def recv(self, shape, dtype, device="cpu") -> torch.Tensor:
        out = torch.empty(shape, dtype=dtype, device=device)
        dist.recv(out, self.src, group=self.group)
        return out


class PeerEdge:
    def __init__(self, channel, timeout_ms: int = 5000):
        self.ch, self.timeout_ms = channel, timeout_ms

    def send(self, x: torch.Tensor) -> None:
        self.ch.send(x)

    def recv(self, shape, dtype, device=None) -> torch.Tensor:
        return self.ch.recv(shape, dtype, self.timeout_ms)


@dataclass
class StageIO:
    """Edges of one stage; ``None`` at the ends of the pipeline."""
    fwd_in: object | None = None     # activations from the previous stage
    fwd_out: object | None = None    # activations to the next stage
    bwd_in: object | None = None     # gradients from the next stage
    bwd_out: object | None = None    # gradients to the previous stage


class PipelineStage:
    """Runs ``module`` as stage ``index`` of ``stages``.

    ``step(inputs, loss_fn)``: ``inputs`` is the list of micro-batch inputs on the first stage (ignored elsewhere);
    ``loss_fn(output, microbatch_index) -> scalar`` is called on the last stage.  Parameter gradients accumulate in
    ``.grad`` (or ``main_grad`` for modules built on the framework's ops) over the micro-batches.  Returns the list
    of micro-batch losses on the last stage, ``[]`` elsewhere.
    """

    def __init__(self, module, index: int, stages: int, io: StageIO, act_shape, act_dtype, device,
                 schedule: PipelineSchedule = PipelineSchedule.ONE_F_ONE_B,
                 checkpoint: ActivationCheckpoint = ActivationCheckpoint.KEEP):
        self.module, self.index, self.stages, self.io = module, index, stages, io
        self.act_shape, self.act_dtype, self.device = tuple(act_shape), act_dtype, device
        self.schedule, self.checkpoint = schedule, checkpoint

    def _forward(self, x, m, loss_fn):
        y = self.module(x)
        if self.index == self.stages - 1:
            return loss_fn(y, m)
        return y

    def step(self, inputs, loss_fn, microbatches: int | None = None):
        M = microbatches if microbatches is not None else len(inputs)
        timeline = build_timeline(self.schedule, self.stages, M, self.checkpoint)
        first, last = self.index == 0, self.index == self.stages - 1
        saved: dict[int, tuple] = {}
        losses = []
        for row in timeline.clocks:
            act = row[self.index]
            if act is None:
                continue
            kind, m = act[0], int(act[1:])
            if kind == "F":
                x = inputs[m] if first else self.io.fwd_in.recv(self.act_shape, self.act_dtype, self.device)
                if not first:
                    x.requires_grad_(True)
                if self.checkpoint is ActivationCheckpoint.RECOMPUTE:
                    with torch.no_grad():
                        y = self._forward(x, m, loss_fn)
                    saved[m] = (x, None)
                else:
                    y = self._forward(x, m, loss_fn)
                    saved[m] = (x, y)
                if last:
                    losses.append(y.detach())
                else:
                    self.io.fwd_out.send(y.detach())
            else:
                x, y = saved.pop(m)
                if y is None:      # recompute the stage with autograd on
                    y = self._forward(x, m, loss_fn)
                if last:
                    (y / M).backward()
                else:
                    g = self.io.bwd_in.recv(self.act_shape, self.act_dtype, self.device)
                    y.backward(g)
                if not first:
                    self.io.bwd_out.send(x.grad)
        for edge in (self.io.fwd_out, self.io.bwd_out):
            if edge is not None and hasattr(edge, "flush"):
                edge.flush()
        return losses
