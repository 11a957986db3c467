"""The training-step engine: zero-grad -> forward -> backward -> (gradient reduction) -> optimiser,
eager for the first calls, then one CUDA-graph replay per step.

Everything in a step is enqueued on CUDA streams by hand-written kernels that
take no host-side decisions, so after two eager steps the whole step is
captured once and replayed; hyper-parameters that change per step (lr, step
count) live in device memory the kernels read.  On the CPU backend the same
object runs the PyTorch-CPU twins of the ops eagerly.

The reference's single-device loop is ``Trainer::fit``
(crates/incin/src/train.rs:576-617): per batch ``loss -> backward ->
optimizer.step -> loss.to_scalar()``.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch

from .optim.flat import ParamStore, _FlatOptimizer


class TrainStep:
    def __init__(self, model: torch.nn.Module, optimizer: _FlatOptimizer, *,
                 loss_fn: Callable[..., torch.Tensor] | None = None, use_graph: bool = True,
                 eager_steps: int = 2, reducer=None):
        self.model = model
        self.opt = optimizer
        self.store: ParamStore = optimizer.store
        self.loss_fn = loss_fn or (lambda m, *a: m(*a))
        self.device = self.store.device
        self.use_graph = bool(use_graph) and self.device.type == "cuda"
        self.eager_steps = eager_steps
        self.reducer = reducer  # data-parallel gradient reducer (fused reduce + optimiser), or None
        self.calls = 0
        self.graph: torch.cuda.CUDAGraph | None = None
        self.capture_error: str | None = None
        self.static_inputs: list[torch.Tensor] | None = None
        self.static_loss: torch.Tensor | None = None
        self.launches_per_step: int | None = None

    # one full step, enqueued on the current stream
    def _enqueue(self, inputs: Sequence[torch.Tensor]) -> torch.Tensor:
        from .telemetry import trace
        with trace.op_range("zero_grad"):
            self.store.zero_grad()
            if self.reducer is not None:
                self.reducer.begin_step()
        with trace.op_range("forward"):
            loss = self.loss_fn(self.model, *inputs)
        with trace.op_range("backward"):
            loss.backward()
            if self.device.type != "cuda":
                self.store.collect_autograd_grads()
        with trace.op_range("optimizer"):
            if self.reducer is not None:
                self.reducer.finish_step(self.opt)  # reduce-scatter + optimiser + all-gather, fused
            else:
                self.opt.launch()
        return loss.detach()

    def _capture(self, inputs: Sequence[torch.Tensor], mode: str = "global") -> None:
        self.static_inputs = [t.clone() for t in inputs]
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side, capture_error_mode=mode):
                self.static_loss = self._enqueue(self.static_inputs)
        torch.cuda.current_stream().wait_stream(side)
        self.graph = g

    def __call__(self, *inputs: torch.Tensor) -> torch.Tensor:
        """Run one optimisation step; returns the (device-resident) loss of this step."""
        self.calls += 1
        self.opt.prepare_step()
        if not self.use_graph or self.calls <= self.eager_steps:
            return self._enqueue(inputs)
        if self.graph is None:
            try:
                self._capture(inputs)
            except Exception as e:
                # capture is an optimisation; any failure leaves the eager path in charge (and says why)
                import traceback
                import warnings
                self.capture_error = f"{type(e).__name__}: {e}\n" + "".join(traceback.format_tb(e.__traceback__)[-6:])
                warnings.warn("CUDA-graph capture of the training step failed, running eagerly.  A common cause: a loss "
                              "tensor from a forward pass made BEFORE this step is still referenced, which keeps the "
                              "parameters' gradient-accumulator nodes of the default stream alive; autograd then records "
                              "an event on the default stream during capture, which CUDA forbids.  Drop that reference "
                              f"(del loss) or detach it.  Error: {self.capture_error}")
                self.use_graph = False
                self.graph = None
                torch.cuda.synchronize()
                return self._enqueue(inputs)
        for dst, src in zip(self.static_inputs, inputs):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        self.graph.replay()
        return self.static_loss


class StepPipeline:
    """Feeds a training step from pinned host batches without putting the copies or the loss read-back on the critical
    path.  ``submit(*host_tensors)`` copies the batch to a device staging slot on a copy stream (while the previous step
    still runs), enqueues the step on the current stream once the copy has landed and starts an asynchronous copy of
    that step's loss into pinned memory; ``pop()`` returns the oldest outstanding loss as a float, blocking only until
    that step has finished.  With ``depth`` slots, ``depth - 1`` steps can be in flight before a ``pop`` is needed::

        pipe = StepPipeline(step)
        for i, (tok, tgt) in enumerate(loader):        # pinned host tensors
            pipe.submit(tok, tgt)
            if i:
                log(pipe.pop())                        # loss of step i - 1
        log(pipe.pop())

    ``step`` is any callable taking device tensors and returning a device loss (a :class:`TrainStep`, typically).
    Every step's inputs cross host -> device and every step's loss crosses device -> host; only the waiting moves.
    """

    def __init__(self, step: Callable[..., torch.Tensor], depth: int = 2, device: torch.device | None = None):
        if depth < 2:
            raise ValueError("depth must be at least 2 (one slot being filled while another one runs)")
        self.step = step
        self.depth = depth
        self.device = device or getattr(step, "device", None) or torch.device("cuda", torch.cuda.current_device())
        self.copy_stream = torch.cuda.Stream(device=self.device)
        self._staging: list[list[torch.Tensor] | None] = [None] * depth
        self._loss_host = [torch.zeros((), dtype=torch.float32).pin_memory() for _ in range(depth)]
        self._ev_in = [torch.cuda.Event() for _ in range(depth)]
        self._ev_free: list[torch.cuda.Event | None] = [None] * depth
        self._ev_loss = [torch.cuda.Event() for _ in range(depth)]
        self.submitted = 0
        self.popped = 0

    @property
    def outstanding(self) -> int:
        return self.submitted - self.popped

    def submit(self, *host_inputs: torch.Tensor) -> None:
        if self.outstanding >= self.depth:
            raise RuntimeError(f"{self.outstanding} losses outstanding: call pop() before submitting another step")
        k = self.submitted % self.depth
        if self._staging[k] is None or any(s.shape != h.shape or s.dtype != h.dtype
                                           for s, h in zip(self._staging[k], host_inputs)):
            self._staging[k] = [torch.empty(h.shape, dtype=h.dtype, device=self.device) for h in host_inputs]
            self._ev_free[k] = None
        main = torch.cuda.current_stream(self.device)
        if self._ev_free[k] is not None:
            self.copy_stream.wait_event(self._ev_free[k])      # the step that last read this slot has consumed it
        with torch.cuda.stream(self.copy_stream):
            for dst, src in zip(self._staging[k], host_inputs):
                dst.copy_(src, non_blocking=True)
            self._ev_in[k].record(self.copy_stream)
        main.wait_event(self._ev_in[k])
        loss = self.step(*self._staging[k])
        ev = torch.cuda.Event()
        ev.record(main)
        self._ev_free[k] = ev
        self._loss_host[k].copy_(loss.detach().float().reshape(()), non_blocking=True)
        self._ev_loss[k].record(main)
        self.submitted += 1

    def pop(self) -> float:
        if self.outstanding <= 0:
            raise RuntimeError("no step outstanding")
        k = self.popped % self.depth
        self._ev_loss[k].synchronize()
        self.popped += 1
        return float(self._loss_host[k])

    def drain(self) -> list[float]:
        return [self.pop() for _ in range(self.outstanding)]
