"""Collective session: the control channel, the agreed plan and the launch cursor that the fused kernels run under.

What the reference's NCCL transport does around every collective (crates/incin-backends/src/dist/nccl.rs):
``connect_context`` exchanges mesh digest + plan hash and rejects divergent ranks BEFORE a communicator exists
(:454-512, :1539-1587); ``validate_launch`` checks every launch against the agreed plan — position in the sequence,
semantic tag, collective kind, dtype, element count (:1016-1134, :1241-1280); a ``ContextOperationGuard`` checks the
shared fail-stop state first and invalidates it when the operation fails (:985-1014).

Here the "communicator" is a set of peer-mapped buffers, so the order is: build the plan -> :meth:`agree` (hash
exchange over the repo's own rendezvous channel; a mismatch raises before any IPC handle is opened) -> exchange
handles over the same channel (:meth:`allgather`) -> per fused launch :meth:`launch` (``ensure_active`` + cursor).
A device-side wait that gave up (kernel status word) is reported with :meth:`device_status`, which invalidates the
context so every later operation fails fast.

Without a rendezvous context (single process, or a job that only brought up ``torch.distributed``) a session still
validates launches against the local plan; agreement and handle exchange then fall back to ``torch.distributed``.
"""
from __future__ import annotations

from ..core.dtype import DTypeId
from .context import ContextFailure, DistributedContext, RendezvousError
from .mesh import DeviceMesh
from .plan import AgreedPlan, CollectiveKind, CollectivePlan, PlanCursor, PlanError, PreflightError, preflight


class CollectiveSession:
    def __init__(self, ctx: DistributedContext | None, mesh: DeviceMesh, rank: int | None = None):
        self.ctx, self.mesh = ctx, mesh
        self.rank = ctx.rank if (ctx is not None and rank is None) else int(rank or 0)
        self.launches = 0          # validated launches so far (diagnostics, tests)

    # ------------------------------------------------------------------------------------------ control plane
    def ensure_active(self) -> None:
        if self.ctx is not None:
            self.ctx.ensure_active()

    def allgather(self, blob: bytes, ranks: list[int] | None = None, torch_group=None) -> list[bytes]:
        """One equal-size blob from every rank of ``ranks`` (default: the whole job), in rank order."""
        if self.ctx is not None:
            every = self.ctx.allgather_bytes(blob)
            return every if ranks is None else [every[r] for r in ranks]
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized()):
            return [blob]
        out: list = [None] * dist.get_world_size(torch_group)
        dist.all_gather_object(out, blob, group=torch_group)
        return out

    def barrier(self, ranks: list[int] | None = None, torch_group=None) -> None:
        self.allgather(b"\0" * 8, ranks, torch_group)

    def agree(self, plan: CollectivePlan, ranks: list[int] | None = None, torch_group=None) -> "PlanLane":
        """Exchange (mesh id, plan hash, count) among ``ranks`` and return the lane launches are validated on.
        Raises :class:`PreflightError` (and invalidates the context) on any disagreement."""
        mine = plan.mesh_id.to_bytes(8, "little") + plan.hash.to_bytes(8, "little") + len(plan.descriptors).to_bytes(8, "little")
        blobs = self.allgather(mine, ranks, torch_group)
        reports = [(int.from_bytes(b[:8], "little"), int.from_bytes(b[8:16], "little"), int.from_bytes(b[16:24], "little"))
                   for b in blobs]
        try:
            agreed = preflight(len(reports), reports, plan)
        except PreflightError:
            if self.ctx is not None:
                self.ctx.invalidate(ContextFailure.PLAN_MISMATCH)
            raise
        return PlanLane(self, agreed)

    def device_status(self, code: int) -> None:
        """Report a kernel status word: non-zero means a bounded device wait gave up; the context becomes Failed."""
        if code:
            if self.ctx is not None:
                self.ctx.invalidate(ContextFailure.DEVICE_TIMEOUT)
            raise RendezvousError(ContextFailure.DEVICE_TIMEOUT, f"device status {code}")


class PlanLane:
    """One agreed plan with its cursor.  A plan describes one training step; :meth:`begin_step` rewinds."""

    def __init__(self, session: CollectiveSession, agreed: AgreedPlan):
        self.session, self.agreed = session, agreed
        self.cursor = PlanCursor(agreed)

    def begin_step(self) -> None:
        self.cursor.reset()

    def launch(self, *, tag: int, kind: CollectiveKind, elements: int, dtype: DTypeId = DTypeId.BF16):
        """Check the fail-stop state, then that this launch is the next one of the plan.  A mismatch is a programming
        error on this rank that would desynchronise the group, so it invalidates the context before it raises."""
        s = self.session
        s.ensure_active()
        try:
            d = self.cursor.next(tag=tag, kind=kind, elements=elements, dtype=dtype)
        except PlanError:
            if s.ctx is not None:
                s.ctx.invalidate(ContextFailure.PLAN_MISMATCH)
            raise
        s.launches += 1
        return d

    @property
    def complete(self) -> bool:
        return self.cursor.cursor == len(self.agreed.plan.descriptors)


def bind_session(ctx: DistributedContext, mesh_spec, probe=None) -> CollectiveSession:
    """A session of ``ctx`` over ``mesh_spec`` bound to the job's CUDA devices (one process per GPU on one node: rank r
    runs on the device the rendezvous reports for it).  One context serves several sessions (one per mesh shape)."""
    from ..core import Cuda
    from .mesh import CudaTopologyProbe
    devices = [Cuda(int(ctx.peer_device(r))) for r in range(ctx.world)]
    return CollectiveSession(ctx, DeviceMesh.bind(mesh_spec, devices, probe or CudaTopologyProbe()))


def session_from_env(mesh_spec, env=None) -> CollectiveSession:
    """Rendezvous from the environment (``INCIN_*`` variables, or torchrun's RANK / WORLD_SIZE / MASTER_*) and bind."""
    return bind_session(DistributedContext.from_env(env), mesh_spec)
