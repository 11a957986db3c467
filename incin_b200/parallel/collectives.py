"""Stand-alone collectives and pipeline send/recv on peer-mapped buffers (the utility layer under the fused kernels).

Counterparts: ``CollectiveBackend::{all_reduce, all_gather, reduce_scatter, all_to_all, send_recv}``
(crates/incin-backends/src/transport/mod.rs) as executed by the NCCL transport (transport/nccl.rs:1842-1935), with
the result semantics of ``ReferenceTransport`` (transport/reference.rs:170-260): all-gather is rank-major, reduce-
scatter hands rank r the r-th slice, mean divides by the world size.

``PeerCollectives`` owns one symmetric staging buffer per rank.  Every call copies the input into the staging buffer,
passes the cross-GPU barrier kernel, runs one kernel that reads the peers' buffers over NVLink, and passes the barrier
again so the staging buffer can be reused; all on the current stream, so a sequence of calls can be captured in a CUDA
graph.  ``PipelineChannel`` is the stage-to-stage transfer: double-buffered slots in the receiver's memory, a copy
kernel followed by a release of a sequence number, and a bounded wait on the receiving side.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .. import _native as nat
from ..ops.gemm import status_word
from .symm import SymmetricBuffer

c_int, c_ll, c_void_p, c_uint = C.c_int, C.c_longlong, C.c_void_p, C.c_uint
_PTRS8 = C.POINTER(c_void_p)

nat.register_cuda_signatures({
    "incin_coll_all_gather": (c_int, [_PTRS8, c_int, c_int, c_ll, c_ll, c_void_p, c_void_p]),
    "incin_coll_all_to_all": (c_int, [_PTRS8, c_int, c_int, c_ll, c_ll, c_void_p, c_void_p]),
    "incin_coll_reduce": (c_int, [_PTRS8, c_int, c_ll, c_ll, c_ll, c_int, c_int, c_void_p, c_void_p]),
    "incin_p2p_send": (c_int, [c_void_p, c_void_p, c_ll, c_void_p, c_uint, c_void_p]),
    "incin_p2p_wait": (c_int, [c_void_p, c_uint, c_void_p, c_ll, c_void_p]),
    "incin_peer_barrier": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "incin_barrier_pad_bytes": (c_int, []),
})

_RED = {"sum": 0, "mean": 1, "avg": 1, "max": 2, "min": 3}


def _round16(n: int) -> int:
    return (n + 15) // 16 * 16


class PeerCollectives:
    def __init__(self, device: torch.device, group=None, *, max_bytes: int = 64 << 20):
        self.device, self.group = device, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise ValueError("peer collectives span at most the 8 GPUs of one node")
        self.max_bytes = _round16(max_bytes)
        self.buf = SymmetricBuffer(self.max_bytes, device).exchange(group)
        self.pad = SymmetricBuffer(nat.cuda().incin_barrier_pad_bytes(), device).exchange(group)
        self.pad.local_bytes.zero_()
        self._pad_ptrs = torch.tensor(self.pad.ptrs, dtype=torch.int64, device=device)
        self._ptrs = (c_void_p * 8)(*(self.buf.ptrs + [None] * (8 - self.world)))
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def _barrier(self) -> None:
        nat.check(nat.cuda().incin_peer_barrier(self._pad_ptrs.data_ptr(), self.world, self.rank, 1,
                                               status_word(self.device).data_ptr(), nat.stream_ptr()), "peer_barrier")

    def _stage(self, x: torch.Tensor) -> int:
        x = x.contiguous()
        nbytes = x.numel() * x.element_size()
        if nbytes % 16 or nbytes > self.max_bytes:
            raise ValueError(f"collective payload of {nbytes} bytes: need a multiple of 16 and at most {self.max_bytes}")
        self.buf.local_bytes[:nbytes].copy_(x.view(-1).view(torch.uint8))
        return nbytes

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """``[n, ...] -> [world * n, ...]`` (rank-major)."""
        nbytes = self._stage(x)
        out = torch.empty((self.world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=self.device)
        self._barrier()
        nat.check(nat.cuda().incin_coll_all_gather(self._ptrs, self.world, self.rank, 0, nbytes, out.data_ptr(),
                                                  nat.stream_ptr()), "all_gather")
        self._barrier()
        return out

    def all_to_all(self, x: torch.Tensor) -> torch.Tensor:
        """``x`` is ``world`` equal chunks along axis 0; chunk r goes to rank r.  Returns the chunks received."""
        nbytes = self._stage(x)
        if x.shape[0] % self.world or (nbytes // self.world) % 16:
            raise ValueError("all_to_all needs axis 0 divisible by the world size and 16-byte chunks")
        out = torch.empty_like(x, memory_format=torch.contiguous_format)
        self._barrier()
        nat.check(nat.cuda().incin_coll_all_to_all(self._ptrs, self.world, self.rank, 0, nbytes // self.world, out.data_ptr(),
                                                  nat.stream_ptr()), "all_to_all")
        self._barrier()
        return out

    def _reduce(self, x: torch.Tensor, op: str, first: int, n: int, out: torch.Tensor) -> torch.Tensor:
        if x.dtype not in (torch.float32, torch.bfloat16):
            raise TypeError("peer reductions take fp32 or bf16")
        self._stage(x)
        self._barrier()
        nat.check(nat.cuda().incin_coll_reduce(self._ptrs, self.world, 0, first, n, _RED[op], int(x.dtype == torch.bfloat16),
                                              out.data_ptr(), nat.stream_ptr()), "reduce")
        self._barrier()
        return out

    def all_reduce(self, x: torch.Tensor, op: str = "sum") -> torch.Tensor:
        """Every rank reads every peer's buffer once and reduces in rank order: all ranks get bitwise equal results."""
        return self._reduce(x, op, 0, x.numel(), torch.empty_like(x, memory_format=torch.contiguous_format))

    def reduce_scatter(self, x: torch.Tensor, op: str = "sum") -> torch.Tensor:
        """``[world * n, ...] -> [n, ...]``: rank r receives the reduction of everyone's r-th slice."""
        if x.shape[0] % self.world:
            raise ValueError("reduce_scatter needs axis 0 divisible by the world size")
        n = x.numel() // self.world
        out = torch.empty((x.shape[0] // self.world,) + tuple(x.shape[1:]), dtype=x.dtype, device=self.device)
        return self._reduce(x, op, self.rank * n, n, out)

    def close(self) -> None:
        self.buf.close()
        self.pad.close()


class PipelineChannel:
    """One direction of a pipeline edge ``src -> dst`` (ranks of ``group``): activations forward or gradients back.

    The receiver owns ``depth`` slots plus one flag word per slot.  Message k uses slot ``k % depth``; the sender
    copies into the slot and releases sequence number ``k + 1`` into its flag; the receiver waits (bounded) for that
    number and copies the slot out.  With ``depth`` >= the number of micro-batches in flight no acknowledgement is
    needed (GPipe and 1F1B keep at most ``stages`` in flight); reuse beyond that must be separated by the schedule's
    own synchronisation (the backward message of the same micro-batch travels the other way first).
    """

    def __init__(self, device: torch.device, src: int, dst: int, slot_bytes: int, group=None, depth: int = 4):
        self.device, self.src, self.dst, self.depth = device, src, dst, depth
        self.rank = dist.get_rank(group)
        self.slot_bytes = _round16(slot_bytes)
        self.slots = SymmetricBuffer(self.slot_bytes * depth, device).exchange(group)
        self.flags = SymmetricBuffer(256 * depth, device).exchange(group)      # one flag per 256-byte line
        self.flags.local_bytes.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        self.sent = self.received = 0

    def send(self, x: torch.Tensor) -> None:
        assert self.rank == self.src
        x = x.contiguous()
        nbytes = x.numel() * x.element_size()
        if nbytes % 16 or nbytes > self.slot_bytes:
            raise ValueError("pipeline message does not fit its slot (or is not a multiple of 16 bytes)")
        slot = self.sent % self.depth
        self.sent += 1
        nat.check(nat.cuda().incin_p2p_send(self.slots.ptrs[self.dst] + slot * self.slot_bytes, x.data_ptr(), nbytes,
                                           self.flags.ptrs[self.dst] + slot * 256, self.sent, nat.stream_ptr()), "p2p_send")

    def recv(self, shape, dtype, timeout_ms: int = 1000) -> torch.Tensor:
        assert self.rank == self.dst
        slot = self.received % self.depth
        self.received += 1
        nat.check(nat.cuda().incin_p2p_wait(self.flags.ptr + slot * 256, self.received, status_word(self.device).data_ptr(),
                                           timeout_ms, nat.stream_ptr()), "p2p_wait")
        out = torch.empty(shape, dtype=dtype, device=self.device)
        nbytes = out.numel() * out.element_size()
        out.view(-1).view(torch.uint8).copy_(self.slots.local_bytes[slot * self.slot_bytes: slot * self.slot_bytes + nbytes])
        return out

    def close(self) -> None:
        self.slots.close()
        self.flags.close()
