"""Peer-mapped device buffers shared between the per-GPU processes (CUDA IPC over NVLink/NVSwitch).

``SymmetricBuffer.create`` allocates the same number of bytes on every rank, exchanges the IPC handles
through ``torch.distributed`` (the plumbing layer) and maps every peer's allocation into this process.
``buf.local`` is a torch tensor view of the local allocation; ``buf.ptrs[r]`` is the device address of
rank r's allocation as seen from this process (``ptrs[rank]`` is the local address).  Kernels in
``libincin_sm100.so`` use these addresses with plain loads and stores.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .. import _native as nat

nat.register_cuda_signatures({
    "incin_symm_alloc": (C.c_int, [C.c_longlong, C.POINTER(C.c_void_p), C.c_char_p]),
    "incin_symm_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "incin_symm_close": (C.c_int, [C.c_void_p]),
    "incin_symm_free": (C.c_int, [C.c_void_p]),
    "incin_can_access_peer": (C.c_int, [C.c_int, C.c_int]),
})


class _DevMem:
    """Exposes a raw device allocation to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class MulticastBuffer:
    """A buffer that every rank of a group allocates at the same size, mapped into every peer AND bound to one
    NVSwitch multicast object: ``ptrs[r]`` are the peers' unicast addresses (as with :class:`SymmetricBuffer`),
    ``mc_ptr`` is the multicast address, through which ``multimem.ld_reduce`` returns the sum over all ranks and
    ``multimem.st`` writes into all of them.  Allocation, handle exchange and the multicast binding are PyTorch's
    symmetric-memory plumbing (``torch.distributed._symmetric_memory``: cuMem allocations shared by file descriptor);
    the kernels that use the addresses are this library's.

    Every rank must stay alive while such a buffer exists (a rank that exits while bound can fault its peers), so
    jobs that test rank loss keep to :class:`SymmetricBuffer`; ``available()`` is False when NVLS is switched off
    (``NCCL_NVLS_ENABLE=0``) or the platform has no multicast support."""

    @staticmethod
    def available() -> bool:
        import os
        if os.environ.get("NCCL_NVLS_ENABLE", "1") == "0" or os.environ.get("INCIN_MULTIMEM", "1") == "0":
            return False
        try:
            import torch.distributed._symmetric_memory  # noqa: F401
        except Exception:
            return False
        return dist.is_available() and dist.is_initialized() and torch.cuda.is_available()

    def __init__(self, nbytes: int, device: torch.device):
        import torch.distributed._symmetric_memory as symm_mem
        self.nbytes = (int(nbytes) + 15) // 16 * 16
        self.device = device
        self.local_bytes = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.local_bytes.zero_()
        self.ptr = self.local_bytes.data_ptr()
        self.ptrs: list[int] = [self.ptr]
        self.mc_ptr = 0
        self.rank, self.world = 0, 1
        self._hdl = None

    def typed(self, dtype: torch.dtype, numel: int | None = None) -> torch.Tensor:
        t = self.local_bytes.view(dtype)
        return t if numel is None else t[:numel]

    def exchange(self, group=None, session=None, ranks=None) -> "MulticastBuffer":
        import torch.distributed._symmetric_memory as symm_mem
        g = group if group is not None else dist.group.WORLD
        if session is not None:
            session.ensure_active()
        self._hdl = symm_mem.rendezvous(self.local_bytes, g)
        self.world, self.rank = dist.get_world_size(g), dist.get_rank(g)
        self.ptrs = [int(p) for p in self._hdl.buffer_ptrs]
        self.mc_ptr = int(self._hdl.multicast_ptr or 0)
        if self.ptrs[self.rank] != self.ptr or not self.mc_ptr:
            raise nat.NativeError("symmetric-memory rendezvous returned no multicast mapping for this buffer")
        return self

    def close(self) -> None:
        self._hdl = None


class SymmetricBuffer:
    def __init__(self, nbytes: int, device: torch.device):
        self.nbytes = int(nbytes)
        self.device = device
        p = C.c_void_p()
        self._handle = C.create_string_buffer(64)
        with torch.cuda.device(device):
            nat.check(nat.cuda().incin_symm_alloc(self.nbytes, C.byref(p), self._handle), "symm_alloc")
        self.ptr = p.value
        self._owner = _DevMem(self.ptr, self.nbytes)
        self.local_bytes = torch.as_tensor(self._owner, device=device)
        self.ptrs: list[int] = [self.ptr]
        self.rank, self.world = 0, 1
        self._opened: list[int] = []

    def typed(self, dtype: torch.dtype, numel: int | None = None) -> torch.Tensor:
        t = self.local_bytes.view(dtype)
        return t if numel is None else t[:numel]

    def exchange(self, group=None, session=None, ranks: list[int] | None = None) -> "SymmetricBuffer":
        """Collective: share this buffer's handle with every rank of the group and map theirs.  With a
        :class:`~incin_b200.parallel.session.CollectiveSession` that owns a rendezvous context the handles travel over
        the repo's own control channel (``ranks`` = the job ranks of this group, in group order); otherwise over
        ``torch.distributed``."""
        if session is not None and session.ctx is not None:
            if ranks is None:
                ranks = (dist.get_process_group_ranks(group) if group is not None else list(range(session.ctx.world)))
            self.world, self.rank = len(ranks), ranks.index(session.ctx.rank)
            session.ensure_active()
            handles = session.allgather(bytes(self._handle.raw), ranks)
        else:
            self.world = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(self._handle.raw), group=group)
        self.ptrs = []
        with torch.cuda.device(self.device):
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.ptrs.append(self.ptr)
                    continue
                p = C.c_void_p()
                nat.check(nat.cuda().incin_symm_open(h, C.byref(p)), f"symm_open(rank {r})")
                self.ptrs.append(p.value)
                self._opened.append(p.value)
        if session is not None and session.ctx is not None:
            session.barrier(ranks)
        else:
            dist.barrier(group=group)
        return self

    def mapped_over(self, group=None, session=None, ranks: list[int] | None = None) -> "SymmetricBuffer":
        """Collective over ANOTHER group: a second view of the same local memory whose ``ptrs`` are the mappings of that
        group's ranks (a gradient buffer that the data-parallel reducer mapped over its replicas is also summed over
        the tensor-parallel neighbours that share a K/V head).  The view keeps this buffer alive."""
        v = SymmetricBuffer.__new__(SymmetricBuffer)
        v.nbytes, v.device, v._handle, v.ptr = self.nbytes, self.device, self._handle, self.ptr
        v._owner, v.local_bytes, v._parent = self._owner, self.local_bytes, self
        v.ptrs, v.rank, v.world, v._opened = [self.ptr], 0, 1, []
        return v.exchange(group, session=session, ranks=ranks)

    def close(self) -> None:
        for p in self._opened:
            nat.cuda().incin_symm_close(p)
        self._opened = []
