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

    def close(self) -> None:
        for p in self._opened:
            nat.cuda().incin_symm_close(p)
        self._opened = []
