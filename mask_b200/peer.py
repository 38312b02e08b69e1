"""A float32 buffer of the same shape on every rank, each rank's copy mapped into every other
rank's process (CUDA IPC through ``mask_peer_*``): the addresses ``mask_plan_set_peer_outputs``
needs when each GPU is driven by its own process.  ``torch.distributed`` only carries the 64-byte
handles."""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ._lib import check, lib

HANDLE_BYTES = 64


class _Raw:
    """Lets torch view memory that the library allocated."""

    def __init__(self, ptr: int, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f4", "data": (ptr, False), "version": 2}


class PeerBuffer:
    def __init__(self, shape, device: torch.device, rank: int, world: int, group=None):
        self.shape, self.rank, self.world, self.group = tuple(shape), rank, world, group
        n = 1
        for s in self.shape:
            n *= int(s)
        self.bytes = max(4 * n, 4)
        L = lib()
        own = C.c_void_p()
        handle = C.create_string_buffer(HANDLE_BYTES)
        with torch.cuda.device(device):
            check(L.mask_peer_alloc(self.bytes, C.byref(own), handle), "mask_peer_alloc")
        self._own = own.value
        self.ptrs = [0] * world          # ptrs[j]: rank j's buffer as seen from this process
        self.ptrs[rank] = self._own
        self._opened = []
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, handle.raw, group=group)
            with torch.cuda.device(device):
                for j in range(world):
                    if j == rank:
                        continue
                    p = C.c_void_p()
                    check(L.mask_peer_open(handles[j], C.byref(p)), "mask_peer_open")
                    self.ptrs[j] = p.value
                    self._opened.append(p.value)
        self._raw = _Raw(self._own, self.shape)
        self.local = torch.as_tensor(self._raw, device=device)
        self.device = device

    def others(self, byte_offset: int = 0) -> torch.Tensor:
        """Device array of the other ranks' buffer addresses (+ byte_offset), for a plan."""
        a = [self.ptrs[j] + byte_offset for j in range(self.world) if j != self.rank]
        return torch.tensor(a, dtype=torch.int64, device=self.device)

    def close(self) -> None:
        """Collective: unmaps the peers' buffers, then frees this rank's."""
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        L = lib()
        with torch.cuda.device(self.device):
            for p in self._opened:
                check(L.mask_peer_close(C.c_void_p(p)), "mask_peer_close")
            self._opened = []
            if self.world > 1:
                dist.barrier(group=self.group)     # nobody frees while a peer still has it mapped
            self.local = None
            check(L.mask_peer_free(C.c_void_p(self._own)), "mask_peer_free")
        self._own = None
