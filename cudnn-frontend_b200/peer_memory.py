"""Device buffers that the other ranks of one node can address (CUDA IPC through the C ABI).

A :class:`PeerBuffer` is one allocation of the same size on every rank of a process group; after
construction every rank holds the device address of every other rank's copy, as Python ints and as
an int64 device tensor that kernels index by rank.  Kernels then load and store peer memory directly
over NVLink.  Nothing here synchronises the ranks: callers order their kernels with collectives.
"""

from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from . import _lib


class _DevicePointer:
    """Exposes a raw device allocation to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerBuffer:
    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        self.group = group
        self.world = 1 if group is None else dist.get_world_size(group)
        self.rank = 0 if group is None else dist.get_rank(group)
        self.nbytes = int(nbytes)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        lib = _lib.load()
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            _lib.check(lib.b200moe_peer_alloc(self.nbytes, ctypes.byref(ptr), handle))
        self._own = int(ptr.value)
        self._opened: List[int] = []
        self.ptrs: List[int] = [0] * self.world
        self.ptrs[self.rank] = self._own
        if self.world > 1:
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                p = ctypes.c_void_p()
                with torch.cuda.device(self.device):
                    _lib.check(lib.b200moe_peer_open(ctypes.create_string_buffer(h, 64), ctypes.byref(p)))
                self.ptrs[r] = int(p.value)
                self._opened.append(int(p.value))
        self.ptrs_dev = torch.tensor(self.ptrs, dtype=torch.int64, device=self.device)
        # this rank's copy as a flat uint8 tensor (views of it feed the GEMM operators)
        self.local = torch.as_tensor(_DevicePointer(self._own, self.nbytes), device=self.device)

    def view(self, dtype: torch.dtype, shape) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if nbytes > self.nbytes:
            raise ValueError(f"view of {nbytes} bytes exceeds the buffer ({self.nbytes} bytes)")
        return self.local[:nbytes].view(dtype).view(shape)

    def _device_ctx(self):
        """This buffer's device made current, all its work finished (a no-op context for a CPU stand-in)."""
        import contextlib

        if self.device.type != "cuda":
            return contextlib.nullcontext()
        torch.cuda.synchronize(self.device)
        return torch.cuda.device(self.device)

    def unmap_peers(self) -> None:
        """First half of the teardown: drop this rank's mappings of the other ranks' copies.  Every rank
        does this, then the ranks meet at a barrier, then :meth:`free_own` runs: an owner must not free
        memory that another process still has mapped."""
        lib = _lib.load()
        with self._device_ctx():
            for p in self._opened:
                lib.b200moe_peer_close(p)
        self._opened = []

    def free_own(self) -> None:
        """Second half of the teardown: free this rank's own allocation (after every rank has unmapped it)."""
        lib = _lib.load()
        with self._device_ctx():
            if self._own:
                lib.b200moe_peer_free(self._own)
                self._own = 0
        self.local = None

    def close(self) -> None:
        """Unmap the peers' copies, wait for every rank to have done so, free this rank's copy.  Collective
        over the buffer's group; call after a barrier that ends the last use of the buffers."""
        self.unmap_peers()
        if self.world > 1:
            dist.barrier(group=self.group)
        self.free_own()
