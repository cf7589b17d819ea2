"""Symmetric memory: identically laid out device buffers on every rank, mapped into every peer.

Each rank allocates its buffer with cudaMalloc, exports a CUDA IPC handle, and opens the handles of the other ranks
(`torch.distributed.all_gather_object` carries the 64-byte handles; that is the only use of the process group here).
The result is a table of ``world`` device addresses that kernels index by rank: plain peer loads and stores over
NVLink, no NCCL. This is the B200 counterpart of the reference's per-device NCCL communicators
(``parameter-golf-rs/crates/pg-core/src/nccl.rs:99-150``).
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist

from ..ops import native


class SymmetricBuffer:
    def __init__(self, nbytes: int, group=None):
        self.C = native.load()
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.cuda.current_device()
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.local_ptr = self.C.symm_alloc(self.nbytes)
        handles: List[bytes] = [b""] * self.world
        dist.all_gather_object(handles, self.C.symm_export(self.local_ptr), group=group)
        self.ptrs: List[int] = []
        self._opened: List[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.local_ptr)
            else:
                p = self.C.symm_import(h)
                self._opened.append(p)
                self.ptrs.append(p)
        self.table = torch.tensor(self.ptrs, dtype=torch.int64, device="cuda")
        self.bytes_view = self.C.tensor_from_ptr(self.local_ptr, self.nbytes, self.device)
        dist.barrier(group=group)

    def view(self, byte_offset: int, shape, dtype) -> torch.Tensor:
        """A tensor over this rank's copy of the buffer."""
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.empty((), dtype=dtype).element_size()
        return self.bytes_view[byte_offset:byte_offset + nb].view(dtype).view(*shape)

    def peer_view(self, rank: int, byte_offset: int, shape, dtype) -> torch.Tensor:
        """A tensor over rank ``rank``'s copy (for tests and debugging; kernels use `table`)."""
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.empty((), dtype=dtype).element_size()
        t = self.C.tensor_from_ptr(self.ptrs[rank] + byte_offset, nb, self.device)
        return t.view(dtype).view(*shape)

    def close(self):
        """Unmap peers and free the local buffer. Call on every rank, between steps, with no kernel in flight."""
        torch.cuda.synchronize()
        for p in self._opened:
            self.C.symm_close(p)
        self._opened = []
        if self.local_ptr:
            dist.barrier(group=self.group)
            self.C.symm_free(self.local_ptr)
            self.local_ptr = 0
