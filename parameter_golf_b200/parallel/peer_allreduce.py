"""Two-shot all-reduce of a flat fp32 tensor on peer memory (reduce my slice out of every peer, write it back to every peer).

The same kernels as the replicated training step (`dist_engine.DistributedStep._step_replicated`), packaged for callers that
bring their own tensors: the packed gradient all-reduce of distributed test-time training
(``parameter-golf-rs/crates/pg-eval/src/gpu_lora_ttt.rs:551-568``, Python ``records/.../train_gpt.py:1197-1203``) goes through
it instead of an NCCL call. One instance owns a symmetric staging buffer of ``capacity`` floats and a signal pad; `mean_`
copies the tensor in, synchronises the ranks with the bounded barrier kernel, reduces, fans out and copies back, all on the
current stream. Every rank must call it the same number of times with the same element count.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import native as N
from .symm import SymmetricBuffer

_SIG_A, _SIG_B = 0, 64      # two barrier slots of the signal pad


class PeerAllReduce:
    def __init__(self, capacity: int, group=None):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.capacity = (int(capacity) + 3) // 4 * 4
        self.C = N.load()
        self.buf = SymmetricBuffer(self.capacity * 4, group)
        self.sig = SymmetricBuffer(1024 * 4, group)
        self.local = self.buf.view(0, (self.capacity,), torch.float32)
        self.epoch = 0

    def _barrier(self, slot: int):
        self.C.comm_barrier(self.sig.table, self.rank, self.world, slot, self.epoch, N.status_word())

    def mean_(self, flat: torch.Tensor) -> torch.Tensor:
        """In-place mean over ranks of a contiguous fp32 CUDA tensor with at most ``capacity`` elements."""
        n = flat.numel()
        if flat.dtype != torch.float32 or not flat.is_contiguous() or n > self.capacity:
            raise ValueError(f"PeerAllReduce.mean_: need a contiguous fp32 tensor of at most {self.capacity} elements")
        w, r = self.world, self.rank
        n4 = (n + 3) // 4
        self.local[:n].copy_(flat.view(-1))
        if n4 * 4 > n:
            self.local[n:n4 * 4].zero_()
        self.epoch += 1
        self._barrier(_SIG_A)                       # every rank's copy-in is complete
        a, b = (n4 * r // w) * 4, (n4 * (r + 1) // w) * 4
        if b > a:
            mine = self.local[a:b]
            self.C.comm_reduce_peers(self.buf.table, w, a, b - a, mine, 1.0 / w, None, 0.0, None, 0, None)
        self._barrier(_SIG_B)                       # every slice is reduced before anyone overwrites a peer's copy
        if b > a:
            self.C.comm_push_copy(self.local[a:b], self.buf.table, w, r, a)
        self.epoch += 1
        self._barrier(_SIG_A)                       # every slice has landed everywhere
        flat.view(-1).copy_(self.local[:n])
        return flat

    def close(self):
        self.buf.close()
        self.sig.close()
