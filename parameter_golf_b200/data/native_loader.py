"""Python face of the C++ shard loader (``csrc/loader.cpp``): same slicing contract and the same ``state`` /
``restore`` / ``next_span_u16`` surface as :class:`..data.shards.DistributedTokenLoader`, plus a background prefetch
thread that fills a ring of page-locked buffers so that the training loop's host side is one pointer hand-over per
micro-step (the reference's loader does its reads on the step's critical path,
``parameter-golf-rs/crates/pg-data/src/token_stream.rs:222-296``).
"""
from __future__ import annotations

import glob
from typing import Optional

import numpy as np
import torch


class NativeTokenLoader:
    def __init__(self, pattern: str, rank: int = 0, world_size: int = 1):
        from ..ops import native
        files = sorted(glob.glob(pattern))
        if not files:
            raise FileNotFoundError(f"no shard matches {pattern!r}")
        if not (0 <= rank < world_size):
            raise ValueError("rank must be in [0, world_size)")
        self.rank, self.world_size = rank, world_size
        self.files = files
        self._L = native.load_raw().ShardLoader(files, rank, world_size)
        self._prefetching = False
        self._state = {"file_idx": 0, "pos": 0}

    # ---- synchronous path ----------------------------------------------------------------------------------------------
    def next_span_u16(self, global_tokens: int, grad_accum_steps: int = 1, out: Optional[np.ndarray] = None) -> np.ndarray:
        if self._prefetching:
            raise RuntimeError("stop the prefetch before using the synchronous path")
        span = global_tokens // (self.world_size * grad_accum_steps) + 1
        if out is None:
            out = np.empty(span, dtype=np.uint16)
        if out.shape[0] < span or out.dtype != np.uint16 or not out.flags.c_contiguous:
            raise ValueError("span buffer must be a contiguous uint16 array of at least global/(world*accum)+1 tokens")
        self._L.next_span_into(torch.from_numpy(out.view(np.int16))[:span], global_tokens, grad_accum_steps)
        fi, pos = self._L.state()
        self._state = {"file_idx": fi, "pos": pos}
        return out[:span]

    def state(self) -> dict:
        """Stream position after the last span handed out (prefetched spans not yet consumed do not count)."""
        return dict(self._state)

    def restore(self, st: dict) -> None:
        was = self._prefetching
        args = getattr(self, "_prefetch_args", None)
        if was:
            self.stop_prefetch()
        self._L.restore(int(st["file_idx"]) % len(self.files), int(st["pos"]))
        self._state = {"file_idx": int(st["file_idx"]) % len(self.files), "pos": int(st["pos"])}
        if was:
            self.start_prefetch(*args)

    # ---- prefetched path -------------------------------------------------------------------------------------------------
    def start_prefetch(self, global_tokens: int, grad_accum_steps: int = 1, depth: int = 0) -> None:
        """Start the worker thread. ``depth`` ring slots (default ``2*accum + 1``); the spans of one optimizer step
        (``grad_accum_steps`` of them) stay valid until the next step's first span is requested."""
        keep = max(1, grad_accum_steps)
        depth = depth or 2 * keep + 1
        self._L.restore(self._state["file_idx"], self._state["pos"])
        self._L.start_prefetch(global_tokens, grad_accum_steps, depth, keep)
        self._prefetch_args = (global_tokens, grad_accum_steps, depth)
        self._prefetching = True

    def next_prefetched(self) -> torch.Tensor:
        """The next span as an int16 CPU tensor (bit pattern of the uint16 ids) over a page-locked ring slot."""
        t, fi, pos = self._L.next_prefetched()
        self._state = {"file_idx": fi, "pos": pos}
        return t

    @property
    def pinned(self) -> bool:
        return bool(self._L.pinned())

    def stop_prefetch(self) -> None:
        if self._prefetching:
            self._L.stop_prefetch()
            self._prefetching = False
            self._L.restore(self._state["file_idx"], self._state["pos"])    # drop what the worker had fetched ahead
