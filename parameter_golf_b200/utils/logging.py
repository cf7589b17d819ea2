"""Run log (stdout + ``logs/<run_id>.txt``), host stage timers and CUDA-event timers.

Canonical lines follow the Python trainer (``train_gpt.py:1043-1046,992-995,1057-1060``):
``step:{s}/{N} train_loss:… train_time:…ms step_avg:…ms`` and the structured ``key=value`` /
``*_audit_json=`` protocol of the Rust CLI (``parameter-golf-rs/crates/pg-train/src/main.rs:218-431``).
Device timing is the max over ranks of CUDA-event durations
(``parameter-golf-rs/crates/pg-train/src/lib.rs:816-856``).
"""
from __future__ import annotations

import contextlib
import os
import time
from typing import Dict, List, Optional


class RunLog:
    def __init__(self, run_id: str, directory: Optional[str] = None, rank: int = 0, console: bool = True):
        self.rank = rank
        self.console = console
        self.path = None
        self.lines: List[str] = []
        if directory and rank == 0:
            os.makedirs(directory, exist_ok=True)
            self.path = os.path.join(directory, f"{run_id}.txt")

    def raw(self, msg: str):
        if self.rank != 0:
            return
        self.lines.append(msg)
        if self.console:
            print(msg, flush=True)
        if self.path:
            with open(self.path, "a", encoding="utf-8") as f:
                f.write(msg + "\n")

    info = raw


class StageTimers:
    """Accumulating host wall-clock timers keyed by stage name."""

    def __init__(self):
        self.total_ms: Dict[str, float] = {}
        self.count: Dict[str, int] = {}

    @contextlib.contextmanager
    def time(self, name: str):
        t0 = time.perf_counter()
        try:
            yield
        finally:
            self.total_ms[name] = self.total_ms.get(name, 0.0) + 1000.0 * (time.perf_counter() - t0)
            self.count[name] = self.count.get(name, 0) + 1

    def summary(self) -> Dict[str, float]:
        return {f"{k}_ms": round(v, 3) for k, v in self.total_ms.items()}


class CudaStageTimers:
    """CUDA-event stage timing on the launching stream. ``skip`` leading measurements per stage are
    dropped from the mean (warm-up); `reduce_max` takes the max over ranks."""

    def __init__(self, skip: int = 0):
        import torch
        self.torch = torch
        self.skip = skip
        self.pending: List[tuple] = []
        self.samples: Dict[str, List[float]] = {}

    @contextlib.contextmanager
    def time(self, name: str):
        a = self.torch.cuda.Event(enable_timing=True)
        b = self.torch.cuda.Event(enable_timing=True)
        a.record()
        try:
            yield
        finally:
            b.record()
            self.pending.append((name, a, b))

    def collect(self):
        self.torch.cuda.synchronize()
        for name, a, b in self.pending:
            self.samples.setdefault(name, []).append(a.elapsed_time(b))
        self.pending.clear()

    def mean_ms(self) -> Dict[str, float]:
        self.collect()
        return {k: sum(v[self.skip:]) / max(len(v[self.skip:]), 1) for k, v in self.samples.items()}

    def reduce_max(self) -> Dict[str, float]:
        import torch.distributed as dist
        m = self.mean_ms()
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            keys = sorted(m)
            t = self.torch.tensor([m[k] for k in keys], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            m = dict(zip(keys, t.tolist()))
        return m


_NVTX = os.environ.get("PGB_NVTX", "0") not in ("", "0")


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range around a stage (forward, backward, optimizer, collectives) so that a timeline profiler groups the
    launches of one stage. Off unless ``PGB_NVTX=1`` (a push/pop per stage per micro-batch is otherwise wasted work);
    a no-op when CUDA is not available."""
    if not _NVTX:
        yield
        return
    import torch
    if not torch.cuda.is_available():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
