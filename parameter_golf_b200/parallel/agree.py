"""Cross-rank agreement on host-side decisions.

Every rank times its own loop, so a decision derived from a local clock (the wall-clock cap, a wall-clock learning-rate
scale, an evaluation deadline) can flip on different steps on different ranks; a rank that leaves the loop one step
early deadlocks or corrupts the collectives of the ranks that stay. The fix is the one the reference uses for its cap
(``train_gpt.py:1049-1053``: ``reached_cap`` all-reduced with MAX): reduce the local value first and let every rank act
on the same number.
"""
from __future__ import annotations

from typing import Sequence

import torch


def agree(values: Sequence[float], op: str = "max", world_size: int = 1, device="cpu") -> list:
    """All-reduce a few host floats (``op`` = ``max`` or ``min``) over the default process group and return the agreed
    values; the identity when the job has one rank or no process group."""
    vals = [float(v) for v in values]
    if world_size <= 1:
        return vals
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return vals
    dev = torch.device(device)
    if dist.get_backend() == "gloo":
        dev = torch.device("cpu")
    t = torch.tensor(vals, dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.MIN)
    return [float(x) for x in t.tolist()]
