"""Complementary training: tokens that plain bigram statistics already predict get a smaller training-loss weight.

Counterpart of ``parameter-golf-rs/crates/pg-kernels/src/complementary.rs`` (`BigramStats` :27-150, weighting curves
:156-200, `complementary_weights` :204-224, `weighted_mean_loss` :226-240, `scale_grad_logits_by_weight` :245-254).

* `BigramStats` — dense add-one-smoothed table ``counts[prev, curr]`` with incrementally kept row sums, mergeable across
  shards and serialisable as ``[u32 vocab][u64 row_sums[V]][u32 counts[V*V]]`` little-endian (the reference's layout).
* `apply_shape` — the three curves: ``linear`` ``w = max(0, 1 - a p)``; ``power`` ``w = max(0, 1 - a p^k)``;
  ``floored`` (default, floor 0.2, min_w 0.25) ``w = 1`` for ``p <= floor`` else ``max(min_w, 1 - a (p - floor)/(1 - floor))``.
* `weight_table` — the curve applied to the whole table once: a ``[V, V]`` fp32 array. The CUDA engine looks the weight
  of a (previous token, target) pair up in this table inside its loss kernel, so the per-step cost is one 4-byte read
  per token; the CPU path indexes it with NumPy.
* `weighted_mean_loss` normalises by the SUM of weights, so down-weighted tokens shrink the denominator too.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Optional

import numpy as np


@dataclass(frozen=True)
class WeightShape:
    kind: str = "floored"          # "linear" | "power" | "floored"
    power: float = 2.0
    floor: float = 0.2
    min_w: float = 0.25

    def __post_init__(self):
        if self.kind not in ("linear", "power", "floored"):
            raise ValueError(f"unknown complementary weight shape {self.kind!r}")


class BigramStats:
    """Counts of adjacent token pairs; ``prob`` is add-one smoothed and uniform for a row never seen."""

    def __init__(self, vocab_size: int):
        if vocab_size <= 0:
            raise ValueError("vocab_size must be positive")
        self.vocab_size = int(vocab_size)
        self.counts = np.zeros((self.vocab_size, self.vocab_size), dtype=np.uint32)
        self.row_sums = np.zeros(self.vocab_size, dtype=np.uint64)

    # ---- building ----------------------------------------------------------------------------------------------------
    def add_sequence(self, tokens) -> None:
        """Add every adjacent pair of ``tokens`` (a 1-D integer array); ids outside the vocabulary are an error."""
        t = np.asarray(tokens).astype(np.int64, copy=False).reshape(-1)
        if t.size < 2:
            return
        if t.min() < 0 or t.max() >= self.vocab_size:
            raise ValueError("token id outside the vocabulary")
        V = self.vocab_size
        flat = np.bincount(t[:-1] * V + t[1:], minlength=V * V)
        self.counts += flat.reshape(V, V).astype(np.uint32)
        self.row_sums += np.bincount(t[:-1], minlength=V).astype(np.uint64)

    def merge(self, other: "BigramStats") -> None:
        if other.vocab_size != self.vocab_size:
            raise ValueError("cannot merge bigram tables of different vocabularies")
        self.counts += other.counts
        self.row_sums += other.row_sums

    # ---- queries -----------------------------------------------------------------------------------------------------
    def count(self, prev: int, curr: int) -> int:
        return int(self.counts[prev, curr])

    def prob(self, prev: int, curr: int) -> float:
        return float((float(self.counts[prev, curr]) + 1.0) / (float(self.row_sums[prev]) + self.vocab_size))

    def prob_table(self) -> np.ndarray:
        """``P(curr | prev)`` for every pair, fp32 ``[V, V]``; rows sum to one."""
        den = self.row_sums.astype(np.float64)[:, None] + float(self.vocab_size)
        return ((self.counts.astype(np.float64) + 1.0) / den).astype(np.float32)

    def row_entropy(self, prev: int) -> float:
        """Entropy of the smoothed row in nats."""
        den = float(self.row_sums[prev]) + self.vocab_size
        p = (self.counts[prev].astype(np.float64) + 1.0) / den
        return float(-(p * np.log(p)).sum())

    # ---- serialisation -----------------------------------------------------------------------------------------------
    def to_bytes(self) -> bytes:
        return (struct.pack("<I", self.vocab_size) + self.row_sums.astype("<u8").tobytes() +
                self.counts.astype("<u4").tobytes())

    @classmethod
    def from_bytes(cls, data: bytes) -> "BigramStats":
        if len(data) < 4:
            raise ValueError("bigram table: truncated header")
        (V,) = struct.unpack_from("<I", data, 0)
        need = 4 + 8 * V + 4 * V * V
        if V == 0 or len(data) != need:
            raise ValueError(f"bigram table: expected {need} bytes for vocab {V}, got {len(data)}")
        st = cls(V)
        st.row_sums = np.frombuffer(data, dtype="<u8", count=V, offset=4).astype(np.uint64)
        st.counts = np.frombuffer(data, dtype="<u4", count=V * V, offset=4 + 8 * V).astype(np.uint32).reshape(V, V)
        if not np.array_equal(st.counts.sum(axis=1, dtype=np.uint64), st.row_sums):
            raise ValueError("bigram table: row sums do not match the counts")
        return st


def apply_shape(p, alpha: float, shape: WeightShape = WeightShape()):
    """Weight of a token whose bigram probability is ``p`` (scalar or array)."""
    p = np.asarray(p, dtype=np.float32)
    a = np.float32(alpha)
    if shape.kind == "linear":
        w = np.maximum(1.0 - a * p, 0.0)
    elif shape.kind == "power":
        w = np.maximum(1.0 - a * np.power(p, np.float32(shape.power)), 0.0)
    else:
        norm = (p - np.float32(shape.floor)) / max(1.0 - shape.floor, 1e-6)
        w = np.where(p <= shape.floor, 1.0, np.maximum(1.0 - a * norm, shape.min_w))
    return w.astype(np.float32)


def weight_table(stats: BigramStats, alpha: float, shape: WeightShape = WeightShape()) -> np.ndarray:
    """``[V, V]`` fp32 weights ``w[prev, curr]``; all ones when ``alpha <= 0``."""
    if alpha <= 0:
        return np.ones((stats.vocab_size, stats.vocab_size), dtype=np.float32)
    return apply_shape(stats.prob_table(), alpha, shape)


def complementary_weights(prev_tokens, curr_tokens, stats: BigramStats, alpha: float, shape: WeightShape = WeightShape(),
                          table: Optional[np.ndarray] = None) -> np.ndarray:
    """One weight per target: ``prev_tokens[i]`` is the context token of target ``curr_tokens[i]``."""
    prev = np.asarray(prev_tokens).astype(np.int64, copy=False)
    curr = np.asarray(curr_tokens).astype(np.int64, copy=False)
    if prev.shape != curr.shape:
        raise ValueError("prev and curr token arrays must have the same shape")
    if alpha <= 0:
        return np.ones(prev.shape, dtype=np.float32)
    if table is not None:
        return table[prev, curr].astype(np.float32, copy=False)
    den = stats.row_sums[prev].astype(np.float64) + float(stats.vocab_size)
    p = ((stats.counts[prev, curr].astype(np.float64) + 1.0) / den).astype(np.float32)
    return apply_shape(p, alpha, shape)


def weighted_mean_loss(losses, weights) -> float:
    l = np.asarray(losses, dtype=np.float64).reshape(-1)
    w = np.asarray(weights, dtype=np.float64).reshape(-1)
    if l.shape != w.shape:
        raise ValueError("losses and weights must have the same length")
    den = w.sum()
    return 0.0 if den <= 1e-12 else float((l * w).sum() / den)


def scale_grad_logits_by_weight(grad_logits: np.ndarray, weights, vocab_size: int) -> np.ndarray:
    """Scale row ``t`` of a ``[T, V]`` (or flat ``T*V``) logits gradient by ``weights[t]``, in place."""
    w = np.asarray(weights, dtype=grad_logits.dtype).reshape(-1)
    if grad_logits.size != w.size * vocab_size:
        raise ValueError("gradient size must be len(weights) * vocab_size")
    g = grad_logits.reshape(w.size, vocab_size)
    g *= w[:, None]
    return grad_logits


def stats_from_stream(pattern: str, vocab_size: int, max_tokens: int) -> BigramStats:
    """Table built from the first ``max_tokens`` tokens of the shards matching ``pattern`` (sorted, shard by shard;
    pairs that straddle two shards are not counted)."""
    import glob

    from ..data.shards import open_shard
    st = BigramStats(vocab_size)
    left = int(max_tokens)
    for path in sorted(glob.glob(pattern)):
        if left <= 1:
            break
        tok = open_shard(path)[:left]
        st.add_sequence(np.asarray(tok))
        left -= int(tok.size)
    return st
