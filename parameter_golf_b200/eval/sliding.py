"""Sliding-window scoring and the score-first chunk schedule.

Window rule (``parameter-golf-rs/crates/pg-eval/src/sliding.rs:46-53,78-93``; Python twin
``records/track_10min_16mb/2026-03-23_LeakyReLU_LegalTTT_ParallelMuon/train_gpt.py:1003-1071``): window starts
are ``0, stride, 2*stride, …`` as long as the window holds at least one target; window 0 scores all
of its tokens, every other window scores its last ``stride`` tokens (``s = max(wlen - stride, 0)``), so each
scored token sees at least ``window - stride`` tokens of context. Windows are split contiguously
over ranks and three scalars (loss sum, token count, byte count) are all-reduced.

Chunk rule for score-first test-time training (``sliding.rs:121-155``): a window belongs to the chunk
that contains the first token it scores.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import numpy as np
import torch

from ..data.bpb import BpbLuts, compute_bpb


def window_starts(total_tokens: int, window: int, stride: int, min_len: int = 1) -> List[int]:
    return [ws for ws in range(0, total_tokens, stride) if min(ws + window, total_tokens) - ws >= min_len or ws == 0]


def scored_range(ws: int, total_tokens: int, window: int, stride: int) -> Tuple[int, int]:
    """(s, wlen): the window scores its positions ``[s, wlen)``."""
    wlen = min(ws + window, total_tokens) - ws
    return (0 if ws == 0 else max(wlen - stride, 0)), wlen


def build_ttt_chunks(total_tokens: int, window: int, stride: int, chunk_tokens: int) -> List[List[int]]:
    starts = window_starts(total_tokens, window, stride, min_len=stride)
    n_chunks = (total_tokens + chunk_tokens - 1) // chunk_tokens
    chunks: List[List[int]] = [[] for _ in range(n_chunks)]
    for ws in starts:
        s, _ = scored_range(ws, total_tokens, window, stride)
        chunks[min((ws + s) // chunk_tokens, n_chunks - 1)].append(ws)
    return chunks


def rank_slice(n: int, rank: int, world: int) -> Tuple[int, int]:
    return (n * rank) // world, (n * (rank + 1)) // world


@dataclass
class ScoreSums:
    loss: float = 0.0
    tokens: float = 0.0
    bytes: float = 0.0

    def add(self, o: "ScoreSums"):
        self.loss += o.loss
        self.tokens += o.tokens
        self.bytes += o.bytes

    def all_reduce(self, device=None):
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            t = torch.tensor([self.loss, self.tokens, self.bytes], dtype=torch.float64, device=device or "cpu")
            dist.all_reduce(t)
            self.loss, self.tokens, self.bytes = (float(x) for x in t.tolist())
        return self

    def result(self) -> Tuple[float, float]:
        return compute_bpb(self.loss, self.tokens, self.bytes)


def score_windows(nll_fn: Callable, tokens: np.ndarray, starts: List[int], window: int, stride: int, luts: BpbLuts,
                  batch_windows: int = 32, device="cpu", deadline: Optional[Callable[[], bool]] = None) -> ScoreSums:
    """Score the given windows. ``nll_fn(ids[B,T], targets[B,T]) -> nll[B,T]`` (float)."""
    total = tokens.shape[0] - 1
    sums = ScoreSums()
    tok64 = tokens.astype(np.int64)
    for bi in range(0, len(starts), batch_windows):
        if deadline is not None and deadline():
            break
        batch = starts[bi:bi + batch_windows]
        x = np.zeros((len(batch), window), dtype=np.int64)
        y = np.zeros((len(batch), window), dtype=np.int64)
        mask = np.zeros((len(batch), window), dtype=bool)
        pos = np.zeros((len(batch), window), dtype=np.int64)          # index of each target in the validation stream
        for i, ws in enumerate(batch):
            s, wlen = scored_range(ws, total, window, stride)
            x[i, :wlen] = tok64[ws:ws + wlen]
            y[i, :wlen] = tok64[ws + 1:ws + wlen + 1]
            pos[i, :wlen] = np.arange(ws + 1, ws + wlen + 1)
            mask[i, s:wlen] = True
        nll = nll_fn(torch.from_numpy(x).to(device), torch.from_numpy(y).to(device))
        mt = torch.from_numpy(mask).to(nll.device)
        sums.loss += float((nll.double() * mt).sum())
        sums.tokens += float(mask.sum())
        sums.bytes += float(luts.token_bytes(x[mask], y[mask], pos[mask]).sum())
    return sums


def eval_sliding(nll_fn: Callable, tokens: np.ndarray, window: int, stride: int, luts: BpbLuts, rank: int = 0, world: int = 1,
                 batch_windows: int = 32, device="cpu") -> Tuple[float, float]:
    """(val_loss nats/token, bits per byte) over all windows, distributed by contiguous rank split."""
    total = tokens.shape[0] - 1
    starts = window_starts(total, window, stride)
    a, b = rank_slice(len(starts), rank, world)
    sums = score_windows(nll_fn, tokens, starts[a:b], window, stride, luts, batch_windows, device)
    return sums.all_reduce(device).result()


def find_temperature(runner, tokens: np.ndarray, seq_len: int, grid, batch_seqs: int = 16, device="cpu") -> Tuple[float, dict]:
    """Score ``tokens`` (training data, never the validation split) once per temperature of ``grid`` through ``runner.nll`` and
    return the temperature with the lowest mean loss and the whole table (the five-point search of the ternary record,
    ``records/track_10min_16mb/2026-03-24_74M_Ternary_.../train_gpt_cuda_ternary.py:1044-1054``). The runner's temperature is
    left at the winner."""
    n = (tokens.shape[0] - 1) // seq_len
    if n <= 0:
        raise ValueError("not enough calibration tokens for one sequence")
    tok64 = tokens.astype(np.int64)
    x = torch.from_numpy(tok64[: n * seq_len].reshape(n, seq_len)).to(device)
    y = torch.from_numpy(tok64[1: n * seq_len + 1].reshape(n, seq_len)).to(device)
    table = {}
    for t in grid:
        runner.temperature = float(t)
        total = 0.0
        for i in range(0, n, batch_seqs):
            total += float(runner.nll(x[i:i + batch_seqs], y[i:i + batch_seqs]).double().sum())
        table[float(t)] = total / (n * seq_len)
    best = min(table, key=table.get)
    runner.temperature = best
    return best, table


def eval_contiguous(nll_fn: Callable, tokens: np.ndarray, seq_len: int, luts: BpbLuts, rank: int = 0, world: int = 1,
                    batch_seqs: int = 32, device="cpu") -> Tuple[float, float]:
    """Non-overlapping evaluation of ``train_gpt.py:221-278``: every sequence scored once, rank-contiguous split."""
    total_seqs = (tokens.shape[0] - 1) // seq_len
    a, b = rank_slice(total_seqs, rank, world)
    sums = ScoreSums()
    tok64 = tokens.astype(np.int64)
    for s0 in range(a, b, batch_seqs):
        s1 = min(s0 + batch_seqs, b)
        span = tok64[s0 * seq_len: s1 * seq_len + 1]
        x, y = span[:-1].reshape(-1, seq_len), span[1:].reshape(-1, seq_len)
        nll = nll_fn(torch.from_numpy(x).to(device), torch.from_numpy(y).to(device))
        sums.loss += float(nll.double().sum())
        sums.tokens += float(x.size)
        sums.bytes += float(luts.token_bytes(x.reshape(-1), y.reshape(-1), np.arange(s0 * seq_len + 1, s1 * seq_len + 1)).sum())
    return sums.all_reduce(device).result()


def cosine_over_chunks(base_lr: float, chunk: int, num_chunks: int) -> float:
    return base_lr * 0.5 * (1.0 + math.cos(math.pi * chunk / max(num_chunks - 1, 1)))
