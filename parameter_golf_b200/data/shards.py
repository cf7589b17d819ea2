"""uint16 token shards: file format, synthetic generator, sequential stream and per-rank loader.

Shard format (``parameter-golf-rs/crates/pg-data/src/shard.rs:6-17,36-77``; written by
``data/download_hf_docs_and_tokenize.py:134-150`` and read by ``train_gpt.py:429-443``):
a header of 256 little-endian int32 (``[0]=20240520`` magic, ``[1]=1`` version, ``[2]=num_tokens``)
followed by ``num_tokens`` little-endian uint16 ids; the file length must be ``1024 + 2*num_tokens``.

The loader contract (``pg-data/src/token_stream.rs:20-42,193-248``, ``train_gpt.py:486-494``): shards are
visited in sorted-glob order and wrap around; for one (micro-)step the stream hands out
``world * (L+1)`` tokens and rank ``r`` keeps the span ``[r*(L+1), (r+1)*(L+1))`` where
``L = global_tokens / (world * grad_accum)``; inputs are ``span[:-1]`` and targets ``span[1:]``.

There is no network here, so training data is a seeded order-1 Markov chain whose rows are
Zipf(s) distributions over the vocabulary (`generate_markov_tokens`).
"""
from __future__ import annotations

import glob
import os
from typing import Optional

import numpy as np

SHARD_MAGIC = 20240520
SHARD_VERSION = 1
HEADER_INTS = 256
HEADER_BYTES = HEADER_INTS * 4


class ShardError(ValueError):
    pass


def write_shard(path: str, tokens: np.ndarray) -> None:
    tokens = np.ascontiguousarray(tokens)
    if tokens.dtype != np.uint16:
        if tokens.size and (tokens.min() < 0 or tokens.max() > 65535):
            raise ShardError("token ids do not fit uint16")
        tokens = tokens.astype("<u2")
    header = np.zeros(HEADER_INTS, dtype="<i4")
    header[0], header[1], header[2] = SHARD_MAGIC, SHARD_VERSION, tokens.size
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = f"{path}.tmp{os.getpid()}"          # readers never see a partially written shard: write aside, then rename
    with open(tmp, "wb") as f:
        f.write(header.tobytes())
        f.write(tokens.astype("<u2", copy=False).tobytes())
    os.replace(tmp, path)


def read_shard_header(path: str) -> int:
    size = os.path.getsize(path)
    if size < HEADER_BYTES:
        raise ShardError(f"{path}: shorter than the 1024-byte header")
    header = np.fromfile(path, dtype="<i4", count=HEADER_INTS)
    if int(header[0]) != SHARD_MAGIC:
        raise ShardError(f"{path}: bad magic {int(header[0])}")
    if int(header[1]) != SHARD_VERSION:
        raise ShardError(f"{path}: unsupported version {int(header[1])}")
    n = int(header[2])
    if n < 0 or size != HEADER_BYTES + 2 * n:
        raise ShardError(f"{path}: size {size} does not match header token count {n}")
    return n


def open_shard(path: str) -> np.ndarray:
    """Memory-map a shard and return its uint16 token array (read-only view)."""
    n = read_shard_header(path)
    if n == 0:
        return np.zeros(0, dtype=np.uint16)
    return np.memmap(path, dtype="<u2", mode="r", offset=HEADER_BYTES, shape=(n,))


# ---- synthetic data -------------------------------------------------------------------------------

def zipf_cdf(vocab: int, s: float = 1.1) -> np.ndarray:
    p = 1.0 / np.arange(1, vocab + 1, dtype=np.float64) ** s
    c = np.cumsum(p / p.sum())
    c[-1] = 1.0
    return c


def markov_row_maps(vocab: int, seed: int):
    """Per-previous-token bijection rank -> id: ``id = (mul[prev] * rank + add[prev]) mod vocab`` when
    ``vocab`` is a power of two (odd multiplier), else a rotation ``(rank + add[prev]) mod vocab``."""
    rng = np.random.default_rng(seed ^ 0x5EED)
    add = rng.integers(0, vocab, size=vocab, dtype=np.int64)
    if vocab & (vocab - 1) == 0:
        mul = rng.integers(0, vocab // 2, size=vocab, dtype=np.int64) * 2 + 1
    else:
        mul = np.ones(vocab, dtype=np.int64)
    return mul, add


def generate_markov_tokens(n: int, vocab: int = 1024, seed: int = 0, s: float = 1.1, streams: int = 4096,
                           chain_seed: Optional[int] = None) -> np.ndarray:
    """``n`` ids from a seeded order-1 Markov chain whose transition rows are Zipf(``s``) over ``vocab``
    ids. ``streams`` independent chains are advanced in lock-step (vectorised) and laid out
    back to back, so the result is a function of ``(n, vocab, seed, s, streams, chain_seed)`` only.
    ``chain_seed`` fixes the transition structure (which id each rank of a row maps to) separately from the sampling
    ``seed``: shards of one dataset share the chain and differ in the draws, so a model trained on one shard is
    evaluated on the same process."""
    if n <= 0:
        return np.zeros(0, dtype=np.uint16)
    streams = max(1, min(streams, n))
    steps = -(-n // streams)
    cdf = zipf_cdf(vocab, s)
    mul, add = markov_row_maps(vocab, seed if chain_seed is None else chain_seed)
    rng = np.random.default_rng(seed)
    out = np.empty((streams, steps), dtype=np.uint16)
    prev = rng.integers(0, vocab, size=streams, dtype=np.int64)
    for t in range(steps):
        rank = np.searchsorted(cdf, rng.random(streams), side="left").astype(np.int64)
        np.minimum(rank, vocab - 1, out=rank)
        prev = (mul[prev] * rank + add[prev]) % vocab
        out[:, t] = prev
    return out.reshape(-1)[:n].copy()


def write_synthetic_dataset(root: str, vocab: int = 1024, train_tokens: int = 1 << 24, val_tokens: int = 1 << 20,
                            train_shards: int = 1, seed: int = 1337, prefix: str = "fineweb") -> str:
    """Write ``<prefix>_train_NNNNNN.bin`` / ``<prefix>_val_000000.bin`` shards under ``root``."""
    os.makedirs(root, exist_ok=True)
    per = train_tokens // max(train_shards, 1)
    for i in range(train_shards):
        p = os.path.join(root, f"{prefix}_train_{i:06d}.bin")
        if not (os.path.exists(p) and os.path.getsize(p) == HEADER_BYTES + 2 * per):
            write_shard(p, generate_markov_tokens(per, vocab, seed + 17 * i, chain_seed=seed))
    p = os.path.join(root, f"{prefix}_val_000000.bin")
    if not (os.path.exists(p) and os.path.getsize(p) == HEADER_BYTES + 2 * val_tokens):
        write_shard(p, generate_markov_tokens(val_tokens, vocab, seed + 99991, chain_seed=seed))
    return root


# ---- stream + loader ---------------------------------------------------------------------------------

class TokenStream:
    """Sequential reader over sorted shards with wrap-around."""

    def __init__(self, pattern: str):
        self.files = sorted(glob.glob(pattern))
        if not self.files:
            raise FileNotFoundError(f"no shard matches {pattern!r}")
        self.file_idx = 0
        self.tokens = open_shard(self.files[0])
        self.pos = 0

    def _advance(self) -> None:
        self.file_idx = (self.file_idx + 1) % len(self.files)
        self.tokens = open_shard(self.files[self.file_idx])
        self.pos = 0

    def state(self) -> dict:
        return {"file_idx": self.file_idx, "pos": self.pos}

    def restore(self, st: dict) -> None:
        self.file_idx = int(st["file_idx"]) % len(self.files)
        self.tokens = open_shard(self.files[self.file_idx])
        self.pos = int(st["pos"])

    def take_into(self, out: np.ndarray) -> np.ndarray:
        n, done = out.shape[0], 0
        empties = 0
        while done < n:
            avail = self.tokens.shape[0] - self.pos
            if avail <= 0:
                self._advance()
                empties += 1
                if empties > len(self.files):
                    raise ShardError("all shards are empty")
                continue
            empties = 0
            k = min(n - done, avail)
            out[done:done + k] = self.tokens[self.pos:self.pos + k]
            self.pos += k
            done += k
        return out

    def take(self, n: int) -> np.ndarray:
        return self.take_into(np.empty(n, dtype=np.uint16))

    def skip(self, n: int) -> None:
        while n > 0:
            avail = self.tokens.shape[0] - self.pos
            if avail <= 0:
                self._advance()
                continue
            k = min(n, avail)
            self.pos += k
            n -= k


class DistributedTokenLoader:
    """Per-rank disjoint spans of the shared token stream (every rank reads the same files and skips
    the other ranks' spans, so no communication is needed and batches are bit-identical to the
    reference loader given the same shards)."""

    def __init__(self, pattern: str, rank: int = 0, world_size: int = 1):
        if not (0 <= rank < world_size):
            raise ValueError("rank must be in [0, world_size)")
        self.rank, self.world_size = rank, world_size
        self.stream = TokenStream(pattern)

    def next_span_u16(self, global_tokens: int, grad_accum_steps: int = 1, out: Optional[np.ndarray] = None) -> np.ndarray:
        local = global_tokens // (self.world_size * grad_accum_steps)
        span = local + 1
        self.stream.skip(self.rank * span)
        if out is None:
            out = np.empty(span, dtype=np.uint16)
        self.stream.take_into(out[:span])
        self.stream.skip((self.world_size - 1 - self.rank) * span)
        return out[:span]

    def next_batch(self, global_tokens: int, seq_len: int, grad_accum_steps: int = 1):
        """(inputs, targets) as int64 numpy arrays of shape [local_tokens/seq_len, seq_len]."""
        span = self.next_span_u16(global_tokens, grad_accum_steps).astype(np.int64)
        return span[:-1].reshape(-1, seq_len), span[1:].reshape(-1, seq_len)

    def state(self) -> dict:
        return self.stream.state()

    def restore(self, st: dict) -> None:
        self.stream.restore(st)


def is_byte_sidecar_path(path: str) -> bool:
    """Byte-count sidecars share the shard format and often the directory of the token shards; their file names carry
    ``_bytes_`` or ``val_bytes`` (``pg-data/src/token_stream.rs:347-352``)."""
    name = os.path.basename(path)
    return "_bytes_" in name or "val_bytes" in name


def load_validation_byte_sidecar(pattern: str, max_tokens: Optional[int] = None) -> np.ndarray:
    """Bytes per validation position as float32, from shards aligned one-to-one with the token shards
    (``pg-data/src/token_stream.rs:354-369``). ``max_tokens`` keeps the same ``max_tokens + 1`` prefix as the token loader."""
    files = sorted(glob.glob(pattern))
    if not files:
        raise FileNotFoundError(f"no byte sidecar matches {pattern!r}")
    raw = np.concatenate([np.asarray(open_shard(f)) for f in files])
    if max_tokens is not None:
        raw = raw[: max_tokens + 1]
    return raw.astype(np.float32)


def load_validation_tokens(pattern: str, seq_len: int, max_tokens: Optional[int] = None) -> np.ndarray:
    """All validation shards concatenated, truncated to ``k*seq_len + 1`` tokens
    (``train_gpt.py:211-219``; limit variant ``pg-data/src/token_stream.rs:300-336``). Byte-count sidecars that the
    pattern happens to match are left out."""
    files = sorted(f for f in glob.glob(pattern) if not is_byte_sidecar_path(f))
    if not files:
        raise FileNotFoundError(f"no shard matches {pattern!r}")
    toks = np.concatenate([np.asarray(open_shard(f)) for f in files])
    if max_tokens is not None:
        toks = toks[: max_tokens + 1]
    usable = ((toks.shape[0] - 1) // seq_len) * seq_len
    if usable <= 0:
        raise ShardError(f"validation split is shorter than one sequence of {seq_len}")
    return toks[: usable + 1]


def _main(argv=None) -> int:
    """``python -m parameter_golf_b200.data.shards --root DIR [--vocab 1024] [--train-tokens N] [--val-tokens N] [--train-shards K] [--seed S]``:
    write the seeded Zipf/Markov dataset (stand-in for the reference's FineWeb download and tokenisation tooling, ``data/``)."""
    import argparse
    ap = argparse.ArgumentParser(prog="parameter_golf_b200.data.shards")
    ap.add_argument("--root", required=True)
    ap.add_argument("--vocab", type=int, default=1024)
    ap.add_argument("--train-tokens", type=int, default=1 << 24)
    ap.add_argument("--val-tokens", type=int, default=1 << 20)
    ap.add_argument("--train-shards", type=int, default=1)
    ap.add_argument("--seed", type=int, default=1337)
    a = ap.parse_args(argv)
    write_synthetic_dataset(a.root, a.vocab, a.train_tokens, a.val_tokens, a.train_shards, a.seed)
    print(f"wrote {a.train_shards} training shard(s) of {a.train_tokens // max(a.train_shards, 1)} tokens and {a.val_tokens} validation tokens under {a.root}")
    return 0


if __name__ == "__main__":
    raise SystemExit(_main())
