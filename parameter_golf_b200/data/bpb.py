"""Bits-per-byte metric and byte-count tables.

``bytes(prev, tgt) = base_bytes[tgt] + (has_leading_space[tgt] and not is_boundary[prev])`` and
``bpb = (loss / ln 2) * (tokens / bytes)``
(``parameter-golf-rs/crates/pg-data/src/bpb.rs:106-124``; Python twin ``train_gpt.py:180-204,263-278``).

Three table sources: a SentencePiece model/vocab (same rules as the reference), a placeholder of
4 bytes per token (``bpb.rs:30-36``), and a seeded synthetic table of 1..6 bytes per token for runs on
synthetic data.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np


@dataclass
class BpbLuts:
    base_bytes: np.ndarray          # int16 [V]
    has_leading_space: np.ndarray   # bool  [V]
    is_boundary: np.ndarray         # bool  [V]
    sidecar: "np.ndarray | None" = None   # float32 [tokens]: bytes of the token at each validation position, when given

    @staticmethod
    def placeholder(vocab: int) -> "BpbLuts":
        return BpbLuts(np.full(vocab, 4, np.int16), np.zeros(vocab, bool), np.zeros(vocab, bool))

    @staticmethod
    def seeded(vocab: int, seed: int = 20240520, lo: int = 1, hi: int = 6) -> "BpbLuts":
        rng = np.random.default_rng(seed)
        return BpbLuts(rng.integers(lo, hi + 1, size=vocab).astype(np.int16), np.zeros(vocab, bool), np.zeros(vocab, bool))

    @staticmethod
    def from_pieces(pieces: list, vocab: int, control: set = frozenset(), byte_ids: set = frozenset()) -> "BpbLuts":
        """``pieces[i]`` is the text of token ``i``. Control/unknown/unused ids count 0 bytes and are
        boundaries; ``<0xNN>`` byte pieces count 1; others count their UTF-8 length without the
        leading ``▁`` which instead sets ``has_leading_space``."""
        n = max(vocab, len(pieces))
        base = np.zeros(n, np.int16)
        lead = np.zeros(n, bool)
        bound = np.ones(n, bool)
        for i, piece in enumerate(pieces):
            if i in control:
                continue
            bound[i] = False
            if i in byte_ids or (len(piece) == 6 and piece.startswith("<0x") and piece.endswith(">")):
                base[i] = 1
                continue
            if piece.startswith("▁"):
                lead[i] = True
                piece = piece[1:]
            base[i] = len(piece.encode("utf-8"))
        return BpbLuts(base, lead, bound)

    @staticmethod
    def from_sentencepiece(model_file: str, vocab: int) -> "BpbLuts":
        import sentencepiece as spm
        sp = spm.SentencePieceProcessor(model_file=model_file)
        n = int(sp.vocab_size())
        control = {i for i in range(n) if sp.is_control(i) or sp.is_unknown(i) or sp.is_unused(i)}
        byte_ids = {i for i in range(n) if sp.is_byte(i)}
        return BpbLuts.from_pieces([sp.id_to_piece(i) for i in range(n)], vocab, control, byte_ids)

    def with_sidecar(self, bytes_per_position: np.ndarray) -> "BpbLuts":
        """Byte counts read from a sidecar aligned one-to-one with the validation tokens (CaseOps / SP8192 validation,
        ``pg-data/src/token_stream.rs:354-369``) instead of derived from token surfaces."""
        return BpbLuts(self.base_bytes, self.has_leading_space, self.is_boundary, np.asarray(bytes_per_position, dtype=np.float32))

    def token_bytes(self, prev_ids: np.ndarray, tgt_ids: np.ndarray, positions: "np.ndarray | None" = None) -> np.ndarray:
        """Bytes of each target token. ``positions`` are the targets' indices in the validation stream; they select
        from the sidecar when one is attached."""
        if self.sidecar is not None:
            if positions is None:
                raise ValueError("a byte sidecar is attached: token positions are required")
            return self.sidecar[np.asarray(positions, dtype=np.int64)].astype(np.float64)
        b = self.base_bytes[tgt_ids].astype(np.int64)
        b += (self.has_leading_space[tgt_ids] & ~self.is_boundary[prev_ids]).astype(np.int64)
        return b


def compute_bpb(loss_sum_nats: float, token_count: float, byte_count: float) -> tuple:
    """Return (mean loss in nats, bits per byte)."""
    val_loss = loss_sum_nats / max(token_count, 1.0)
    return val_loss, (val_loss / math.log(2.0)) * (token_count / max(byte_count, 1.0))
