"""Binary (1-bit) weight quantisation, the export idea of the non-record submission
``records/track_non_record_16mb/2026-03-24_106M_Binary_Asymmetric_UNet_FP8_15L_8192BPE_YaRN_NeoMuon_Smear``
(``train_gpt_cuda_binary.py:186-208`` export, ``:221-232`` load, ``:417-428`` the layer's straight-through form): weights in
{-1, +1}, one absmean scale per group of input columns, one bit per weight, LZMA on top.

* a row is cut into groups of ``group`` columns (the tail group of a row whose width is no multiple is shorter; its scale is
  the mean over the columns that exist); ``s = mean(|w|)`` per group, never below 1e-8; ``q = +1`` where ``w >= 0`` else ``-1``.
  With no zero code the absmean is already the scale that minimises ``||w - s q||^2`` for that ``q``, so there is no
  correction step as in the ternary scheme;
* packing: bit ``(q + 1) / 2``, eight per byte, element ``i`` in bit ``i mod 8`` of byte ``i / 8`` (least significant bit
  first, the order the submission's ``pack_binary`` uses, ``:117-127``), the tail padded with zero bits; scales are fp16.
"""
from __future__ import annotations

from typing import Tuple

import numpy as np
import torch


def quantize_binary(w: torch.Tensor, group: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(q int8 [rows, cols] in {-1, +1}, scale fp32 [rows, ceil(cols / group)])``."""
    if w.ndim != 2:
        raise ValueError("binary quantisation takes a matrix")
    rows, cols = w.shape
    ng = -(-cols // group)
    pad = ng * group - cols
    wp = torch.nn.functional.pad(w.float(), (0, pad)).reshape(rows, ng, group)
    cnt = torch.full((ng,), float(group))
    if pad:
        cnt[-1] = group - pad
    s = (wp.abs().sum(-1) / cnt[None, :]).clamp_min(1e-8)
    q = torch.where(w.float() >= 0, 1, -1).to(torch.int8)
    return q.contiguous(), s.contiguous()


def dequantize_binary(q: torch.Tensor, scale: torch.Tensor, group: int = 128) -> torch.Tensor:
    cols = q.shape[1]
    return q.float() * scale.float().repeat_interleave(group, dim=1)[:, :cols]


def pack_signs(q: np.ndarray) -> bytes:
    a = np.asarray(q, dtype=np.int8).reshape(-1)
    if a.size and not np.all((a == 1) | (a == -1)):
        raise ValueError("binary codes must be -1 or +1")
    return np.packbits((a > 0).astype(np.uint8), bitorder="little").tobytes()


def unpack_signs(data: bytes, count: int) -> np.ndarray:
    b = np.frombuffer(data, dtype=np.uint8)
    if b.size * 8 < count:
        raise ValueError("bit stream shorter than the element count")
    bits = np.unpackbits(b, count=count, bitorder="little")
    return bits.astype(np.int8) * 2 - 1
