"""Ternary (BitNet b1.58) weight quantisation with base-3 packing, the export idea of the record
``records/track_10min_16mb/2026-03-24_74M_Ternary_UNet_FP8_10L_8192BPE_YaRN_NeoMuon`` (its README: weights in
{-1, 0, +1}, per-group (128) absmean scaling, 5 trits per byte, LZMA preset 9, and a scale correction for the fraction of
zeros; ``train_gpt_cuda_ternary.py:186-260`` is its export). The statements below are this framework's own form of it:

* a row is cut into groups of ``group`` columns; ``s = mean(|w|)`` per group; ``q = clamp(round(w / s), -1, 1)``;
* *shrinkage fix*: after rounding, the scale that minimises ``||w - s q||^2`` for the chosen ``q`` is
  ``s* = sum(|w| [q != 0]) / count(q != 0)``; using the absmean of ALL entries instead biases the reconstruction low by
  the fraction of zeros. ``fix_scale=True`` (default) stores ``s*``;
* packing: ``t = q + 1`` in {0, 1, 2}, five trits per byte as ``t0 + 3 t1 + 9 t2 + 27 t3 + 81 t4`` (< 243), tail padded
  with ones (q = 0); scales are stored as fp16;
* container: ``PGT3`` + u32 rows + u32 cols + u32 group, packed trits, scales; `compress` wraps it in one xz stream.
"""
from __future__ import annotations

import lzma
import struct
from typing import Tuple

import numpy as np
import torch

MAGIC = b"PGT3"
_POW3 = np.array([1, 3, 9, 27, 81], dtype=np.uint16)


def quantize_ternary(w: torch.Tensor, group: int = 128, fix_scale: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(q int8 [rows, cols] in {-1, 0, 1}, scale fp32 [rows, ceil(cols / group)])``."""
    if w.ndim != 2:
        raise ValueError("ternary quantisation takes a matrix")
    rows, cols = w.shape
    ng = -(-cols // group)
    pad = ng * group - cols
    wp = torch.nn.functional.pad(w.float(), (0, pad)).reshape(rows, ng, group)
    valid = torch.ones(rows, ng * group, dtype=torch.bool)
    if pad:
        valid[:, cols:] = False
    valid = valid.reshape(rows, ng, group)
    cnt = valid.sum(-1).clamp_min(1)
    s = (wp.abs() * valid).sum(-1) / cnt
    s = s.clamp_min(1e-12)
    q = torch.clamp(torch.round(wp / s[..., None]), -1, 1) * valid
    if fix_scale:
        nz = (q != 0)
        s_fix = (wp.abs() * nz).sum(-1) / nz.sum(-1).clamp_min(1)
        s = torch.where(nz.any(-1), s_fix, s)
    return q.reshape(rows, ng * group)[:, :cols].to(torch.int8).contiguous(), s.contiguous()


def dequantize_ternary(q: torch.Tensor, scale: torch.Tensor, group: int = 128) -> torch.Tensor:
    rows, cols = q.shape
    s = scale.float().repeat_interleave(group, dim=1)[:, :cols]
    return q.float() * s


def pack_trits(q: np.ndarray) -> bytes:
    t = (np.asarray(q, dtype=np.int8).reshape(-1) + 1).astype(np.uint16)
    if t.size and (t.min() < 0 or t.max() > 2):
        raise ValueError("ternary codes must be -1, 0 or 1")
    pad = (-t.size) % 5
    if pad:
        t = np.concatenate([t, np.ones(pad, dtype=np.uint16)])
    return (t.reshape(-1, 5) * _POW3).sum(axis=1).astype(np.uint8).tobytes()


def unpack_trits(data: bytes, count: int) -> np.ndarray:
    b = np.frombuffer(data, dtype=np.uint8).astype(np.uint16)
    if b.size * 5 < count:
        raise ValueError("trit stream shorter than the element count")
    if b.size and b.max() >= 243:
        raise ValueError("byte outside the base-3 range")
    out = np.empty((b.size, 5), dtype=np.int8)
    for i in range(5):
        out[:, i] = (b % 3).astype(np.int8) - 1
        b = b // 3
    return out.reshape(-1)[:count]


def serialize(q: torch.Tensor, scale: torch.Tensor, group: int = 128) -> bytes:
    rows, cols = q.shape
    return (MAGIC + struct.pack("<III", rows, cols, group) + pack_trits(q.numpy()) +
            scale.to(torch.float16).numpy().astype("<f2").tobytes())


def deserialize(raw: bytes) -> Tuple[torch.Tensor, torch.Tensor, int]:
    if raw[:4] != MAGIC:
        raise ValueError("not a ternary container")
    rows, cols, group = struct.unpack_from("<III", raw, 4)
    nt = -(-(rows * cols) // 5)
    ng = -(-cols // group)
    need = 16 + nt + 2 * rows * ng
    if len(raw) != need:
        raise ValueError(f"ternary container: expected {need} bytes, got {len(raw)}")
    q = torch.from_numpy(unpack_trits(raw[16:16 + nt], rows * cols).copy()).reshape(rows, cols)
    s = torch.from_numpy(np.frombuffer(raw, dtype="<f2", count=rows * ng, offset=16 + nt).astype(np.float32)).reshape(rows, ng)
    return q, s, group


def compress(q: torch.Tensor, scale: torch.Tensor, group: int = 128) -> bytes:
    return lzma.compress(serialize(q, scale, group), format=lzma.FORMAT_XZ, preset=9)


def decompress(blob: bytes) -> torch.Tensor:
    q, s, group = deserialize(lzma.decompress(blob, format=lzma.FORMAT_XZ))
    return dequantize_ternary(q, s, group)


def bits_per_param(q: torch.Tensor, scale: torch.Tensor, group: int = 128) -> float:
    return 8.0 * len(compress(q, scale, group)) / q.numel()
