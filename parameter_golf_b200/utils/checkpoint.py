"""Full training-state checkpoint (a superset of the reference, whose only persisted state is the
final artifact, ``parameter-golf-rs/crates/pg-train/src/lib.rs:1559-1576``): fp32 parameters, Muon momentum,
Adam moments, EMA shadow, step, loader position, RNG state and the variant fingerprint. Written
atomically (temp file + rename) so a crash mid-write never leaves a truncated checkpoint, and
guarded by a CRC32 of the payload."""
from __future__ import annotations

import io
import os
import struct
import zlib
from typing import Dict, Optional

import torch

MAGIC = b"PGCK"


def save_checkpoint(path: str, fingerprint: str, step: int, params: Dict[str, torch.Tensor], optim_state: dict,
                    loader_state: dict, ema_shadow: Optional[Dict[str, torch.Tensor]] = None) -> None:
    buf = io.BytesIO()
    torch.save({"fingerprint": fingerprint, "step": step,
                "params": {k: v.detach().cpu() for k, v in params.items()},
                "optim": optim_state, "loader": loader_state,
                "ema": None if ema_shadow is None else {k: v.detach().cpu() for k, v in ema_shadow.items()},
                "rng": torch.get_rng_state()}, buf)
    payload = buf.getvalue()
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(MAGIC + struct.pack("<QI", len(payload), zlib.crc32(payload) & 0xFFFFFFFF) + payload)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def load_checkpoint(path: str) -> dict:
    with open(path, "rb") as f:
        head = f.read(16)
        if len(head) < 16 or head[:4] != MAGIC:
            raise ValueError(f"{path}: not a training checkpoint")
        size, crc = struct.unpack("<QI", head[4:])
        payload = f.read(size)
    if len(payload) != size or zlib.crc32(payload) & 0xFFFFFFFF != crc:
        raise ValueError(f"{path}: checkpoint is truncated or corrupted")
    return torch.load(io.BytesIO(payload), map_location="cpu", weights_only=False)
