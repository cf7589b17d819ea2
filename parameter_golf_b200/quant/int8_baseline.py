"""The baseline trainer's export: per-row int8 + zlib level 9, and its round trip.

Same rules as ``train_gpt.py:296-422`` (`quantize_float_tensor`, `quantize_state_dict_int8`,
`dequantize_state_dict_int8`) and the export / reload / re-evaluate sequence at ``:1076-1119``:

* a 2-D float tensor gets one scale per row: ``clip = quantile(|w|, 0.9999984)`` per row,
  ``scale = max(clip / 127, 1 / 127)``, ``q = clamp(round(clamp(w, ±clip) / scale), ±127)``, scale stored as fp16;
* any other float tensor gets one scale for the whole tensor (fp32);
* tensors of at most 65,536 elements are not quantised: stored as fp16, or fp32 when their name contains one of the
  control patterns (`attn_scale`, `mlp_scale`, `resid_mix`, `q_gain`, `skip_weight`);
* non-float tensors pass through unchanged.

The reference pickles the resulting dict with ``torch.save`` and compresses that with zlib; here the dict is written as
a small self-describing container (JSON header + raw little-endian buffers) before the same ``zlib.compress(level=9)``, so
no pickle is needed to read an artifact. The 3-D parameter banks of this framework are quantised per matrix row, which is
what the reference's per-layer 2-D weights amount to.
"""
from __future__ import annotations

import json
import struct
import zlib
from typing import Dict, Tuple

import numpy as np
import torch

KEEP_FLOAT_MAX_NUMEL = 65_536
CLIP_Q = 99.99984 / 100.0
CONTROL_PATTERNS = ("attn_scale", "attn_scales", "mlp_scale", "mlp_scales", "resid_mix", "resid_mixes", "q_gain", "skip_weight",
                    "skip_weights")
FORMAT = "int8_clean_per_row_v1"
MAGIC = b"PGI8"


def _row_quantile(a: torch.Tensor, q: float) -> torch.Tensor:
    """``torch.quantile(a, q, dim=1)`` (linear interpolation) without its 16 M element limit."""
    n = a.shape[1]
    pos = q * (n - 1)
    lo = int(np.floor(pos))
    hi = min(lo + 1, n - 1)
    top = torch.topk(a, n - lo, dim=1, largest=True, sorted=True).values       # descending: [:, -1] is order statistic `lo`
    v_lo = top[:, -1]
    v_hi = top[:, -2] if hi > lo else v_lo
    return v_lo + (v_hi - v_lo) * (pos - lo)


def quantize_float_tensor(t: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    t32 = t.float()
    if t32.ndim >= 2:
        rows = t32.reshape(-1, t32.shape[-1])
        clip = _row_quantile(rows.abs(), CLIP_Q) if rows.numel() else torch.empty(rows.shape[0])
        clipped = torch.maximum(torch.minimum(rows, clip[:, None]), -clip[:, None])
        scale = (clip / 127.0).clamp_min(1.0 / 127.0)
        q = torch.clamp(torch.round(clipped / scale[:, None]), -127, 127).to(torch.int8)
        return q.reshape(t32.shape).contiguous(), scale.to(torch.float16).reshape(t32.shape[:-1]).contiguous()
    flat = t32.abs().flatten()
    clip = float(_row_quantile(flat[None, :], CLIP_Q)[0]) if flat.numel() else 0.0
    scale = torch.tensor(clip / 127.0 if clip > 0 else 1.0, dtype=torch.float32)
    q = torch.clamp(torch.round(torch.clamp(t32, -clip, clip) / scale), -127, 127).to(torch.int8).contiguous()
    return q, scale


def coarsen_bank_codes(name: str, q: torch.Tensor, layers, step: int, num_layers: int) -> torch.Tensor:
    """Round the int8 codes of the listed blocks to multiples of ``step`` (4 leaves 64 levels, 16 leaves 16): the entropy coder
    then spends fewer bits on those blocks (records/track_10min_16mb/2026-03-19_10L_MixedPrecision/train_gpt.py:1089-1101, which
    picks the middle blocks). Works on the stacked banks: slot ``s`` of ``qo_bank`` / ``kv_bank`` belongs to block ``s mod n``."""
    if step <= 1 or not layers or name not in ("qo_bank", "kv_bank", "mlp_up_bank", "mlp_down_bank"):
        return q
    q = q.clone()
    for slot in range(q.shape[0]):
        if slot % num_layers in layers:
            q[slot] = (torch.round(q[slot].float() / step) * step).clamp(-127, 127).to(torch.int8)
    return q


def quantize_state_dict_int8(state: Dict[str, torch.Tensor], keep_fp16=(), coarse_layers=(), coarse_step: int = 1, num_layers: int = 0):
    """Returns ``(obj, stats)``; ``obj`` has the reference's keys (`quantized`, `scales`, `dtypes`, `passthrough`,
    `passthrough_orig_dtypes`, `qmeta`, `__quant_format__`). ``keep_fp16``: names stored as fp16 whatever their size (the tied
    embedding of records/track_10min_16mb/2026-03-18_FP16Embed_WD3600, whose int8 error enters at both ends of the model)."""
    obj = {"__quant_format__": FORMAT, "quantized": {}, "scales": {}, "dtypes": {}, "passthrough": {}, "passthrough_orig_dtypes": {},
           "qmeta": {}}
    stats = {"param_count": 0, "num_tensors": 0, "baseline_tensor_bytes": 0, "int8_payload_bytes": 0}
    for name, tensor in state.items():
        t = tensor.detach().cpu().contiguous()
        stats["param_count"] += t.numel()
        stats["num_tensors"] += 1
        stats["baseline_tensor_bytes"] += t.numel() * t.element_size()
        if not t.is_floating_point():
            obj["passthrough"][name] = t
            stats["int8_payload_bytes"] += t.numel() * t.element_size()
            continue
        if t.numel() <= KEEP_FLOAT_MAX_NUMEL or name in keep_fp16:
            if any(p in name for p in CONTROL_PATTERNS):
                kept = t.float().contiguous()
            elif t.dtype in (torch.float32, torch.bfloat16):
                obj["passthrough_orig_dtypes"][name] = str(t.dtype).removeprefix("torch.")
                kept = t.to(torch.float16).contiguous()
            else:
                kept = t
            obj["passthrough"][name] = kept
            stats["int8_payload_bytes"] += kept.numel() * kept.element_size()
            continue
        q, s = quantize_float_tensor(t)
        q = coarsen_bank_codes(name, q, set(int(l) for l in coarse_layers), coarse_step, num_layers)
        if s.ndim > 0:
            obj["qmeta"][name] = {"scheme": "per_row", "axis": 0}
        obj["quantized"][name], obj["scales"][name] = q, s
        obj["dtypes"][name] = str(t.dtype).removeprefix("torch.")
        stats["int8_payload_bytes"] += q.numel() + s.numel() * s.element_size()
    return obj, stats


def dequantize_state_dict_int8(obj) -> Dict[str, torch.Tensor]:
    if obj.get("__quant_format__") != FORMAT:
        raise ValueError(f"unknown int8 export format {obj.get('__quant_format__')!r}")
    out: Dict[str, torch.Tensor] = {}
    for name, q in obj["quantized"].items():
        dtype = getattr(torch, obj["dtypes"][name])
        s = obj["scales"][name]
        if obj["qmeta"].get(name, {}).get("scheme") == "per_row" or s.ndim > 0:
            out[name] = (q.float() * s.float().reshape(*q.shape[:-1], 1)).to(dtype).contiguous()
        else:
            out[name] = (q.float() * float(s)).to(dtype).contiguous()
    for name, t in obj["passthrough"].items():
        orig = obj["passthrough_orig_dtypes"].get(name)
        out[name] = t.to(getattr(torch, orig)).contiguous() if orig else t.clone()
    return out


# ---- container + zlib --------------------------------------------------------------------------------------------------
_NP = {"int8": "i1", "float16": "<f2", "float32": "<f4", "int32": "<i4", "int64": "<i8", "bfloat16": None, "uint8": "u1", "bool": "?"}


def _to_bytes(t: torch.Tensor) -> Tuple[str, bytes]:
    name = str(t.dtype).removeprefix("torch.")
    if name == "bfloat16":
        return name, t.contiguous().view(torch.int16).numpy().astype("<i2").tobytes()
    return name, t.contiguous().numpy().astype(_NP[name]).tobytes()


def _from_bytes(dtype: str, shape, data: bytes) -> torch.Tensor:
    if dtype == "bfloat16":
        return torch.from_numpy(np.frombuffer(data, dtype="<i2").copy()).view(torch.bfloat16).reshape(shape)
    return torch.from_numpy(np.frombuffer(data, dtype=_NP[dtype]).copy()).reshape(shape)


def serialize(obj) -> bytes:
    """``PGI8`` + u32 header length + JSON header + concatenated raw buffers (offsets in the header)."""
    header = {"format": obj["__quant_format__"], "dtypes": obj["dtypes"], "qmeta": obj["qmeta"],
              "passthrough_orig_dtypes": obj["passthrough_orig_dtypes"], "tensors": []}
    body = bytearray()
    for section in ("quantized", "scales", "passthrough"):
        for name, t in obj[section].items():
            dt, raw = _to_bytes(t)
            header["tensors"].append({"section": section, "name": name, "dtype": dt, "shape": list(t.shape), "offset": len(body),
                                      "nbytes": len(raw)})
            body += raw
    h = json.dumps(header, separators=(",", ":")).encode()
    return MAGIC + struct.pack("<I", len(h)) + h + bytes(body)


def deserialize(raw: bytes):
    if raw[:4] != MAGIC:
        raise ValueError("not an int8 baseline container")
    (hl,) = struct.unpack_from("<I", raw, 4)
    header = json.loads(raw[8:8 + hl])
    body = memoryview(raw)[8 + hl:]
    obj = {"__quant_format__": header["format"], "dtypes": header["dtypes"], "qmeta": header["qmeta"],
           "passthrough_orig_dtypes": header["passthrough_orig_dtypes"], "quantized": {}, "scales": {}, "passthrough": {}}
    for rec in header["tensors"]:
        data = bytes(body[rec["offset"]: rec["offset"] + rec["nbytes"]])
        if len(data) != rec["nbytes"]:
            raise ValueError(f"int8 container truncated at tensor {rec['name']!r}")
        obj[rec["section"]][rec["name"]] = _from_bytes(rec["dtype"], rec["shape"], data)
    return obj


def export_int8_zlib(state: Dict[str, torch.Tensor], path: str = None, keep_fp16=(), coarse_layers=(), coarse_step: int = 1, num_layers: int = 0):
    """Quantise, serialise and compress; returns ``(blob, stats)`` with the byte counts the baseline logs."""
    obj, stats = quantize_state_dict_int8(state, keep_fp16, coarse_layers, coarse_step, num_layers)
    raw = serialize(obj)
    blob = zlib.compress(raw, level=9)
    stats.update(raw_bytes=len(raw), compressed_bytes=len(blob),
                 payload_ratio=stats["baseline_tensor_bytes"] / max(stats["int8_payload_bytes"], 1))
    if path:
        with open(path, "wb") as f:
            f.write(blob)
    return blob, stats


def load_int8_zlib(blob: bytes) -> Dict[str, torch.Tensor]:
    return dequantize_state_dict_int8(deserialize(zlib.decompress(blob)))
