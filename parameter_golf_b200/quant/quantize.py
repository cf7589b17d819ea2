"""Per-row integer quantisation with percentile clip search, pruning masks, LQER residual factors.

Quantiser rule (``parameter-golf-rs/crates/pg-quant/src/scheme.rs:30-57,260-304``): for each row sort
``|x|``; for each ``p`` in {.999, .9995, .9999, .99999, 1.0}: ``idx = min(floor(n*p), n-1)``,
``clip = max(sorted[idx], 1e-8)``, ``scale = max(clip/qmax, 1e-8)``,
``q = clamp(round_half_away(x/scale), qmin, qmax)`` with ``qmax = 2^(b-1)-1``, ``qmin = -2^(b-1)``;
the first ``p`` with the strictly smallest squared error wins. Scales are stored as f16 and
de-quantisation multiplies by the f16-rounded value (``pg-quant/src/export.rs:372-383,967-985``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

CLIP_PERCENTILES = (0.999, 0.9995, 0.9999, 0.99999, 1.0)


def qrange(bits: int) -> Tuple[int, int]:
    return -(1 << (bits - 1)), (1 << (bits - 1)) - 1


def round_half_away(x: torch.Tensor) -> torch.Tensor:
    """Rust ``f32::round`` semantics (ties away from zero); ``torch.round`` is ties-to-even."""
    return torch.sign(x) * torch.floor(x.abs() + 0.5)


def quantize_rows(w: torch.Tensor, bits: int, percentiles=CLIP_PERCENTILES) -> Tuple[torch.Tensor, torch.Tensor]:
    """Return (q int8 [rows, cols], scale f32 [rows]) using the clip search above."""
    w = w.float()
    rows, n = w.shape
    qmin, qmax = qrange(bits)
    srt = w.abs().sort(dim=1).values
    best_err = torch.full((rows,), float("inf"), device=w.device)
    best_q = torch.zeros_like(w, dtype=torch.int8)
    best_s = torch.ones(rows, device=w.device)
    for p in percentiles:
        idx = min(int(n * p), n - 1)
        clip = srt[:, idx].clamp_min(1e-8)
        scale = (clip / qmax).clamp_min(1e-8)
        q = round_half_away(w / scale[:, None]).clamp_(qmin, qmax)
        err = (w - q * scale[:, None]).pow(2).sum(1)
        better = err < best_err
        best_err = torch.where(better, err, best_err)
        best_s = torch.where(better, scale, best_s)
        best_q[better] = q[better].to(torch.int8)
    return best_q, best_s


def dequantize_rows(q: torch.Tensor, scale_f16: torch.Tensor) -> torch.Tensor:
    return q.float() * scale_f16.float()[:, None]


def quantize_int6_legacy(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Legacy int6 path: i8 values in [-32, 31] with f16 row scales from the row max
    (``pg-quant/src/int6.rs:15-103``)."""
    w = w.float()
    scale = (w.abs().amax(1) / 31.0).clamp_min(1e-8)
    q = round_half_away(w / scale[:, None]).clamp_(-32, 31).to(torch.int8)
    return q, scale.half()


# ---- scheme -> bits per group -------------------------------------------------------------------------------

GROUPS = ("qo_bank.q", "qo_bank.o", "kv_bank.k", "kv_bank.v", "mlp_up_bank", "mlp_down_bank", "tok_emb")


def scheme_bits(scheme: str, matrix_bits: int = 6, embed_bits: int = 8) -> Dict[str, int]:
    """Bits per artifact group (``pg-quant/src/export.rs:224-277``). ``mixed_int5_int6`` in the reference
    uses ``matrix_bits`` for every matrix group; the int5-MLP/int6-attention split of the Python record
    (``records/track_10min_16mb/2026-03-20_10L_Int5MLP_MuonWD04_SWA50/train_gpt.py:334-367``) is what the
    name promises, so it is applied when ``matrix_bits`` is left at 6."""
    attn = ("qo_bank.q", "qo_bank.o", "kv_bank.k", "kv_bank.v")
    mlp = ("mlp_up_bank", "mlp_down_bank")
    if scheme in ("gptq_lite_int6", "full_gptq_int6", "none"):
        a = m = matrix_bits
        e = embed_bits
    elif scheme == "mixed_int5_int6":
        a, m, e = matrix_bits, (5 if matrix_bits == 6 else matrix_bits), embed_bits
    elif scheme == "aggressive":
        a, m, e = 8, 4, 8
    elif scheme == "tight_int7_int4":
        a, m, e = 7, 4, 8
    elif scheme == "ternary_b158":       # matrix groups are ternary codes (stored base-3, 1.6 bits each); the value is a marker
        a, m, e = 2, 2, embed_bits
    elif scheme == "binary_b1":          # matrix groups are sign codes, one bit each; the value is a marker
        a, m, e = 1, 1, embed_bits
    else:
        raise ValueError(f"unknown quant scheme {scheme!r}")
    out = {g: a for g in attn}
    out.update({g: m for g in mlp})
    out["tok_emb"] = e
    return out


# ---- pruning --------------------------------------------------------------------------------------------------

def prune_topk_per_row(w: torch.Tensor, keep_ratio: float) -> torch.Tensor:
    k = max(1, int(round(w.shape[1] * keep_ratio)))
    idx = w.abs().topk(k, dim=1).indices
    mask = torch.zeros_like(w, dtype=torch.bool)
    mask.scatter_(1, idx, True)
    return mask


def prune_global_magnitude(w: torch.Tensor, keep_ratio: float) -> torch.Tensor:
    k = max(1, int(round(w.numel() * keep_ratio)))
    thr = w.abs().flatten().kthvalue(w.numel() - k + 1).values
    return w.abs() >= thr


def prune_2_of_4(w: torch.Tensor) -> torch.Tensor:
    r, c = w.shape
    if c % 4:
        raise ValueError("2:4 pruning needs a column count divisible by 4")
    g = w.abs().reshape(r, c // 4, 4)
    idx = g.topk(2, dim=2).indices
    mask = torch.zeros_like(g, dtype=torch.bool)
    mask.scatter_(2, idx, True)
    return mask.reshape(r, c)


def prune_rows(w: torch.Tensor, keep_ratio: float, mode: str = "topk_per_row") -> torch.Tensor:
    """Masked copy of ``w`` (``pg-quant/src/prune.rs:41-54,108-232``)."""
    if mode == "topk_per_row":
        mask = prune_topk_per_row(w, keep_ratio)
    elif mode == "global_magnitude":
        mask = prune_global_magnitude(w, keep_ratio)
    elif mode == "2:4":
        mask = prune_2_of_4(w)
    else:
        raise ValueError(f"unknown prune mode {mode!r}")
    return w * mask


def prune_then_quantize(w: torch.Tensor, keep_ratio: float, bits: int, mode: str = "topk_per_row"):
    return quantize_rows(prune_rows(w, keep_ratio, mode), bits)


def ordering_ab_test(w: torch.Tensor, keep_ratio: float, bits: int) -> Dict[str, float]:
    """Reconstruction error of prune→quantise vs quantise→prune (``pg-quant/src/prune.rs:269-308``)."""
    q1, s1 = prune_then_quantize(w, keep_ratio, bits)
    e1 = (w - dequantize_rows(q1, s1.half())).pow(2).mean().item()
    q2, s2 = quantize_rows(w, bits)
    d2 = dequantize_rows(q2, s2.half()) * prune_topk_per_row(w, keep_ratio)
    e2 = (w - d2).pow(2).mean().item()
    return {"prune_then_quantize_mse": e1, "quantize_then_prune_mse": e2}


# ---- LQER ---------------------------------------------------------------------------------------------------------

@dataclass
class LqerFactors:
    a_q: torch.Tensor   # int8 [rows, r]
    a_s: torch.Tensor   # f16 [rows]
    b_q: torch.Tensor   # int8 [r, cols]
    b_s: torch.Tensor   # f16 [r]


def lqer_factors(residual: torch.Tensor, rank: int, a_bits: int = 8, b_bits: int = 8, iters: int = 12) -> LqerFactors:
    """Rank-``rank`` factors ``A B ≈ residual`` by block power iteration, each quantised per row
    (``pg-quant/src/export.rs:321-361,438-499``)."""
    r = min(rank, *residual.shape)
    g = torch.Generator().manual_seed(0)
    v = torch.randn(residual.shape[1], r, generator=g).to(residual)
    for _ in range(iters):
        u, _ = torch.linalg.qr(residual @ v)
        v, _ = torch.linalg.qr(residual.t() @ u)
    a = residual @ v            # [rows, r]
    b = v.t()                   # [r, cols]
    aq, as_ = quantize_rows(a, a_bits)
    bq, bs = quantize_rows(b, b_bits)
    return LqerFactors(aq, as_.half(), bq, bs.half())


def lqer_reconstruct(f: LqerFactors) -> torch.Tensor:
    return dequantize_rows(f.a_q, f.a_s) @ dequantize_rows(f.b_q, f.b_s)


# ---- ±1 pruning to a byte target ------------------------------------------------------------------------------------

def selective_prune_to_target(qs: Dict[str, torch.Tensor], scales: Dict[str, torch.Tensor], size_fn, target_bytes: int,
                              max_iters: int = 24, max_magnitude: int = 1) -> Tuple[Dict[str, torch.Tensor], int]:
    """Zero the cheapest ``|q| == 1`` entries (ordered by ``scale^2``, the squared error their removal
    adds) until ``size_fn(qs) <= target_bytes``, by bisection on the count
    (``records/track_10min_16mb/2026-03-25_ValCalib_GPTQ_XSA_BigramHash3072/train_gpt.py:1997-2040``).
    ``max_magnitude`` > 1 extends the candidates to ``|q| <= max_magnitude`` (cost ``(q * scale)^2``) when zeroing every
    +-1 is not enough: a barely trained model has near-uniform codes and few ones. Magnitudes are tried in turn, so a
    target that +-1 can reach is reached with +-1 only."""
    if size_fn(qs) <= target_bytes:
        return qs, 0
    result, used = qs, 0
    for mag in range(1, max(1, max_magnitude) + 1):
        cand = []
        for name, q in qs.items():
            idx = ((q.abs() <= mag) & (q != 0)).nonzero(as_tuple=False)
            if idx.numel():
                qv = q[idx[:, 0], idx[:, 1]].float()
                cost = (scales[name].float()[idx[:, 0]] * qv).pow(2)
                cand.append((name, idx, cost))
        if not cand:
            continue
        costs = torch.cat([c for _, _, c in cand])
        order = costs.argsort()
        owners = torch.cat([torch.full((c.numel(),), i) for i, (_, _, c) in enumerate(cand)])
        local = torch.cat([torch.arange(c.numel()) for _, _, c in cand])

        def apply(count: int):
            out = {k: v.clone() for k, v in qs.items()}
            sel = order[:count]
            for i, (name, idx, _) in enumerate(cand):
                pick = local[sel][owners[sel] == i]
                if pick.numel():
                    rc = idx[pick]
                    out[name][rc[:, 0], rc[:, 1]] = 0
            return out

        lo, hi = 0, costs.numel()
        result, used = apply(hi), hi
        if size_fn(result) > target_bytes:
            continue                                  # not enough at this magnitude: widen the candidate set
        for _ in range(max_iters):
            if hi - lo <= max(1, costs.numel() // 512):
                break
            mid = (lo + hi) // 2
            if size_fn(apply(mid)) <= target_bytes:
                hi = mid
            else:
                lo = mid
        return apply(hi), hi
    return result, used
    for _ in range(max_iters):
        if hi - lo <= max(1, costs.numel() // 512):
            break
        mid = (lo + hi) // 2
        if size_fn(apply(mid)) <= target_bytes:
            hi = mid
        else:
            lo = mid
    return apply(hi), hi
