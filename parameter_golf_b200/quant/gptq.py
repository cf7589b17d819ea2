"""Full-Hessian GPTQ with act-order, block error feedback and a per-row clip search.

Algorithm (``records/track_10min_16mb/2026-03-25_ValCalib_GPTQ_XSA_BigramHash3072/train_gpt.py:1104-1224``):
Hessians ``H = X^T X`` of every linear layer's input, averaged over calibration batches, 1 % mean-diagonal
damping; columns permuted by descending ``diag(H)``; ``U = chol(inv(H))`` upper; columns are quantised
left to right, the scaled error of column ``i`` is pushed into the not-yet-quantised columns through
``U[i, i:]``, block by block; five percentile clips are tried. Differences from the record, on purpose:
the integer range and rounding are the artifact's (``[-2^(b-1), 2^(b-1)-1]``, ties away from zero), and the
best clip is chosen per row (scales are per row) instead of per matrix.

Rows are independent given ``U``, which is what the CUDA kernel exploits (one CTA per row); this file
is the torch statement of the same computation and its oracle.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..models.gpt import bank_views
from ..spec import RunSpec
from .quantize import CLIP_PERCENTILES, GROUPS, qrange, quantize_rows, round_half_away, scheme_bits


def damp_hessian(H: torch.Tensor, damping: float = 0.01) -> torch.Tensor:
    H = H.float().clone()
    d = torch.diagonal(H)
    dead = d == 0
    d[dead] = 1.0
    d += damping * d.mean().clamp_min(1e-6)
    return H


def gptq_prepare(H: torch.Tensor, damping: float = 0.01):
    """Return (perm, inv_perm, U) with ``U`` the upper Cholesky factor of ``inv(H[perm][:, perm])``."""
    Hd = damp_hessian(H, damping)
    perm = torch.argsort(torch.diagonal(Hd), descending=True)
    Hp = Hd[perm][:, perm].double()
    L = torch.linalg.cholesky(Hp)
    Hinv = torch.cholesky_inverse(L)
    U = torch.linalg.cholesky(Hinv, upper=True).float()
    return perm, torch.argsort(perm), U


def gptq_rows_torch(Wp: torch.Tensor, U: torch.Tensor, scales: torch.Tensor, bits: int, block: int = 128) -> torch.Tensor:
    """Quantise the (already permuted) rows ``Wp`` with fixed per-row ``scales``; returns int8 codes."""
    qmin, qmax = qrange(bits)
    rows, cols = Wp.shape
    W = Wp.clone()
    Q = torch.zeros_like(W, dtype=torch.int8)
    s = scales[:, None]
    for i1 in range(0, cols, block):
        i2 = min(i1 + block, cols)
        W1 = W[:, i1:i2].clone()
        Err = torch.zeros_like(W1)
        U1 = U[i1:i2, i1:i2]
        for i in range(i2 - i1):
            w = W1[:, i:i + 1]
            q = round_half_away(w / s).clamp_(qmin, qmax)
            Q[:, i1 + i] = q[:, 0].to(torch.int8)
            err = (w - q * s) / U1[i, i]
            W1[:, i:] -= err * U1[i:i + 1, i:]
            Err[:, i] = err[:, 0]
        if i2 < cols:
            W[:, i2:] -= Err @ U[i1:i2, i2:]
    return Q


def gptq_quantize(W: torch.Tensor, H: torch.Tensor, bits: int = 6, block: int = 128, damping: float = 0.01,
                  rows_fn: Optional[Callable] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(q int8 [rows, cols], scale f32 [rows]). ``rows_fn`` substitutes the CUDA row kernel."""
    W = W.float()
    rows, cols = W.shape
    qmin, qmax = qrange(bits)
    perm, inv_perm, U = gptq_prepare(H.to(W.device), damping)
    Wp = W[:, perm].contiguous()
    srt = W.abs().sort(dim=1).values
    if rows_fn is None:
        if W.is_cuda and block == 128:
            from ..ops import native                  # on a GPU the hand-written row kernel is the path; no silent fallback
            rows_fn = native.gptq_rows
        else:
            rows_fn = gptq_rows_torch
    best_err = torch.full((rows,), float("inf"), device=W.device)
    best_q = torch.zeros_like(Wp, dtype=torch.int8)
    best_s = torch.ones(rows, device=W.device)
    for p in CLIP_PERCENTILES:
        idx = min(int(cols * p), cols - 1)
        scale = (srt[:, idx].clamp_min(1e-8) / qmax).clamp_min(1e-8)
        scale = scale.half().float().clamp_min(6e-8)          # what de-quantisation will multiply by
        Q = rows_fn(Wp, U, scale, bits, block)
        err = (Wp - Q.float() * scale[:, None]).pow(2).sum(1)
        better = err < best_err
        best_err = torch.where(better, err, best_err)
        best_s = torch.where(better, scale, best_s)
        best_q[better] = Q[better]
    return best_q[:, inv_perm].contiguous(), best_s


class HessianTaps:
    """Accumulates ``X^T X`` of the inputs of every linear layer, keyed ``(layer, site)`` with site in
    ``qkv | o | up | down``; plugged into the oracle forward through ``block_forward(..., taps=...)``."""

    def __init__(self):
        self.H: Dict[Tuple[int, str], torch.Tensor] = {}
        self.batches = 0

    def add(self, layer: int, site: str, x: torch.Tensor):
        x = x.detach().reshape(-1, x.shape[-1]).float()
        h = x.t() @ x
        key = (layer, site)
        if key in self.H:
            self.H[key] += h
        else:
            self.H[key] = h

    def finish(self) -> Dict[Tuple[int, str], torch.Tensor]:
        n = max(self.batches, 1)
        return {k: v / n for k, v in self.H.items()}


GROUP_SITES = {"qo_bank.q": "qkv", "kv_bank.k": "qkv", "kv_bank.v": "qkv", "qo_bank.o": "o", "mlp_up_bank": "up", "mlp_down_bank": "down"}


def gptq_quantize_model(spec: RunSpec, params: Dict[str, torch.Tensor], hessians: Dict[Tuple[int, str], torch.Tensor],
                        rows_fn: Optional[Callable] = None, device=None) -> Dict[str, Tuple[torch.Tensor, torch.Tensor]]:
    """Quantise every bank group layer by layer with its Hessian; ``tok_emb`` uses the plain clip search.
    Returns the ``precomputed`` map accepted by `export_model`."""
    m, q = spec.model, spec.quant
    bits = scheme_bits(q.scheme, q.matrix_bits, q.embed_bits)
    views = bank_views(m, params)
    out = {}
    for g in GROUPS:
        W = views[g].detach().float()
        if device is not None:
            W = W.to(device)
        if g == "tok_emb":
            qq, ss = (W.half(), torch.ones(W.shape[0])) if bits[g] == 16 else quantize_rows(W, bits[g])     # 16: the table stays fp16
            out[g] = (qq.cpu(), ss.cpu())
            continue
        per = W.shape[0] // m.num_layers
        qs, ss = [], []
        for i in range(m.num_layers):
            H = hessians[(i, GROUP_SITES[g])]
            qi, si = gptq_quantize(W[i * per:(i + 1) * per], H.to(W.device), bits[g], q.gptq_block_size, q.gptq_damping, rows_fn)
            qs.append(qi.cpu())
            ss.append(si.cpu())
        out[g] = (torch.cat(qs), torch.cat(ss))
    return out
