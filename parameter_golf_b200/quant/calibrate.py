"""Self-generated calibration data and Hessian collection for GPTQ.

The trained model writes its own calibration set: ``num_seqs`` sequences of ``seq_len`` tokens sampled
autoregressively at temperature 0.8 from a random first token, seeded; no external data is read
(``records/track_10min_16mb/2026-03-25_ValCalib_GPTQ_XSA_BigramHash3072/train_gpt.py:1081-1102``). Hessians
``H = X^T X`` of every linear input are then accumulated over those sequences and averaged
(``…:1104-1138``). Generation uses a per-layer K/V cache so each new token costs one row of attention
instead of a full re-prefill.
"""
from __future__ import annotations

import math
from typing import Dict, Tuple

import torch
import torch.nn.functional as F

from ..models import gpt
from ..ops import reference as R
from ..spec import ModelSpec, RunSpec
from .gptq import HessianTaps


@torch.no_grad()
def generate_autoregressive(m: ModelSpec, p: Dict[str, torch.Tensor], num_seqs: int, seq_len: int, temperature: float = 0.8,
                            seed: int = 42, device="cpu", dtype=torch.float32) -> torch.Tensor:
    """[num_seqs, seq_len] int64 token ids sampled from the model with a K/V cache."""
    p = {k: v.to(device) for k, v in p.items()}
    g = torch.Generator(device=device).manual_seed(seed)
    n, H, Hkv, D, d = m.num_layers, m.num_heads, m.num_kv_heads, m.head_dim, m.model_dim
    rd = m.rope_dims
    cos, sin = R.model_rope_tables(m, seq_len, device=device)
    toks = torch.zeros(num_seqs, seq_len, dtype=torch.int64, device=device)
    toks[:, 0] = torch.randint(0, m.vocab_size, (num_seqs,), generator=g, device=device)
    kc = [torch.zeros(num_seqs, seq_len, Hkv, D, device=device, dtype=dtype) for _ in range(n)]
    vc = [torch.zeros(num_seqs, seq_len, Hkv, D, device=device, dtype=dtype) for _ in range(n)]
    enc = n // 2
    unet = m.skip_topology == "unet" and "skip_weights" in p
    sched = gpt.layer_schedule(m)
    if any(r for _, r in sched):
        raise NotImplementedError("cached generation does not cover recurrent layers; use re-prefill")
    x_prev_embed = torch.zeros(num_seqs, d, device=device, dtype=dtype)
    run_sum = [torch.zeros(num_seqs, d, device=device, dtype=dtype) for _ in range(n)] if m.block_smear else None
    for t in range(seq_len - 1):
        ids = toks[:, t]
        x = gpt.embed_tokens(m, p, ids, dtype)
        if m.bigram.enabled:
            if t == 0:
                b = torch.full_like(ids, m.bigram.vocab_size - 1)
            else:
                b = torch.bitwise_xor((36313 * ids) & 0xFFFFFFFF, (27191 * toks[:, t - 1]) & 0xFFFFFFFF) % (m.bigram.vocab_size - 1)
            bg = p["bigram_embed"][b].to(dtype)
            if m.bigram.trigram:
                tri = R.trigram_hash(toks[:, max(t - 2, 0): t + 1], m.bigram.vocab_size)[:, -1] if t >= 2 else torch.full_like(ids, m.bigram.vocab_size - 1)
                bg = bg + p["bigram_embed"][tri].to(dtype)
            if "bigram_proj" in p:
                bg = F.linear(bg, p["bigram_proj"].to(dtype))
            x = x + p["bigram_scale"][0].to(dtype) * bg
        x = R.rms_norm(x)
        if m.smear_gate:
            s = torch.sigmoid(p["smear_gate"].float()).to(dtype)[None, :]
            prev = x_prev_embed if t > 0 else torch.zeros_like(x)
            if m.smear_gate_boundary_token_id is not None:
                prev = prev * (ids != m.smear_gate_boundary_token_id).to(dtype)[:, None]
            x_new = (1 - s) * x + s * prev
            x_prev_embed = x
            x = x_new
        x0 = x
        skips = []
        v0 = None
        for i in range(n):
            if unet and i >= enc and skips:
                x = x + p["skip_weights"][i - enc].to(dtype)[None, :] * skips.pop()
            mix = p["resid_mix"][i].to(dtype)
            x_in = mix[0][None, :] * x + mix[1][None, :] * x0
            s_l = gpt.layer_ln_scale(m, i)
            h = R.rms_norm(x_in, s_l)
            q = F.linear(h, p["qo_bank"][i].to(dtype)).reshape(num_seqs, 1, H, D)
            k = F.linear(h, p["kv_bank"][i].to(dtype)).reshape(num_seqs, 1, Hkv, D)
            v = F.linear(h, p["kv_bank"][n + i].to(dtype))
            if m.value_embedding.enabled and i in m.value_embedding.layers:
                li = m.value_embedding.layers.index(i)
                v = v + (p["ve_layer_scales"][li] * p["ve_scale"][0]).to(dtype) * F.linear(p["ve_embed"][ids].to(dtype), p["ve_proj"].to(dtype))
            v = v.reshape(num_seqs, 1, Hkv, D)
            if m.value_residual:
                if v0 is None:
                    v0 = v
                else:
                    lam = p["vr_lambda"][i].to(dtype)
                    v = lam[0] * v0 + lam[1] * v
            q = R.rms_norm(q)
            k = R.rms_norm(k)
            if rd > 0:
                q = R.apply_rope(q, cos[t:t + 1], sin[t:t + 1], rd)
                k = R.apply_rope(k, cos[t:t + 1], sin[t:t + 1], rd)
            q = q * p["q_gain"][i].to(dtype)[None, None, :, None]
            kc[i][:, t] = k[:, 0]
            vc[i][:, t] = v[:, 0]
            K = kc[i][:, : t + 1].float()
            V = vc[i][:, : t + 1].float()
            qg = q[:, 0].float().reshape(num_seqs, Hkv, H // Hkv, D)
            sc = torch.einsum("bkgd,btkd->bkgt", qg, K) / math.sqrt(D)
            y = torch.einsum("bkgt,btkd->bkgd", torch.softmax(sc, -1), V).reshape(num_seqs, 1, H, D).to(dtype)
            if i in m.xsa_layers():
                y = R.xsa(y, v)
            if m.attn_out_gate.enabled:
                y = R.attn_out_gate(y, h[:, None], p["attn_gate_weight"][i], p["attn_gate_bias"][i])
            if m.sparse_attn_gate.enabled:
                y = R.sparse_attn_gate(y, h[:, None], p["sparse_attn_gate_weight"][i], m.sparse_attn_gate.scale)
            if m.gated_attention:
                y = y * torch.sigmoid(F.linear(h, p["gated_attn_weight"][i].to(dtype), p["gated_attn_bias"][i].to(dtype)))[:, None, :, None]
            y = y.reshape(num_seqs, d)
            if m.normed_out_proj:
                y = R.rms_norm(y)
            x_mid = x_in + p["attn_scale"][i].to(dtype)[None, :] * F.linear(y, p["qo_bank"][n + i].to(dtype))
            mlp_in = R.rms_norm(x_in if m.parallel else x_mid, s_l)
            hid = gpt.mlp_hidden(m, F.linear(mlp_in, p["mlp_up_bank"][i].to(dtype)))
            x = x_mid + p["mlp_scale"][i].to(dtype)[None, :] * F.linear(hid, p["mlp_down_bank"][i].to(dtype))
            if m.dtg:
                gate = torch.sigmoid(F.linear(x_in, p["dtg_gate_weight"][i].to(dtype)[None, :], p["dtg_gate_bias"][i].to(dtype)[None]))
                x = x_in + gate * (x - x_in)
            if m.block_smear:
                run_sum[i] = run_sum[i] + x           # the running mean over positions 0..t of this block's output
                x = x + torch.tanh(p["block_smear_gate"][i].float()).to(dtype)[None, :] * (run_sum[i] / (t + 1) - x)
            if unet and i < enc:
                skips.append(x)
        hfin = R.rms_norm(x)
        z = R.softcap(gpt.output_logits(m, p, hfin), m.logit_softcap, m.softcap_kind)
        probs = torch.softmax(z / temperature, dim=-1)
        toks[:, t + 1] = torch.multinomial(probs, 1, generator=g)[:, 0]
    return toks


def self_generated_hessians(spec: RunSpec, params: Dict[str, torch.Tensor], device="cpu", num_seqs: int = 64, seq_len: int = 2048,
                            batch: int = 8, seed: int = 42) -> Dict[Tuple[int, str], torch.Tensor]:
    m = spec.model
    dtype = torch.float32 if str(device) == "cpu" else torch.bfloat16
    p = {k: v.to(device) for k, v in params.items()}
    toks = generate_autoregressive(m, p, num_seqs, seq_len, spec.quant.gptq_temperature, seed, device,
                                   torch.float32 if str(device) == "cpu" else torch.bfloat16)
    taps = HessianTaps()
    pc = {k: (v.to(dtype) if v.ndim >= 2 else v) for k, v in p.items()}
    with torch.no_grad():
        for b0 in range(0, num_seqs, batch):
            gpt.gpt_hidden(m, pc, toks[b0:b0 + batch, :-1], dtype=dtype, taps=taps)
            taps.batches += 1
    return {k: v.cpu() for k, v in taps.finish().items()}
