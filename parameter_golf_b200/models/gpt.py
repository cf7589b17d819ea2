"""Bank-parameterised GPT: parameters, initialisation and the autograd (oracle) forward.

Parameter layout (``parameter-golf-rs/crates/pg-model/src/model.rs:18-67``; Python record
``records/track_10min_16mb/2026-03-23_LeakyReLU_LegalTTT_ParallelMuon/train_gpt.py:812-870``):
``tok_emb[V,d]`` (tied output), banks ``qo_bank[2n,d,d]`` (Q then O), ``kv_bank[2n,kv,d]`` (K then V),
``mlp_up_bank[n,mlp,d]``, ``mlp_down_bank[n,d,mlp]``; per-block controls are stored stacked over layers:
``attn_scale[n,d]``, ``mlp_scale[n,d]``, ``resid_mix[n,2,d]``, ``q_gain[n,H]``; ``skip_weights[min(n/2,n-n/2),d]``,
``smear_gate[d]``, ``block_smear_gate[n,d]`` (per-block running-mean smear), BigramHash ``bigram_embed[B,bd]``/``bigram_proj[d,bd]``/``bigram_scale``, value embedding
``ve_embed[V,ve]``/``ve_proj[kv,ve]``/``ve_scale``/``ve_layer_scales``, optional attention gates.

`gpt_forward` is the single definition of the model function (forward math of
``model.rs:681-827`` / block ``:448-663``); the CUDA engine is tested against it.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn.functional as F

from ..ops import reference as R
from ..spec import ModelSpec

BANKS = ("qo_bank", "kv_bank", "mlp_up_bank", "mlp_down_bank")
EMBEDS = ("tok_emb", "bigram_embed", "ve_embed", "lm_head")
TRAIN_ONLY = ("mtp_heads",)          # never exported (records/.../2026-03-23_.../train_gpt.py:1778)


def up_rows(m: ModelSpec) -> int:
    """Rows of one block's slice of ``mlp_up_bank``: the hidden width, twice that for SwiGLU (gate rows, then up rows)."""
    return 2 * m.mlp_dim if m.activation == "swiglu" else m.mlp_dim


def param_shapes(m: ModelSpec) -> Dict[str, tuple]:
    n, d, kv, mlp, H = m.num_layers, m.model_dim, m.kv_dim, m.mlp_dim, m.num_heads
    enc = m.depth // 2                 # the U-Net split counts virtual layers (= blocks unless they are cycled)
    sh = {
        "tok_emb": (m.vocab_size, m.embed_dim if m.embed_dim > 0 else d),
        "qo_bank": (2 * n, d, d),
        "kv_bank": (2 * n, kv, d),
        "mlp_up_bank": (n, up_rows(m), d),
        "mlp_down_bank": (n, d, mlp),
        "attn_scale": (n, d),
        "mlp_scale": (n, d),
        "resid_mix": (n, 2, d),
        "q_gain": (n, H),
    }
    if m.skip_topology == "unet" and min(enc, m.depth - enc) > 0:
        sh["skip_weights"] = (min(enc, m.depth - enc), d)
    if m.smear_gate:
        sh["smear_gate"] = (d,)
    if m.bigram.enabled:
        sh["bigram_embed"] = (m.bigram.vocab_size, m.bigram.dim)
        if m.bigram.dim != d:
            sh["bigram_proj"] = (d, m.bigram.dim)
        sh["bigram_scale"] = (1,)
    if m.value_embedding.enabled:
        sh["ve_embed"] = (m.vocab_size, m.value_embedding.dim)
        sh["ve_proj"] = (kv, m.value_embedding.dim)
        sh["ve_scale"] = (1,)
        sh["ve_layer_scales"] = (len(m.value_embedding.layers),)
    if m.attn_out_gate.enabled:
        sh["attn_gate_weight"] = (n, H, m.attn_out_gate.width)
        sh["attn_gate_bias"] = (n, H)
    if m.sparse_attn_gate.enabled:
        sh["sparse_attn_gate_weight"] = (n, H, m.sparse_attn_gate.width)
    if not m.tie_embeddings:
        sh["lm_head"] = (m.vocab_size, d)
    if m.embed_dim > 0:
        sh["embed_proj_in"] = (d, m.embed_dim)           # embedding -> model width at the input
        sh["embed_proj_out"] = (m.embed_dim, d)          # model width -> embedding before the tied output product
    if m.value_residual:
        sh["vr_lambda"] = (n, 2)
    if m.dtg:
        sh["dtg_gate_weight"] = (n, d)
        sh["dtg_gate_bias"] = (n,)
    if m.mtp_num_heads > 0:
        sh["mtp_heads"] = (m.mtp_num_heads, m.vocab_size, d)
    if m.block_smear:
        sh["block_smear_gate"] = (n, d)
    if m.vocab_bias:
        sh["vocab_bias"] = (m.vocab_size,)
    if m.gated_attention:
        sh["gated_attn_weight"] = (n, H, d)
        sh["gated_attn_bias"] = (n, H)
    r = m.recurrence.depth_lora_rank if m.cycled else 0
    if r > 0:
        sh["depth_lora_q_down"] = (m.depth, r, d)
        sh["depth_lora_q_up"] = (m.depth, d, r)
        sh["depth_lora_v_down"] = (m.depth, r, d)
        sh["depth_lora_v_up"] = (m.depth, kv, r)
    return sh


def count_params(m: ModelSpec) -> int:
    return sum(math.prod(s) for s in param_shapes(m).values())


def _orthogonal(rows: int, cols: int, gen: torch.Generator) -> torch.Tensor:
    a = torch.randn(max(rows, cols), min(rows, cols), generator=gen, dtype=torch.float32)
    q, r = torch.linalg.qr(a)
    q = q * torch.sign(torch.diagonal(r))[None, :]
    return q if rows >= cols else q.t().contiguous()


def init_params(m: ModelSpec, seed: int = 1337, device="cpu", dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """Random initialisation of the Python records (``…03-23…/train_gpt.py:875-897``): tied embedding
    N(0, std), orthogonal Q/K/V/up, zero O/down, zero bigram tables, scale 0.05; controls at identity."""
    g = torch.Generator().manual_seed(seed)
    n, d = m.num_layers, m.model_dim
    p: Dict[str, torch.Tensor] = {}
    for name, shape in param_shapes(m).items():
        p[name] = torch.zeros(shape, dtype=torch.float32)
    p["tok_emb"].normal_(0.0, m.tied_embed_init_std if m.tie_embeddings else 1.0, generator=g)
    if m.embed_init == "overtone" and m.tie_embeddings:
        # records/track_10min_16mb/2026-03-19_SlidingWindow_FP16Emb_10L_MuonWD_OvertoneInit/train_gpt.py:723-728: keep the singular
        # vectors of the random table and give it the spectrum s_1 k^(-1/2)
        U, S, Vh = torch.linalg.svd(p["tok_emb"], full_matrices=False)
        target = S[0] * torch.arange(1, S.shape[0] + 1, dtype=S.dtype).rsqrt()
        p["tok_emb"] = ((U * target[None, :]) @ Vh).contiguous()
    for i in range(n):
        p["qo_bank"][i] = _orthogonal(d, d, g)
        p["kv_bank"][i] = _orthogonal(m.kv_dim, d, g)
        p["kv_bank"][n + i] = _orthogonal(m.kv_dim, d, g)
        p["mlp_up_bank"][i] = _orthogonal(up_rows(m), d, g)
    p["attn_scale"].fill_(1.0)
    p["mlp_scale"].fill_(1.0)
    p["resid_mix"][:, 0].fill_(1.0)
    if m.resid_mix_init == "phase":
        # …OvertoneInit/train_gpt.py:731-737: early blocks lean on the embedding stream x0, late ones on the residual stream
        for i in range(n):
            phase = float(torch.sigmoid(torch.tensor(3.0 * (i / max(n - 1, 1) - 0.5))))
            p["resid_mix"][i, 0].fill_(phase)
            p["resid_mix"][i, 1].fill_(1.0 - phase)
    p["q_gain"].fill_(m.qk_gain_init)
    if "skip_weights" in p:
        p["skip_weights"].fill_(1.0)
    if "bigram_scale" in p:
        p["bigram_scale"].fill_(0.05)
    if "ve_embed" in p:
        p["ve_embed"].normal_(0.0, 0.01, generator=g)
        p["ve_scale"].fill_(0.1)
        p["ve_layer_scales"].fill_(1.0)
    if "attn_gate_bias" in p:
        p["attn_gate_bias"].fill_(4.0)
    if "gated_attn_bias" in p:
        p["gated_attn_bias"].fill_(4.0)           # sigmoid(4) = 0.98: the gate starts almost open, its weight at zero
    if "embed_proj_in" in p:
        p["embed_proj_in"] = _orthogonal(d, m.embed_dim, g)
        p["embed_proj_out"] = p["embed_proj_in"].t().contiguous().clone()     # starts as the transpose: the tied pair is consistent
    if "vr_lambda" in p:
        p["vr_lambda"].fill_(0.5)
    for k in ("depth_lora_q_down", "depth_lora_v_down"):          # the up halves stay zero: the adapters start as no-ops
        if k in p:
            p[k].uniform_(-1.0 / math.sqrt(d), 1.0 / math.sqrt(d), generator=g)
    if "dtg_gate_bias" in p:
        p["dtg_gate_bias"].fill_(2.0)             # sigmoid(2) = 0.88 of the block's update at the start, the weight at zero
    return {k: v.to(device=device, dtype=dtype) for k, v in p.items()}


def fill_deterministic(m: ModelSpec, device="cpu", dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """Seed-free, dense, non-degenerate weights for parity tests: element ``i`` of tensor number ``t``
    is ``amp * sin(0.37*i + 1.3*t + 0.11*(i mod 97))`` with a per-tensor amplitude, so every code
    path (O/down projections, bigram, gates) carries signal. Same role as the reference's
    ``fill_deterministic`` (``pg-model/src/model.rs:281-331``); the pattern itself is this project's."""
    p: Dict[str, torch.Tensor] = {}
    for t, (name, shape) in enumerate(sorted(param_shapes(m).items())):
        numel = math.prod(shape)
        i = torch.arange(numel, dtype=torch.float64)
        fan_in = shape[-1] if len(shape) >= 2 else 1
        amp = {"tok_emb": 0.3, "bigram_embed": 0.3, "ve_embed": 0.3}.get(name, 1.0 / math.sqrt(fan_in) if len(shape) >= 2 else 0.2)
        v = amp * torch.sin(0.37 * i + 1.3 * t + 0.11 * (i % 97))
        if name == "vr_lambda":
            v = 0.5 + 0.2 * v / amp * 0.2
        if name in ("attn_scale", "mlp_scale", "skip_weights", "q_gain"):
            v = 1.0 + 0.25 * v / amp * 0.2
        if name == "resid_mix":
            v = v.reshape(shape)
            v[:, 0] = 0.9 + 0.1 * v[:, 0]
            v[:, 1] = 0.2 * v[:, 1]
        if name in ("bigram_scale", "ve_scale"):
            v = torch.full(shape, 0.3, dtype=torch.float64)
        if name == "ve_layer_scales":
            v = torch.full(shape, 0.8, dtype=torch.float64)
        p[name] = v.reshape(shape).to(device=device, dtype=dtype)
    return p


def _small(m: ModelSpec, p, name: str, qat: bool):
    """A small 2-D float tensor as the forward sees it: through the FP8 round trip while QAT is on and the spec stores it so."""
    w = p[name]
    return R.fake_quant_fp8_ste(w) if (qat and m.fp8_qat) else w


def embed_tokens(m: ModelSpec, p, ids, dt, qat: bool = False):
    """Token embedding at model width: a table row, through the input projection when the embedding is factored."""
    x = p["tok_emb"][ids].to(dt)
    if m.embed_dim > 0:
        x = F.linear(x, _small(m, p, "embed_proj_in", qat).to(dt))
    return x


def output_logits(m: ModelSpec, p, h, qat: bool = False, lora=None):
    """Un-capped logits of final hidden states: the tied table (after the output projection when the embedding is factored) or
    the untied head; plus the per-batch-element head adapter of per-document test-time training when ``lora`` carries one."""
    bias = p["vocab_bias"].to(h.dtype) if m.vocab_bias else None      # train_gpt_cuda_ternary.py:851
    extra = 0
    if lora is not None and "head_a" in lora:
        extra = torch.bmm(torch.bmm(h, lora["head_a"].to(h.dtype).mT), lora["head_b"].to(h.dtype).mT)
    if not m.tie_embeddings:
        return F.linear(h, _small(m, p, "lm_head", qat).to(h.dtype), bias) + extra
    if m.embed_dim > 0:
        h = F.linear(h, _small(m, p, "embed_proj_out", qat).to(h.dtype))
    return F.linear(h, p["tok_emb"].to(h.dtype), bias) + extra


def mlp_hidden(m: ModelSpec, u):
    """The MLP's hidden activation from the up-projection's output: the squared (leaky) ReLU, or for SwiGLU
    ``silu(gate) * up`` with the gate in the first half of the columns
    (records/track_non_record_16mb/2026-03-24_106M_Binary_.../train_gpt_cuda_binary.py:635-639), followed by the RMSNorm that the
    ternary and binary submissions put in front of their down projection when ``normed_out_proj`` is set."""
    if m.activation == "swiglu":
        gate, up = u.chunk(2, dim=-1)
        hid = F.silu(gate) * up
    else:
        hid = R.act_sq(u, m.leaky_slope if m.activation == "leaky_relu_sq" else 0.0)
    return R.rms_norm(hid) if m.normed_out_proj else hid


def layer_ln_scale(m: ModelSpec, layer: int) -> float:
    return 1.0 / math.sqrt(layer + 1) if m.ln_scale else 1.0


def layer_schedule(m: ModelSpec):
    """Execution order as (layer index, pass index): recurrent layers run the block twice in a row
    (``pg-model/src/model.rs:666-671``); in the cycled form the blocks run round robin for ``effective_depth`` executions
    (records/track_non_record_16mb/2026-03-21_DepthRecurrence_MixedPrecisionQuant/train_gpt.py:863)."""
    if m.cycled:
        return [(v % m.num_layers, v // m.num_layers) for v in range(m.depth)]
    order = []
    for i in range(m.num_layers):
        reps = m.recurrence.repeats if (m.recurrence.enabled and m.recurrence.start_layer <= i < m.recurrence.start_layer + m.recurrence.repeat_layers) else 1
        order.extend((i, r) for r in range(reps))
    return order


def shared_layers(m: ModelSpec) -> set:
    """Blocks that run more than once in a forward pass."""
    seen, twice = set(), set()
    for i, _ in layer_schedule(m):
        (twice if i in seen else seen).add(i)
    return twice


def block_forward(m: ModelSpec, p, i: int, x, x0, ids, cos, sin, qat: bool = False, lora=None, return_kv: bool = False, taps=None, v0=None,
                  return_raw_v: bool = False, depth_index: Optional[int] = None):
    """One block. ``v0`` / ``return_raw_v`` serve the value residual (records/.../2026-03-23_.../train_gpt.py:655-658): the
    block's own value projection is handed back, and when an earlier layer's is given the attention runs on
    ``lambda_0 * v0 + lambda_1 * v``."""
    n, H, Hkv, D = m.num_layers, m.num_heads, m.num_kv_heads, m.head_dim
    B, T, d = x.shape
    dt = x.dtype
    wq = p["qo_bank"][i]
    wo = p["qo_bank"][n + i]
    wk, wv = p["kv_bank"][i], p["kv_bank"][n + i]
    wu, wd = p["mlp_up_bank"][i], p["mlp_down_bank"][i]
    if qat:
        if m.qat_kind == "ternary":
            wq, wo, wk, wv, wu, wd = (R.fake_quant_ternary_ste(w, m.qat_ternary_group) for w in (wq, wo, wk, wv, wu, wd))
        elif m.qat_kind == "binary":
            wq, wo, wk, wv, wu, wd = (R.fake_quant_binary_ste(w, m.qat_ternary_group) for w in (wq, wo, wk, wv, wu, wd))
        elif m.qat_kind == "noise":
            shared = shared_layers(m)
            if not shared or i in shared:
                wq, wo, wk, wv, wu, wd = (R.quant_noise(w, m.qat_noise_qmax) for w in (wq, wo, wk, wv, wu, wd))
        else:
            wq, wo, wk, wv, wu, wd = (R.fake_quant_int6_ste(w) for w in (wq, wo, wk, wv, wu, wd))
    s_l = layer_ln_scale(m, i)
    mix = p["resid_mix"][i].to(dt)
    x_in = mix[0][None, None, :] * x + mix[1][None, None, :] * x0
    h = R.rms_norm(x_in, s_l)
    if taps is not None:
        taps.add(i, "qkv", h)
    q = F.linear(h, wq.to(dt))
    k = F.linear(h, wk.to(dt))
    v = F.linear(h, wv.to(dt))
    if lora is not None and "q_a" in lora:
        # one adapter per batch element on the query and value projections (per-document test-time training,
        # records/track_10min_16mb/2026-03-17_LoRA_TTT/train_gpt.py:755-766): A [B, r, d], B [B, out, r]
        q = q + torch.bmm(torch.bmm(h, lora["q_a"][i].to(dt).mT), lora["q_b"][i].to(dt).mT)
        v = v + torch.bmm(torch.bmm(h, lora["v_a"][i].to(dt).mT), lora["v_b"][i].to(dt).mT)
    elif lora is not None:
        a, b, alpha = lora["a"][i], lora["b"][i], lora["alpha"]
        q = q + (alpha / a.shape[0]) * F.linear(F.linear(h, a.to(dt)), b.to(dt))
    if depth_index is not None and "depth_lora_q_up" in p:
        # per-virtual-layer corrections of a shared block's query and value projections (…DepthRecurrence…/train_gpt.py:771-793, :755-760)
        q = q + F.linear(F.linear(h, p["depth_lora_q_down"][depth_index].to(dt)), p["depth_lora_q_up"][depth_index].to(dt))
        v = v + F.linear(F.linear(h, p["depth_lora_v_down"][depth_index].to(dt)), p["depth_lora_v_up"][depth_index].to(dt))
    if m.value_embedding.enabled and i in m.value_embedding.layers:
        li = m.value_embedding.layers.index(i)
        ve = F.linear(_small(m, p, "ve_embed", qat)[ids].to(dt), _small(m, p, "ve_proj", qat).to(dt))
        v = v + (p["ve_layer_scales"][li] * p["ve_scale"][0]).to(dt) * ve
    q = q.reshape(B, T, H, D)
    k = k.reshape(B, T, Hkv, D)
    v = v.reshape(B, T, Hkv, D)
    raw_v = v
    if m.value_residual and v0 is not None:
        lam = p["vr_lambda"][i].to(dt)
        v = lam[0] * v0 + lam[1] * v
    q, k = R.qk_norm_rope_gain(q, k, cos, sin, m.rope_dims, p["q_gain"][i])
    y = R.causal_gqa_attention(q, k, v)
    if i in m.xsa_layers():
        y = R.xsa(y, v)
    if m.attn_out_gate.enabled:
        y = R.attn_out_gate(y, h, p["attn_gate_weight"][i], p["attn_gate_bias"][i])
    if m.sparse_attn_gate.enabled:
        y = R.sparse_attn_gate(y, h, p["sparse_attn_gate_weight"][i], m.sparse_attn_gate.scale)
    if m.gated_attention:
        # records/.../2026-03-23_.../train_gpt.py:668-671: the gate reads the whole normed block input
        gate = torch.sigmoid(F.linear(h, p["gated_attn_weight"][i].to(dt), p["gated_attn_bias"][i].to(dt)))
        y = y * gate[..., None]
    y = y.reshape(B, T, d)
    if m.normed_out_proj:
        y = R.rms_norm(y)                 # train_gpt_cuda_ternary.py:468-470: the output projection norms its own input
    if taps is not None:
        taps.add(i, "o", y)
    attn = F.linear(y, wo.to(dt))
    x_mid = x_in + p["attn_scale"][i].to(dt)[None, None, :] * attn
    mlp_in = R.rms_norm(x_in if m.parallel else x_mid, s_l)
    if taps is not None:
        taps.add(i, "up", mlp_in)
    hid = mlp_hidden(m, F.linear(mlp_in, wu.to(dt)))
    if taps is not None:
        taps.add(i, "down", hid)
    out = x_mid + p["mlp_scale"][i].to(dt)[None, None, :] * F.linear(hid, wd.to(dt))
    if m.dtg:
        # records/.../2026-03-23_.../train_gpt.py:769-771: the gate reads the block input without sending it a gradient
        gate = torch.sigmoid(F.linear(x_in.detach(), p["dtg_gate_weight"][i].to(dt)[None, :], p["dtg_gate_bias"][i].to(dt)[None]))
        out = x_in + gate * (out - x_in)
    if m.block_smear:
        out = R.running_mean_smear(out, p["block_smear_gate"][i])
    if return_kv:
        return out, (k, v)
    if return_raw_v:
        return out, raw_v
    return out


def gpt_hidden(m: ModelSpec, p, ids: torch.Tensor, qat: bool = False, lora=None, dtype=None, taps=None):
    """Final-norm hidden states [B,T,d]."""
    dt = dtype or p["tok_emb"].dtype
    B, T = ids.shape
    x = embed_tokens(m, p, ids, dt, qat)
    if m.bigram.enabled:
        table = _small(m, p, "bigram_embed", qat)
        bg = table[R.bigram_hash(ids, m.bigram.vocab_size)].to(dt)
        if m.bigram.trigram:
            bg = bg + table[R.trigram_hash(ids, m.bigram.vocab_size)].to(dt)
        if "bigram_proj" in p:
            bg = F.linear(bg, _small(m, p, "bigram_proj", qat).to(dt))
        x = x + p["bigram_scale"][0].to(dt) * bg
    x = R.rms_norm(x)
    if m.smear_gate:
        x = R.smear_gate(x, p["smear_gate"], ids, m.smear_gate_boundary_token_id)
    x0 = x
    rd = m.rope_dims
    cos, sin = R.model_rope_tables(m, T, device=ids.device)
    enc = m.depth // 2
    unet = m.skip_topology == "unet" and "skip_weights" in p
    skips = []
    sched = layer_schedule(m)
    v0 = None
    for j, (i, rep) in enumerate(sched):
        last_pass = j + 1 == len(sched) or sched[j + 1][0] != i
        # position in the U-Net: the block index, or the execution index when the blocks are cycled (every execution is then a layer of its own)
        pos, first, last = (j, True, True) if m.cycled else (i, rep == 0, last_pass)
        if unet and pos >= enc and first and skips:
            x = x + p["skip_weights"][pos - enc].to(dt)[None, None, :] * skips.pop()
        if m.value_residual:
            x, raw_v = block_forward(m, p, i, x, x0, ids, cos, sin, qat=qat, lora=lora, taps=taps, v0=v0, return_raw_v=True,
                                     depth_index=j if m.cycled else None)
            if v0 is None:
                v0 = raw_v                  # the first block's values, mixed into every later block's
        else:
            x = block_forward(m, p, i, x, x0, ids, cos, sin, qat=qat, lora=lora, taps=taps, depth_index=j if m.cycled else None)
        if unet and pos < enc and last:
            skips.append(x)
    return R.rms_norm(x)


def gpt_logits(m: ModelSpec, p, ids, qat: bool = False, lora=None, dtype=None):
    """Soft-capped logits [B,T,V]."""
    h = gpt_hidden(m, p, ids, qat=qat, lora=lora, dtype=dtype)
    z = output_logits(m, p, h, qat, lora)
    return R.softcap(z, m.logit_softcap, m.softcap_kind)


def mtp_loss(m: ModelSpec, p, h, targets):
    """Mean over the extra heads of the soft-capped cross-entropy of head k (on the final hidden state of position t) against
    the token k + 2 positions ahead, i.e. ``targets[:, t + k + 1]`` (records/.../2026-03-23_.../train_gpt.py:947-962)."""
    T = h.shape[1]
    total, count = None, 0
    for k in range(m.mtp_num_heads):
        valid = T - (k + 1)
        if valid <= 0:
            continue
        z = F.linear(h[:, :valid], p["mtp_heads"][k].to(h.dtype))
        l = R.softcap_cross_entropy(z, targets[:, k + 1:], m.logit_softcap, reduction="mean", kind=m.softcap_kind)
        total = l if total is None else total + l
        count += 1
    return None if count == 0 else total / count


def gpt_forward(m: ModelSpec, p, ids, targets, qat: bool = False, lora=None, dtype=None, reduction: str = "mean", token_weights=None,
                mtp: bool = False, train: bool = False, temperature: float = 1.0):
    """Training loss: mean soft-capped cross-entropy over all tokens (``reduction='none'`` gives the
    per-token losses [B,T]). With ``token_weights`` (same shape as ``targets``) the mean is weighted and normalised
    by the sum of the weights (complementary training, ``pg-kernels/src/complementary.rs:226-240``). ``mtp`` (training steps
    only) adds ``mtp_loss_weight`` times the multi-token-prediction loss of the extra heads; ``train`` adds the z-loss term
    (``model.z_loss_weight`` times the mean squared log-partition), which evaluation never includes."""
    h = gpt_hidden(m, p, ids, qat=qat, lora=lora, dtype=dtype)
    z = output_logits(m, p, h, qat, lora)
    extra = None
    if mtp and reduction == "mean" and m.mtp_num_heads > 0 and m.mtp_loss_weight > 0.0 and "mtp_heads" in p:
        extra = mtp_loss(m, p, h, targets)
    if token_weights is not None and reduction == "mean":
        per = R.softcap_cross_entropy(z, targets, m.logit_softcap, reduction="none", kind=m.softcap_kind, temperature=temperature).reshape(-1).float()
        tw = token_weights.reshape(-1).to(per.dtype)
        loss = (per * tw).sum() / tw.sum().clamp_min(1e-12)
        return loss if extra is None else loss + m.mtp_loss_weight * extra
    loss = R.softcap_cross_entropy(z, targets, m.logit_softcap, reduction=reduction, kind=m.softcap_kind, z_loss=m.z_loss_weight if (train or mtp) else 0.0,
                                   temperature=temperature)
    if extra is not None:
        loss = loss + m.mtp_loss_weight * extra
    return loss.reshape(ids.shape) if reduction == "none" else loss


def bank_views(m: ModelSpec, p) -> Dict[str, torch.Tensor]:
    """Zero-copy per-group 2-D views used by export and quantisation: ``qo_bank.q`` [n*d, d] etc.
    (``parameter-golf-rs/crates/pg-quant/src/export.rs:48-126``)."""
    n, d, kv, mlp = m.num_layers, m.model_dim, m.kv_dim, m.mlp_dim
    return {
        "qo_bank.q": p["qo_bank"][:n].reshape(n * d, d),
        "qo_bank.o": p["qo_bank"][n:].reshape(n * d, d),
        "kv_bank.k": p["kv_bank"][:n].reshape(n * kv, d),
        "kv_bank.v": p["kv_bank"][n:].reshape(n * kv, d),
        "mlp_up_bank": p["mlp_up_bank"].reshape(n * up_rows(m), d),
        "mlp_down_bank": p["mlp_down_bank"].reshape(n * d, mlp),
        "tok_emb": p["tok_emb"],
    }


def overlaps_storage(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Alias guard: do two tensors share any byte of the same storage?
    (``parameter-golf-rs/crates/pg-core/src/tensor.rs:349-367``)."""
    if a.untyped_storage().data_ptr() != b.untyped_storage().data_ptr():
        return False

    def span(t):
        lo = t.storage_offset() * t.element_size()
        ext = sum((s - 1) * st for s, st in zip(t.shape, t.stride()) if s > 0) + 1 if t.numel() else 0
        return lo, lo + ext * t.element_size()

    (a0, a1), (b0, b1) = span(a), span(b)
    return a0 < b1 and b0 < a1
