"""Plain PyTorch fp32 statements of every model op (the CPU oracle).

Each function is the mathematical definition that the sm_100a kernels are tested against, and the
implementation used on CPU. Backward passes come from autograd and are checked against central
finite differences in the tests, as the reference does for its own CPU oracles
(``parameter-golf-rs/crates/pg-kernels/src/{rms_norm,rope,attention,xsa,smear_gate,bigram_hash,
cross_entropy,activations}.rs``).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

RMS_EPS = 1e-6


def _f(x: torch.Tensor) -> torch.Tensor:
    """Promote to fp32 for the arithmetic; float64 inputs (finite-difference tests) stay float64."""
    return x if x.dtype == torch.float64 else x.float()


def rms_norm(x: torch.Tensor, scale: float = 1.0, eps: float = RMS_EPS) -> torch.Tensor:
    """``y = x * scale / sqrt(mean(x^2) + eps)`` over the last dim (``rms_norm.rs``; eps 1e-6 as in
    ``pg-model/src/model.rs:470``)."""
    xf = _f(x)
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * scale).to(x.dtype)


def rope_tables(seq_len: int, rope_dims: int, base: float = 10000.0, train_seq_len: int = 0, device=None, yarn_max_len: int = 0):
    """cos/sin tables of shape [seq_len, rope_dims/2], ``theta = pos / base^(2i/rope_dims)``
    (``pg-kernels/src/rope.rs:13-28``). When ``seq_len > train_seq_len > 0`` the base is rescaled
    NTK-style (``records/.../2026-03-23_.../train_gpt.py:578-584``).

    ``yarn_max_len`` > 0 selects the YaRN-style frequency ramp of the ternary record instead
    (``records/track_10min_16mb/2026-03-24_74M_Ternary_.../train_gpt_cuda_ternary.py:570-575``): with
    ``scale = train_seq_len / yarn_max_len`` the low-frequency pairs (the last three quarters of the index range,
    linearly ramped) are slowed down by up to ``1 / scale``; the base is left alone."""
    rd = rope_dims
    idx = torch.arange(0, rd, 2, dtype=torch.float32, device=device)
    if yarn_max_len > 0:
        inv = 1.0 / (base ** (idx / rd))
        scale = (train_seq_len or seq_len) / yarn_max_len
        ramp = torch.clamp((idx / rd - 0.25) / 0.75, 0.0, 1.0)
        inv = inv / (ramp * (1.0 / scale - 1.0) + 1.0)
    else:
        if train_seq_len and seq_len > train_seq_len and rd > 2:
            base = base * ((seq_len / train_seq_len) ** (rd / (rd - 2)))
        inv = 1.0 / (base ** (idx / rd))
    fr = torch.outer(torch.arange(seq_len, dtype=torch.float32, device=device), inv)
    return fr.cos(), fr.sin()


def model_rope_tables(m, seq_len: int, device=None):
    """The tables a model spec asks for (``m`` is a `ModelSpec`): partial or full rotary with the NTK rescale beyond 1024
    positions, or the YaRN ramp when ``rope.mode == "yarn"``. ``(None, None)`` without rotary dims."""
    rd = m.rope_dims
    if rd <= 0:
        return None, None
    if m.rope.mode == "yarn":
        return rope_tables(seq_len, rd, m.rope.base, train_seq_len=m.rope.yarn_train_len, device=device, yarn_max_len=m.rope.yarn_max_len)
    return rope_tables(seq_len, rd, m.rope.base, train_seq_len=1024, device=device)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rope_dims: int) -> torch.Tensor:
    """Half-split rotary on the first ``rope_dims`` of the last dim. ``x``: [B, T, H, D]."""
    if rope_dims <= 0:
        return x
    half = rope_dims // 2
    c = cos[None, : x.shape[1], None, :].to(x.dtype)
    s = sin[None, : x.shape[1], None, :].to(x.dtype)
    x1, x2, rest = x[..., :half], x[..., half:rope_dims], x[..., rope_dims:]
    return torch.cat((x1 * c + x2 * s, -x1 * s + x2 * c, rest), dim=-1)


def qk_norm_rope_gain(q, k, cos, sin, rope_dims, q_gain, eps: float = RMS_EPS):
    """Per-head RMSNorm of q and k, partial RoPE, then ``q *= gain[h]``. q: [B,T,H,D], k: [B,T,Hkv,D]."""
    q = apply_rope(rms_norm(q, eps=eps), cos, sin, rope_dims)
    k = apply_rope(rms_norm(k, eps=eps), cos, sin, rope_dims)
    return q * q_gain.to(q.dtype)[None, None, :, None], k


def causal_gqa_attention(q, k, v):
    """Causal softmax attention with grouped KV heads, scale 1/sqrt(D), batched (each batch row is
    one sequence). q: [B,T,H,D]; k, v: [B,T,Hkv,D] -> [B,T,H,D]. Written out explicitly in fp32."""
    B, T, H, D = q.shape
    Hkv = k.shape[2]
    g = H // Hkv
    qf = _f(q).permute(0, 2, 1, 3).reshape(B, Hkv, g, T, D)
    kf = _f(k).permute(0, 2, 1, 3)[:, :, None]
    vf = _f(v).permute(0, 2, 1, 3)[:, :, None]
    s = (qf @ kf.transpose(-1, -2)) / math.sqrt(D)
    mask = torch.ones(T, T, dtype=torch.bool, device=q.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    y = torch.softmax(s, dim=-1) @ vf
    return y.reshape(B, H, T, D).permute(0, 2, 1, 3).to(q.dtype)


def xsa(y, v, eps: float = 1e-8):
    """Exclusive self attention: remove from each head output its component along that token's own
    value vector, ``z = y - (<y,v>/(|v|^2+eps)) v`` (``pg-kernels/src/xsa.rs:35``). y: [B,T,H,D], v: [B,T,Hkv,D]."""
    B, T, H, D = y.shape
    Hkv = v.shape[2]
    yg = _f(y).reshape(B, T, Hkv, H // Hkv, D)
    vf = _f(v)[:, :, :, None, :]
    coef = (yg * vf).sum(-1, keepdim=True) / (vf.pow(2).sum(-1, keepdim=True) + eps)
    return (yg - coef * vf).reshape(B, T, H, D).to(y.dtype)


def attn_out_gate(y, h, weight, bias):
    """``y *= 2*sigmoid(bias_h + W_h . h[:w])`` per (token, head). y: [B,T,H,D], h: [B,T,d], weight: [H,w]."""
    w = weight.shape[1]
    g = 2.0 * torch.sigmoid(_f(h[..., :w]) @ _f(weight).t() + _f(bias))
    return (_f(y) * g[..., None]).to(y.dtype)


def sparse_attn_gate(y, h, weight, scale: float):
    """``y *= sigmoid(scale * W_h . h[:w])`` per (token, head)."""
    w = weight.shape[1]
    g = torch.sigmoid(scale * (_f(h[..., :w]) @ _f(weight).t()))
    return (_f(y) * g[..., None]).to(y.dtype)


def smear_gate(x, gate, ids=None, boundary_id=None):
    """``out = (1-s)*x + s*x_prev`` with ``s = sigmoid(gate)`` per feature; ``x_prev`` is zero at the
    first position of a sequence and, when ``boundary_id`` is given, where the current token equals
    it (``pg-kernels/src/smear_gate.rs:33-51``). x: [B,T,d]."""
    s = torch.sigmoid(_f(gate)).to(x.dtype)[None, None, :]
    x_prev = torch.cat([torch.zeros_like(x[:, :1]), x[:, :-1]], dim=1)
    if boundary_id is not None and ids is not None:
        x_prev = x_prev * (ids != boundary_id).to(x.dtype)[..., None]
    return (1 - s) * x + s * x_prev


def trigram_hash(ids: torch.Tensor, buckets: int) -> torch.Tensor:
    """``((36313*cur) xor (27191*prev) xor (51497*prev2)) mod (buckets-1)`` in wrapping 32-bit arithmetic into the bigram table;
    the first two positions of each sequence map to the sentinel bucket
    (records/track_10min_16mb/2026-03-25_ValCalib_GPTQ_XSA_BigramHash3072/train_gpt.py:698-705). ids: [B,T]."""
    t = ids.to(torch.int64)
    mod = buckets - 1
    out = torch.full_like(t, mod)
    if t.shape[-1] > 2:
        # int32 products wrap; xor and the remainder then act on the signed value, as torch does on int32 tensors
        def wrap(v):
            v = v & 0xFFFFFFFF
            return torch.where(v >= 2 ** 31, v - 2 ** 32, v)
        h = wrap(36313 * t[..., 2:]) ^ wrap(27191 * t[..., 1:-1]) ^ wrap(51497 * t[..., :-2])
        out[..., 2:] = torch.remainder(h, mod)
    return out


def running_mean_smear(x, gate):
    """``x + tanh(gate) * (m - x)`` where ``m[t]`` is the mean of ``x[0..t]`` of the same sequence: every position is blended with
    the causal running mean of its sequence, per feature, by a gate that starts at zero
    (records/track_non_record_16mb/2026-03-24_106M_Binary_.../train_gpt_cuda_binary.py:647-656). x: [B,T,d], gate: [d]."""
    counts = torch.arange(1, x.shape[1] + 1, device=x.device, dtype=x.dtype)[None, :, None]
    mean = x.cumsum(dim=1) / counts
    return x + torch.tanh(_f(gate)).to(x.dtype)[None, None, :] * (mean - x)


def bigram_hash(ids: torch.Tensor, buckets: int) -> torch.Tensor:
    """``((36313*cur) xor (27191*prev)) mod (buckets-1)`` in wrapping 32-bit arithmetic; the first
    position of each sequence maps to the sentinel bucket ``buckets-1``
    (``pg-kernels/src/bigram_hash.rs``; ``records/.../2026-03-23_.../train_gpt.py:700-706``). ids: [B,T]."""
    t = ids.to(torch.int64)
    mod = buckets - 1
    cur = (36313 * t[..., 1:]) & 0xFFFFFFFF
    prev = (27191 * t[..., :-1]) & 0xFFFFFFFF
    out = torch.empty_like(t)
    out[..., 0] = mod
    out[..., 1:] = torch.bitwise_xor(cur, prev) % mod
    return out


def act_sq(x, slope: float):
    """``leaky_relu(x, slope)^2``; slope 0 is relu^2."""
    return F.leaky_relu(x, negative_slope=slope).square()


def softcap(z, cap: float, kind: str = "tanh"):
    """Soft cap of logits to (-cap, cap) in fp32. ``tanh``: ``cap * tanh(z / cap)``. ``poly5``: the degree-5 odd polynomial of the
    ternary record, ``x (1 - x^2/3 + x^4/15)`` of ``x = clamp(z / cap, -2, 2)``, clamped to [-1, 1] and scaled by ``cap``
    (``records/track_10min_16mb/2026-03-24_74M_Ternary_.../train_gpt_cuda_ternary.py:859-865``)."""
    zf = _f(z)
    if kind == "tanh":
        return cap * torch.tanh(zf / cap)
    if kind == "poly5":
        x = torch.clamp(zf / cap, -2.0, 2.0)
        x2 = x * x
        return cap * torch.clamp(x * (1.0 - x2 / 3.0 + x2 * x2 / 15.0), -1.0, 1.0)
    raise ValueError(f"unknown softcap kind {kind!r}")


def softcap_cross_entropy(logits, targets, cap: float, reduction: str = "mean", kind: str = "tanh", z_loss: float = 0.0, temperature: float = 1.0):
    """``CE(softcap(z) / temperature)`` in fp32 (``pg-kernels/src/cross_entropy.rs``); ``z_loss`` > 0 adds that weight times the
    mean squared log-partition (only to the mean reduction: a training-time regulariser). ``temperature`` != 1 is the evaluation-time
    scaling of the ternary record (its capped logits are slightly under-confident)."""
    c = softcap(logits, cap, kind)
    if temperature != 1.0:
        c = c / temperature
    c2, t = c.reshape(-1, c.shape[-1]), targets.reshape(-1)
    loss = F.cross_entropy(c2, t, reduction=reduction)
    if z_loss > 0.0 and reduction == "mean":
        loss = loss + z_loss * torch.logsumexp(c2, dim=-1).pow(2).mean()
    return loss


def fake_quant_fp8_ste(w: torch.Tensor) -> torch.Tensor:
    """Straight-through estimator of FP8 (e4m3) storage: forward uses the value after a round trip through
    ``float8_e4m3fn``, the gradient passes to ``w``
    (``records/track_10min_16mb/2026-03-24_74M_Ternary_.../train_gpt_cuda_ternary.py:418-431``)."""
    with torch.no_grad():
        wq = _f(w).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).to(w.dtype)
    return w + (wq - w).detach()


def fake_quant_ternary_ste(w: torch.Tensor, group: int = 128) -> torch.Tensor:
    """Straight-through estimator of BitNet b1.58 weights: the forward uses ``s * q`` with ``q`` in {-1, 0, 1} and one scale per
    group of ``group`` input columns, computed by the same rule as the ternary export (`quant.ternary.quantize_ternary`, scale
    fitted to the non-zero codes), so what is trained is what is stored; the gradient passes to ``w``. Matrices or stacks of
    matrices (the last axis is the input dimension)."""
    from ..quant.ternary import dequantize_ternary, quantize_ternary
    with torch.no_grad():
        w2 = _f(w).reshape(-1, w.shape[-1])
        q, s = quantize_ternary(w2, group)
        wq = dequantize_ternary(q, s.half().float(), group).reshape(w.shape).to(w.dtype)       # scales are stored as fp16
    return w + (wq - w).detach()


def fake_quant_binary_ste(w: torch.Tensor, group: int = 128) -> torch.Tensor:
    """Straight-through estimator of 1-bit weights: the forward uses ``s * sign(w)`` (zero counts as +1) with ``s`` the mean
    magnitude of each group of ``group`` input columns, the rule of the binary export (`quant.binary.quantize_binary`) with the
    scale rounded to fp16 as it is stored; the gradient passes to ``w``
    (records/track_non_record_16mb/2026-03-24_106M_Binary_.../train_gpt_cuda_binary.py:417-428). Matrices or stacks of matrices."""
    from ..quant.binary import dequantize_binary, quantize_binary
    with torch.no_grad():
        w2 = _f(w).reshape(-1, w.shape[-1])
        q, s = quantize_binary(w2, group)
        wq = dequantize_binary(q, s.half().float(), group).reshape(w.shape).to(w.dtype)
    return w + (wq - w).detach()


def quant_noise(w: torch.Tensor, qmax: int = 127) -> torch.Tensor:
    """``w + u * step`` with ``u`` uniform in [-0.5, 0.5) and ``step = max|row| / qmax``: noise of the size of a per-row
    quantisation step instead of the rounding itself. Unlike the straight-through forms the perturbation is part of the
    graph, so a block that runs several times per pass learns weights that tolerate the error it will carry after export
    (records/track_non_record_16mb/2026-03-21_DepthRecurrence_MixedPrecisionQuant/README.md "Noisy QAT"). The noise comes from
    torch's global generator (seed it for a repeatable run)."""
    with torch.no_grad():
        step = _f(w).abs().amax(dim=-1, keepdim=True).clamp_min(1e-12) / float(qmax)
    return w + (torch.rand_like(w) - 0.5) * step.to(w.dtype)


def fake_quant_int6_ste(w: torch.Tensor) -> torch.Tensor:
    """Late-QAT straight-through estimator: per-row ``s = max(|w|)/31`` (floored at 1/31),
    ``w_q = clamp(round(w/s), -32, 31) * s``; forward uses ``w_q`` and the gradient passes to ``w``
    (``records/.../2026-03-23_.../train_gpt.py:541-553``)."""
    with torch.no_grad():
        w32 = _f(w)
        scale = (w32.abs().amax(dim=-1, keepdim=True) / 31.0).clamp_min(1.0 / 31.0)
        wq = (torch.clamp(torch.round(w32 / scale), -32, 31) * scale).to(w.dtype)
    return w + (wq - w).detach()
