"""CPU oracle ops: closed forms and central finite differences (float64 gradcheck)."""
import math

import pytest
import torch

from parameter_golf_b200.ops import reference as R

torch.manual_seed(0)


def _gc(fn, *args):
    args = [a.double().requires_grad_(True) if torch.is_tensor(a) and a.is_floating_point() else a for a in args]
    assert torch.autograd.gradcheck(fn, args, eps=1e-6, atol=1e-5, rtol=1e-4)


def test_rms_norm_value_and_grad():
    x = torch.randn(3, 5, 8)
    y = R.rms_norm(x, 0.5)
    assert torch.allclose((y / 0.5).pow(2).mean(-1), torch.ones(3, 5), atol=1e-4)
    _gc(lambda t: R.rms_norm(t, 0.7), x)


def test_rope_is_a_rotation_and_partial():
    cos, sin = R.rope_tables(6, 4)
    x = torch.randn(2, 6, 3, 8)
    y = R.apply_rope(x, cos, sin, 4)
    assert torch.allclose(y[..., 4:], x[..., 4:])
    assert torch.allclose(y[..., :4].norm(dim=-1), x[..., :4].norm(dim=-1), atol=1e-5)
    assert torch.allclose(y[:, 0], x[:, 0])              # position 0 is the identity
    _gc(lambda t: R.apply_rope(t, cos.double(), sin.double(), 4), x)


def test_yarn_tables_slow_down_the_low_frequencies_only():
    """The ramp of the ternary record (train_gpt_cuda_ternary.py:570-575): the first quarter of the frequency pairs is left
    alone, the last one is slowed down by exactly yarn_max_len / train_seq_len, and the ones between are ramped linearly."""
    rd, S = 16, 64
    plain = R.rope_tables(S, rd, 5000.0)
    yarn = R.rope_tables(S, rd, 5000.0, train_seq_len=1024, yarn_max_len=2048)
    idx = torch.arange(0, rd, 2, dtype=torch.float32)
    inv = 1.0 / (5000.0 ** (idx / rd))
    ramp = torch.clamp((idx / rd - 0.25) / 0.75, 0.0, 1.0)
    want = torch.outer(torch.arange(S, dtype=torch.float32), inv / (ramp * (2.0 - 1.0) + 1.0))
    assert torch.allclose(yarn[0], want.cos(), atol=1e-6) and torch.allclose(yarn[1], want.sin(), atol=1e-6)
    assert torch.equal(yarn[0][:, :2], plain[0][:, :2])             # index / rd <= 0.25: untouched
    assert not torch.allclose(yarn[0][:, -1], plain[0][:, -1])
    # through the model spec
    from parameter_golf_b200.spec import family_preset
    m = family_preset("tiny_cpu").apply_overrides(["model.rope.mode=yarn", "model.rope.yarn_max_len=4096"]).validate().model
    c, s_ = R.model_rope_tables(m, 32)
    c2, s2 = R.rope_tables(32, m.rope_dims, m.rope.base, train_seq_len=1024, yarn_max_len=4096)
    assert torch.equal(c, c2) and torch.equal(s_, s2)


def test_rope_ntk_rescale_only_beyond_train_len():
    a = R.rope_tables(16, 8, 10000.0, train_seq_len=16)[0]
    b = R.rope_tables(16, 8, 10000.0, train_seq_len=0)[0]
    c = R.rope_tables(32, 8, 10000.0, train_seq_len=16)[0]
    assert torch.equal(a, b) and not torch.allclose(c[:16], a)


def test_attention_matches_sdpa_and_is_causal():
    B, T, H, Hkv, D = 2, 7, 4, 2, 8
    q, k, v = torch.randn(B, T, H, D), torch.randn(B, T, Hkv, D), torch.randn(B, T, Hkv, D)
    y = R.causal_gqa_attention(q, k, v)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2).repeat_interleave(2, 1), v.transpose(1, 2).repeat_interleave(2, 1), is_causal=True).transpose(1, 2)
    assert torch.allclose(y, ref, atol=1e-5)
    k2, v2 = k.clone(), v.clone()
    k2[:, 5:] += 3.0
    v2[:, 5:] -= 2.0
    assert torch.allclose(R.causal_gqa_attention(q, k2, v2)[:, :5], y[:, :5], atol=1e-6)
    _gc(R.causal_gqa_attention, q[:1, :4], k[:1, :4], v[:1, :4])


def test_xsa_removes_value_component():
    y, v = torch.randn(2, 3, 4, 8), torch.randn(2, 3, 2, 8)
    z = R.xsa(y, v)
    vv = v.repeat_interleave(2, dim=2)
    assert (z * vv).sum(-1).abs().max() < 1e-4
    _gc(R.xsa, y, v)


def test_gates():
    y, h = torch.randn(2, 3, 4, 8), torch.randn(2, 3, 16)
    w = torch.zeros(4, 6)
    assert torch.allclose(R.attn_out_gate(y, h, w, torch.zeros(4)), y)           # 2*sigmoid(0) = 1
    assert torch.allclose(R.sparse_attn_gate(y, h, w, 1.0), 0.5 * y)
    _gc(lambda a, b, c, d: R.attn_out_gate(a, b, c, d), y, h, torch.randn(4, 6), torch.randn(4))
    _gc(lambda a, b, c: R.sparse_attn_gate(a, b, c, 0.7), y, h, torch.randn(4, 6))


def test_smear_gate_boundaries_do_not_leak():
    x = torch.randn(2, 5, 4)
    g = torch.full((4,), 0.3)
    out = R.smear_gate(x, g)
    s = torch.sigmoid(g)
    assert torch.allclose(out[:, 0], (1 - s) * x[:, 0])                          # sequence start: previous is zero
    assert torch.allclose(out[:, 2], (1 - s) * x[:, 2] + s * x[:, 1])
    ids = torch.tensor([[5, 1, 7, 1, 2], [1, 1, 3, 4, 5]])
    ob = R.smear_gate(x, g, ids, boundary_id=1)
    assert torch.allclose(ob[0, 1], (1 - s) * x[0, 1])                           # current token is the boundary id
    assert torch.allclose(ob[0, 2], (1 - s) * x[0, 2] + s * x[0, 1])
    x2 = x.clone()
    x2[0, 0] += 10
    assert torch.allclose(R.smear_gate(x2, g, ids, 1)[0, 1], ob[0, 1])           # nothing crosses the boundary
    _gc(lambda a, b: R.smear_gate(a, b), x, g)


def test_bigram_hash_rule():
    ids = torch.tensor([[3, 9, 1023, 0]])
    h = R.bigram_hash(ids, 3072)
    assert h[0, 0] == 3071
    for t in range(1, 4):
        exp = (((36313 * int(ids[0, t])) & 0xFFFFFFFF) ^ ((27191 * int(ids[0, t - 1])) & 0xFFFFFFFF)) % 3071
        assert int(h[0, t]) == exp
    big = torch.tensor([[65535, 65535]])
    assert 0 <= int(R.bigram_hash(big, 2048)[0, 1]) < 2047


def test_act_sq_and_grad():
    x = torch.tensor([-2.0, -0.5, 0.0, 1.5])
    assert torch.allclose(R.act_sq(x, 0.5), torch.tensor([1.0, 0.0625, 0.0, 2.25]))
    assert torch.allclose(R.act_sq(x, 0.0), torch.tensor([0.0, 0.0, 0.0, 2.25]))
    _gc(lambda t: R.act_sq(t, 0.5), torch.randn(10) + 0.3)


def test_softcap_cross_entropy():
    z = torch.randn(6, 11) * 20
    t = torch.randint(0, 11, (6,))
    c = 30 * torch.tanh(z / 30)
    ref = (torch.logsumexp(c, -1) - c[torch.arange(6), t]).mean()
    assert torch.allclose(R.softcap_cross_entropy(z, t, 30.0), ref, atol=1e-6)
    assert R.softcap_cross_entropy(z, t, 30.0, "none").shape == (6,)
    _gc(lambda a: R.softcap_cross_entropy(a, t, 30.0), z)


def test_fake_quant_ste_forward_and_gradient():
    torch.manual_seed(7)
    w = torch.randn(4, 16, requires_grad=True)
    wq = R.fake_quant_int6_ste(w)
    scale = (w.detach().abs().amax(1, keepdim=True) / 31).clamp_min(1 / 31)
    codes = wq.detach() / scale
    assert torch.allclose(codes, codes.round(), atol=1e-5) and codes.min() >= -32 - 1e-4 and codes.max() <= 31 + 1e-4
    wq.sum().backward()
    assert torch.allclose(w.grad, torch.ones_like(w))


def test_polynomial_softcap_and_z_loss():
    """poly5: x (1 - x^2/3 + x^4/15) of the clamped ratio, within [-cap, cap], odd, close to tanh for small arguments; the
    z-loss adds weight * mean(logsumexp^2) to the mean loss only (train_gpt_cuda_ternary.py:859-865, :903-906)."""
    import torch.nn.functional as F
    z = torch.linspace(-40, 40, 801)
    c = R.softcap(z, 10.0, "poly5")
    assert float(c.abs().max()) <= 10.0 + 1e-6 and torch.allclose(c, -R.softcap(-z, 10.0, "poly5"))
    small = torch.linspace(-3, 3, 61)
    assert torch.allclose(R.softcap(small, 10.0, "poly5"), R.softcap(small, 10.0, "tanh"), atol=2e-3)
    x = torch.tensor([0.5])
    assert torch.allclose(R.softcap(10.0 * x, 10.0, "poly5"), 10.0 * x * (1 - x ** 2 / 3 + x ** 4 / 15))
    logits, tgt = torch.randn(4, 7, 13) * 5, torch.randint(0, 13, (4, 7))
    base = R.softcap_cross_entropy(logits, tgt, 10.0, kind="poly5")
    capped = R.softcap(logits, 10.0, "poly5").reshape(-1, 13)
    assert torch.allclose(base, F.cross_entropy(capped, tgt.reshape(-1)))
    with_z = R.softcap_cross_entropy(logits, tgt, 10.0, kind="poly5", z_loss=1e-2)
    assert torch.allclose(with_z, base + 1e-2 * torch.logsumexp(capped, -1).pow(2).mean())
    assert R.softcap_cross_entropy(logits, tgt, 10.0, reduction="none", z_loss=1.0).shape == (28,)
    _gc(lambda t: R.softcap(t, 10.0, "poly5"), torch.randn(3, 5) * 8)
