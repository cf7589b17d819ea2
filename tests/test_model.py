import copy

import pytest
import torch

from parameter_golf_b200.models import gpt
from parameter_golf_b200.spec import family_preset


def tiny(**ov):
    s = family_preset("tiny_cpu")
    m = s.model
    m.vocab_size, m.num_layers, m.model_dim, m.num_heads, m.num_kv_heads, m.mlp_mult = 32, 3, 16, 4, 2, 2.0
    s.apply_overrides([f"model.{k}={v}" for k, v in ov.items()])
    return s.validate().model


FULL = dict(xsa_last_n=2, ln_scale="true", smear_gate="true", activation="leaky_relu_sq")


def full_model():
    m = tiny(**FULL)
    m.bigram.enabled, m.bigram.vocab_size, m.bigram.dim = True, 24, 8
    m.value_embedding.enabled, m.value_embedding.dim, m.value_embedding.layers = True, 8, [1, 2]
    m.rope.dims = 2
    return m


def test_shapes_and_count():
    m = full_model()
    sh = gpt.param_shapes(m)
    assert sh["qo_bank"] == (6, 16, 16) and sh["kv_bank"] == (6, 8, 16) and sh["mlp_up_bank"] == (3, 32, 16)
    assert sh["skip_weights"] == (1, 16) and sh["bigram_proj"] == (16, 8) and sh["ve_proj"] == (8, 8)
    p = gpt.init_params(m)
    assert sum(v.numel() for v in p.values()) == gpt.count_params(m)
    assert p["qo_bank"][3:].abs().max() == 0 and p["mlp_down_bank"].abs().max() == 0          # zero-init projections
    q = p["qo_bank"][0]
    assert torch.allclose(q @ q.t(), torch.eye(16), atol=1e-5)                                  # orthogonal init


def test_bank_slices_are_zero_copy_and_overlap_guard():
    m = tiny()
    p = gpt.init_params(m)
    v = gpt.bank_views(m, p)
    assert v["qo_bank.o"].data_ptr() == p["qo_bank"][3].data_ptr()
    assert gpt.overlaps_storage(p["qo_bank"][1], p["qo_bank"])
    assert not gpt.overlaps_storage(p["qo_bank"][0], p["qo_bank"][1])
    assert not gpt.overlaps_storage(p["qo_bank"], p["kv_bank"])


def test_finite_loss_near_uniform_at_init():
    m = full_model()
    p = gpt.init_params(m)
    ids = torch.randint(0, 32, (2, 12))
    loss = gpt.gpt_forward(m, p, ids, ids)
    assert torch.isfinite(loss) and abs(float(loss) - torch.log(torch.tensor(32.0))) < 0.1


def test_model_is_causal_and_batch_rows_independent():
    m = full_model()
    p = gpt.fill_deterministic(m)
    ids = torch.randint(0, 32, (2, 10))
    a = gpt.gpt_logits(m, p, ids)
    ids2 = ids.clone()
    ids2[0, 7:] = (ids2[0, 7:] + 5) % 32
    b = gpt.gpt_logits(m, p, ids2)
    assert torch.allclose(a[0, :7], b[0, :7], atol=1e-5) and not torch.allclose(a[0, 7:], b[0, 7:])
    assert torch.allclose(a[1], b[1], atol=1e-6)


def test_identity_gates_are_no_ops():
    base = tiny()
    p = gpt.fill_deterministic(base)
    ids = torch.randint(0, 32, (1, 8))
    ref = gpt.gpt_logits(base, p, ids)
    g = tiny()
    g.attn_out_gate.enabled = True
    pg = dict(p, attn_gate_weight=torch.zeros(3, 4, g.attn_out_gate.width), attn_gate_bias=torch.zeros(3, 4))
    assert torch.allclose(gpt.gpt_logits(g, pg, ids), ref, atol=1e-6)
    s = tiny(smear_gate="true")
    ps = dict(p, smear_gate=torch.full((16,), -40.0))
    assert torch.allclose(gpt.gpt_logits(s, ps, ids), ref, atol=1e-5)


def test_recurrence_runs_block_twice():
    m = tiny()
    m.recurrence.enabled, m.recurrence.start_layer, m.recurrence.repeat_layers = True, 1, 1
    assert gpt.layer_schedule(m) == [(0, 0), (1, 0), (1, 1), (2, 0)]
    p = gpt.fill_deterministic(m)
    ids = torch.randint(0, 32, (1, 8))
    assert not torch.allclose(gpt.gpt_logits(m, p, ids), gpt.gpt_logits(tiny(), p, ids))


def test_numerical_gradient_of_tok_emb_and_bank():
    m = full_model()
    p = {k: v.double() for k, v in gpt.fill_deterministic(m).items()}
    ids = torch.randint(0, 32, (2, 6))
    tgt = torch.randint(0, 32, (2, 6))
    for name, idx in (("tok_emb", (int(ids[0, 0]), 3)), ("qo_bank", (4, 2, 5)), ("resid_mix", (1, 1, 3)), ("bigram_scale", (0,))):
        leaf = p[name].clone().requires_grad_(True)
        loss = gpt.gpt_forward(m, dict(p, **{name: leaf}), ids, tgt)
        (g,) = torch.autograd.grad(loss, leaf)
        eps = 1e-5
        pp, pm = p[name].clone(), p[name].clone()
        pp[idx] += eps
        pm[idx] -= eps
        fd = (gpt.gpt_forward(m, dict(p, **{name: pp}), ids, tgt) - gpt.gpt_forward(m, dict(p, **{name: pm}), ids, tgt)) / (2 * eps)
        assert abs(float(fd) - float(g[idx])) < 1e-3 * max(1.0, abs(float(fd))), name


def test_qat_forward_differs_but_trains():
    m = tiny()
    p = gpt.fill_deterministic(m)
    ids = torch.randint(0, 32, (1, 8))
    a = gpt.gpt_forward(m, p, ids, ids)
    b = gpt.gpt_forward(m, p, ids, ids, qat=True)
    assert torch.isfinite(b) and abs(float(a) - float(b)) < 0.2 and float(a) != float(b)


def test_lora_with_zero_b_is_identity():
    from parameter_golf_b200.eval.ttt import init_q_lora
    m = tiny()
    p = gpt.fill_deterministic(m)
    ids = torch.randint(0, 32, (1, 8))
    lora = init_q_lora(m, 4, 4.0)
    assert torch.allclose(gpt.gpt_logits(m, p, ids, lora=lora), gpt.gpt_logits(m, p, ids), atol=1e-6)


def test_value_residual_mixes_the_first_layers_values_into_later_layers():
    """records/.../2026-03-23_.../train_gpt.py:655-658: layer 0 is unchanged; with lambda = (0, 1) the model is the plain one;
    the lambdas get gradients and match a finite difference."""
    m0, m1 = full_model(), full_model()
    m1.value_residual = True
    p1 = {k: v.double() for k, v in gpt.fill_deterministic(m1).items()}
    assert p1["vr_lambda"].shape == (3, 2)
    ids = torch.randint(0, 32, (2, 7))
    tgt = torch.randint(0, 32, (2, 7))
    p0 = {k: v for k, v in p1.items() if k != "vr_lambda"}
    ident = dict(p1, vr_lambda=torch.tensor([[0.0, 1.0]] * 3, dtype=torch.float64))
    assert torch.allclose(gpt.gpt_forward(m1, ident, ids, tgt), gpt.gpt_forward(m0, p0, ids, tgt), atol=1e-12)
    assert abs(float(gpt.gpt_forward(m1, p1, ids, tgt)) - float(gpt.gpt_forward(m0, p0, ids, tgt))) > 1e-6
    leaf = p1["vr_lambda"].clone().requires_grad_(True)
    (g,) = torch.autograd.grad(gpt.gpt_forward(m1, dict(p1, vr_lambda=leaf), ids, tgt), leaf)
    assert float(g[0].abs().max()) == 0.0                      # the first layer has nothing to mix with
    for idx in ((1, 0), (2, 1)):
        eps = 1e-6
        pp, pm = p1["vr_lambda"].clone(), p1["vr_lambda"].clone()
        pp[idx] += eps
        pm[idx] -= eps
        fd = (gpt.gpt_forward(m1, dict(p1, vr_lambda=pp), ids, tgt) - gpt.gpt_forward(m1, dict(p1, vr_lambda=pm), ids, tgt)) / (2 * eps)
        assert abs(float(fd) - float(g[idx])) < 1e-4 * max(1.0, abs(float(fd)))


def test_multi_token_prediction_heads_add_a_training_only_loss():
    """records/.../2026-03-23_.../train_gpt.py:947-962: head k scores the token k + 2 ahead from the final hidden state; the
    term is weighted, averaged over the heads and left out of evaluation."""
    import torch.nn.functional as F
    from parameter_golf_b200.ops import reference as R
    m = full_model()
    m.mtp_num_heads, m.mtp_loss_weight = 2, 0.3
    p = {k: v.double() for k, v in gpt.fill_deterministic(m).items()}
    assert p["mtp_heads"].shape == (2, 32, 16)
    ids = torch.randint(0, 32, (2, 9))
    tgt = torch.randint(0, 32, (2, 9))
    base = gpt.gpt_forward(m, p, ids, tgt)
    with_mtp = gpt.gpt_forward(m, p, ids, tgt, mtp=True)
    h = gpt.gpt_hidden(m, p, ids)
    want = 0.0
    for k in range(2):
        z = F.linear(h[:, :9 - (k + 1)], p["mtp_heads"][k])
        want = want + R.softcap_cross_entropy(z, tgt[:, k + 1:], m.logit_softcap)
    assert torch.allclose(with_mtp, base + 0.3 * want / 2, atol=1e-12)
    assert gpt.gpt_forward(m, p, ids, tgt, reduction="none").shape == (2, 9)             # evaluation path: no extra term
    leaf = p["mtp_heads"].clone().requires_grad_(True)
    (g,) = torch.autograd.grad(gpt.gpt_forward(m, dict(p, mtp_heads=leaf), ids, tgt, mtp=True), leaf)
    assert float(g[0].abs().max()) > 0 and float(g[1].abs().max()) > 0
    assert gpt.init_params(m)["mtp_heads"].abs().max() == 0                                # zero-initialised heads


def test_dtg_gate_scales_the_block_update_and_reads_a_detached_input():
    """records/.../2026-03-23_.../train_gpt.py:757-771: out = x_in + sigmoid(w . x_in + b) * (block(x_in) - x_in); a large bias
    makes it the plain block, and the gate's input carries no gradient."""
    m0, m1 = full_model(), full_model()
    m1.dtg = True
    p1 = {k: v.double() for k, v in gpt.fill_deterministic(m1).items()}
    assert p1["dtg_gate_weight"].shape == (3, 16) and gpt.init_params(m1)["dtg_gate_bias"].tolist() == [2.0] * 3
    ids = torch.randint(0, 32, (2, 7))
    tgt = torch.randint(0, 32, (2, 7))
    p0 = {k: v for k, v in p1.items() if not k.startswith("dtg_")}
    open_gate = dict(p1, dtg_gate_weight=torch.zeros(3, 16, dtype=torch.float64), dtg_gate_bias=torch.full((3,), 40.0, dtype=torch.float64))
    assert torch.allclose(gpt.gpt_forward(m1, open_gate, ids, tgt), gpt.gpt_forward(m0, p0, ids, tgt), atol=1e-10)
    assert abs(float(gpt.gpt_forward(m1, p1, ids, tgt)) - float(gpt.gpt_forward(m0, p0, ids, tgt))) > 1e-6
    # the last block's gate: no later gate reads (through its detached input) what this one changes, so a finite difference
    # sees exactly what autograd sees
    for name, idx in (("dtg_gate_weight", (2, 3)), ("dtg_gate_bias", (2,))):
        leaf = p1[name].clone().requires_grad_(True)
        (g,) = torch.autograd.grad(gpt.gpt_forward(m1, dict(p1, **{name: leaf}), ids, tgt), leaf)
        eps = 1e-6
        pp, pm = p1[name].clone(), p1[name].clone()
        pp[idx] += eps
        pm[idx] -= eps
        fd = (gpt.gpt_forward(m1, dict(p1, **{name: pp}), ids, tgt) - gpt.gpt_forward(m1, dict(p1, **{name: pm}), ids, tgt)) / (2 * eps)
        assert abs(float(fd) - float(g[idx])) < 1e-4 * max(1.0, abs(float(fd))), name


@pytest.mark.parametrize("value_residual", [False, True])
def test_cached_generation_follows_the_full_forward(value_residual):
    """At a vanishing temperature the K/V-cached sampler must pick the arg-max of the full model's logits at every step."""
    from parameter_golf_b200.quant.calibrate import generate_autoregressive
    m = full_model()
    m.value_residual = value_residual
    m.dtg = value_residual                                     # the gated block update rides along in the same variant
    p = gpt.fill_deterministic(m)
    p["tok_emb"] = p["tok_emb"] * 4.0                           # wider logit margins than the fill pattern gives
    toks = generate_autoregressive(m, p, num_seqs=3, seq_len=10, temperature=1e-4, seed=5)
    logits = gpt.gpt_logits(m, p, toks)
    top2 = logits.topk(2, dim=-1).values
    decided = (top2[..., 0] - top2[..., 1]) > 1e-3              # skip near-ties, where fp32 summation order decides
    pred = logits.argmax(-1)[:, :-1]
    same = (pred == toks[:, 1:]) | ~decided[:, :-1]
    assert bool(same.all()) and int(decided[:, :-1].sum()) >= 20


def test_factored_tied_embedding_projects_in_and_out():
    """model.embed_dim: the table is [V, e]; the input goes through embed_proj_in, the tied output through embed_proj_out
    first. With e = d and identity projections the model is the unfactored one; the projections get gradients; the cached
    sampler follows the full forward."""
    import torch.nn.functional as F
    from parameter_golf_b200.quant.calibrate import generate_autoregressive
    m0, m1 = full_model(), full_model()
    m1.embed_dim = 16
    p0 = {k: v.double() for k, v in gpt.fill_deterministic(m0).items()}
    eye = torch.eye(16, dtype=torch.float64)
    p1 = dict(p0, embed_proj_in=eye, embed_proj_out=eye)
    ids = torch.randint(0, 32, (2, 7))
    tgt = torch.randint(0, 32, (2, 7))
    assert torch.allclose(gpt.gpt_forward(m1, p1, ids, tgt), gpt.gpt_forward(m0, p0, ids, tgt), atol=1e-12)
    m2 = full_model()
    m2.embed_dim = 6
    sh = gpt.param_shapes(m2)
    assert sh["tok_emb"] == (32, 6) and sh["embed_proj_in"] == (16, 6) and sh["embed_proj_out"] == (6, 16)
    init = gpt.init_params(m2)
    assert torch.allclose(init["embed_proj_in"].t() @ init["embed_proj_in"], torch.eye(6), atol=1e-5)
    assert torch.equal(init["embed_proj_out"], init["embed_proj_in"].t())
    p2 = {k: v.double() for k, v in gpt.fill_deterministic(m2).items()}
    h = gpt.gpt_hidden(m2, p2, ids)
    want = m2.logit_softcap * torch.tanh(F.linear(F.linear(h, p2["embed_proj_out"]), p2["tok_emb"]) / m2.logit_softcap)
    assert torch.allclose(gpt.gpt_logits(m2, p2, ids).double(), want, atol=1e-6)
    leaves = {k: p2[k].clone().requires_grad_(True) for k in ("embed_proj_in", "embed_proj_out", "tok_emb")}
    gs = torch.autograd.grad(gpt.gpt_forward(m2, dict(p2, **leaves), ids, tgt), list(leaves.values()))
    assert all(float(g.abs().max()) > 0 for g in gs)
    pf = gpt.fill_deterministic(m2)
    pf["tok_emb"] = pf["tok_emb"] * 6.0
    toks = generate_autoregressive(m2, pf, num_seqs=2, seq_len=8, temperature=1e-4, seed=1)
    logits = gpt.gpt_logits(m2, pf, toks)
    top2 = logits.topk(2, dim=-1).values
    decided = (top2[..., 0] - top2[..., 1]) > 1e-3
    assert bool(((logits.argmax(-1)[:, :-1] == toks[:, 1:]) | ~decided[:, :-1]).all())


def _variant(*ov):
    s = family_preset("tiny_cpu")
    s.apply_overrides(list(ov))
    s.validate()
    return s


def test_swiglu_normed_projections_block_smear_and_vocab_bias_match_plain_statements():
    """The options of the ternary / binary submissions' blocks (train_gpt_cuda_binary.py:617-656, :692-700) against statements
    written out here: SwiGLU with the gate in the first half of the up projection, RMSNorm in front of the two output
    projections, the running-mean smear at the end of every block, a bias per vocabulary entry on the logits."""
    import torch.nn.functional as F
    from parameter_golf_b200.ops import reference as R
    s = _variant("model.activation=swiglu", "model.normed_out_proj=true", "model.block_smear=true", "model.vocab_bias=true", "model.skip_topology=none")
    m = s.model
    shapes = gpt.param_shapes(m)
    assert shapes["mlp_up_bank"] == (m.num_layers, 2 * m.mlp_dim, m.model_dim) and shapes["block_smear_gate"] == (m.num_layers, m.model_dim)
    assert shapes["vocab_bias"] == (m.vocab_size,)
    p = gpt.fill_deterministic(m)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, m.vocab_size, (2, 24), generator=g)
    n, H, Hkv, D, d = m.num_layers, m.num_heads, m.num_kv_heads, m.head_dim, m.model_dim
    x = R.rms_norm(p["tok_emb"][ids])
    x0 = x
    cos, sin = R.model_rope_tables(m, 24)
    for i in range(n):
        x_in = p["resid_mix"][i][0] * x + p["resid_mix"][i][1] * x0
        h = R.rms_norm(x_in)
        q = F.linear(h, p["qo_bank"][i]).reshape(2, 24, H, D)
        k = F.linear(h, p["kv_bank"][i]).reshape(2, 24, Hkv, D)
        v = F.linear(h, p["kv_bank"][n + i]).reshape(2, 24, Hkv, D)
        q, k = R.qk_norm_rope_gain(q, k, cos, sin, m.rope_dims, p["q_gain"][i])
        y = R.causal_gqa_attention(q, k, v).reshape(2, 24, d)
        y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + 1e-6)
        x_mid = x_in + p["attn_scale"][i] * F.linear(y, p["qo_bank"][n + i])
        u = F.linear(R.rms_norm(x_mid), p["mlp_up_bank"][i])
        hid = F.silu(u[..., : m.mlp_dim]) * u[..., m.mlp_dim:]
        hid = hid * torch.rsqrt(hid.pow(2).mean(-1, keepdim=True) + 1e-6)
        out = x_mid + p["mlp_scale"][i] * F.linear(hid, p["mlp_down_bank"][i])
        mean = torch.stack([out[:, : t + 1].mean(1) for t in range(24)], dim=1)
        x = out + torch.tanh(p["block_smear_gate"][i]) * (mean - out)
    z = F.linear(R.rms_norm(x), p["tok_emb"]) + p["vocab_bias"]
    want = R.softcap(z, m.logit_softcap, m.softcap_kind)
    got = gpt.gpt_logits(m, p, ids)
    assert torch.allclose(got, want, atol=2e-5), float((got - want).abs().max())
    # the smear is causal: changing the last token leaves every earlier position as it was
    ids2 = ids.clone()
    ids2[:, -1] = (ids2[:, -1] + 1) % m.vocab_size
    assert torch.allclose(gpt.gpt_logits(m, p, ids2)[:, :-1], got[:, :-1], atol=1e-6)
    # a zero gate and a zero bias are the identity
    p0 = dict(p, block_smear_gate=torch.zeros_like(p["block_smear_gate"]), vocab_bias=torch.zeros_like(p["vocab_bias"]))
    plain = _variant("model.activation=swiglu", "model.normed_out_proj=true", "model.skip_topology=none").model
    assert torch.allclose(gpt.gpt_logits(m, p0, ids), gpt.gpt_logits(plain, {k: v for k, v in p0.items() if k in gpt.param_shapes(plain)}, ids), atol=1e-6)
    with pytest.raises(ValueError):
        family_preset("record_11l").apply_overrides(["model.activation=swiglu"]).validate()


def test_cached_generation_follows_the_block_options():
    """Self-generated calibration decodes with a K/V cache; with the block smear it also keeps a running sum per block. Greedy-free
    check: the logits of the cached decoder at every step equal the full forward's at that position (same seed, same tokens)."""
    from parameter_golf_b200.quant.calibrate import generate_autoregressive
    s = _variant("model.activation=swiglu", "model.normed_out_proj=true", "model.block_smear=true", "model.vocab_bias=true")
    m = s.model
    p = gpt.fill_deterministic(m)
    toks = generate_autoregressive(m, p, 2, 12, temperature=0.8, seed=7)
    again = generate_autoregressive(m, p, 2, 12, temperature=0.8, seed=7)
    assert torch.equal(toks, again) and toks.shape == (2, 12)
    # replay: sampling position t + 1 from the full forward's distribution at t with the same generator state gives the same tokens
    g = torch.Generator().manual_seed(7)
    first = torch.randint(0, m.vocab_size, (2,), generator=g)
    assert torch.equal(first, toks[:, 0])
    for t in range(11):
        z = gpt.gpt_logits(m, p, toks[:, : t + 1])[:, -1]
        nxt = torch.multinomial(torch.softmax(z / 0.8, -1), 1, generator=g)[:, 0]
        assert torch.equal(nxt, toks[:, t + 1]), t


def test_cycled_blocks_with_per_depth_adapters_match_an_unrolled_model():
    """Three unique blocks cycled to seven virtual layers (…DepthRecurrence…/train_gpt.py:863, :897-919): the same function as a
    seven-block model whose blocks are copies in round-robin order, with the U-Net split, skip weights and XSA flags counted on
    virtual layers; the per-depth adapters start as no-ops and, once their up halves are non-zero, add h A^T B^T to q and v."""
    s = _variant("model.num_layers=3", "model.recurrence.enabled=true", "model.recurrence.effective_depth=7", "model.xsa_last_n=2",
                 "model.recurrence.depth_lora_rank=2")
    m = s.model
    assert gpt.layer_schedule(m) == [(0, 0), (1, 0), (2, 0), (0, 1), (1, 1), (2, 1), (0, 2)] and m.depth == 7
    assert m.xsa_layers() == [0, 2]                      # virtual layers 5 and 6 are blocks 2 and 0
    assert gpt.shared_layers(m) == {0, 1, 2}
    shapes = gpt.param_shapes(m)
    assert shapes["skip_weights"] == (3, m.model_dim) and shapes["depth_lora_v_up"] == (7, m.kv_dim, 2)
    p = gpt.fill_deterministic(m)
    p0 = dict(p, depth_lora_q_up=torch.zeros_like(p["depth_lora_q_up"]), depth_lora_v_up=torch.zeros_like(p["depth_lora_v_up"]))
    ids = torch.randint(0, m.vocab_size, (2, 16), generator=torch.Generator().manual_seed(1))
    flat = _variant("model.num_layers=7", "model.xsa_last_n=0").model
    order = [v % 3 for v in range(7)]
    pf = {k: v for k, v in p0.items() if not k.startswith("depth_lora")}
    n = 3
    pf["qo_bank"] = torch.cat([p["qo_bank"][order], p["qo_bank"][[n + i for i in order]]])
    pf["kv_bank"] = torch.cat([p["kv_bank"][order], p["kv_bank"][[n + i for i in order]]])
    for k in ("mlp_up_bank", "mlp_down_bank", "attn_scale", "mlp_scale", "resid_mix", "q_gain"):
        pf[k] = p[k][order]
    assert {k: tuple(v.shape) for k, v in pf.items()} == gpt.param_shapes(flat)
    flat.xsa_last_n = 0
    real_xsa = type(flat).xsa_layers
    try:
        type(flat).xsa_layers = lambda self: [0, 2, 3, 5, 6] if self is flat else real_xsa(self)     # where blocks 0 and 2 sit when unrolled
        want = gpt.gpt_logits(flat, pf, ids)
    finally:
        type(flat).xsa_layers = real_xsa
    got = gpt.gpt_logits(m, p0, ids)
    assert torch.allclose(got, want, atol=1e-5), float((got - want).abs().max())
    moved = gpt.gpt_logits(m, p, ids)
    assert float((moved - got).abs().max()) > 1e-4
    # the adapters of one virtual layer do not touch the other executions of the same block: gradient lands on that slice only
    pg = {k: v.clone().requires_grad_(True) for k, v in p.items()}
    gpt.gpt_forward(m, pg, ids, ids).backward()
    assert all(float(pg["depth_lora_q_up"].grad[v].abs().max()) > 0 for v in range(7))
    with pytest.raises(ValueError):
        family_preset("record_11l").apply_overrides(["model.recurrence.enabled=true", "model.recurrence.effective_depth=22"]).validate()
    with pytest.raises(ValueError):
        _variant("model.recurrence.depth_lora_rank=2")


def test_noisy_qat_perturbs_shared_blocks_by_one_quantisation_step_with_gradients():
    from parameter_golf_b200.ops import reference as R
    torch.manual_seed(0)
    w = torch.randn(8, 64, requires_grad=True)
    out = R.quant_noise(w, 127)
    step = w.detach().abs().amax(-1, keepdim=True) / 127
    delta = (out - w).detach()
    assert float((delta.abs() / step).max()) <= 0.5 + 1e-6 and float(delta.abs().mean()) > 0
    assert abs(float((delta / step).std()) - (1 / 12) ** 0.5) < 0.03            # uniform over one step
    (g,) = torch.autograd.grad(out.sum(), w)
    assert torch.equal(g, torch.ones_like(w))
    s = _variant("model.recurrence.enabled=true", "model.recurrence.start_layer=1", "model.recurrence.repeat_layers=1", "model.qat_kind=noise")
    m = s.model
    assert gpt.shared_layers(m) == {1}
    p = gpt.fill_deterministic(m)
    ids = torch.randint(0, m.vocab_size, (2, 16), generator=torch.Generator().manual_seed(2))
    clean = gpt.gpt_forward(m, p, ids, ids)
    torch.manual_seed(3)
    a = gpt.gpt_forward(m, p, ids, ids, qat=True)
    torch.manual_seed(3)
    b = gpt.gpt_forward(m, p, ids, ids, qat=True)
    assert torch.equal(a, b) and float((a - clean).abs()) > 0
    # only the block that runs twice is perturbed: with its weights zeroed out of the picture the loss is the clean one
    calls = []
    real = R.quant_noise
    try:
        R.quant_noise = lambda w_, q_: calls.append(tuple(w_.shape)) or real(w_, q_)
        gpt.gpt_forward(m, p, ids, ids, qat=True)
    finally:
        R.quant_noise = real
    assert len(calls) == 2 * 6                                                  # six matrices, two passes of block 1, nothing else


def test_overtone_embedding_spectrum_and_phase_residual_mix_initialisation():
    """…OvertoneInit/train_gpt.py:723-737: the tied table keeps its random singular vectors and gets singular values
    s_1 / sqrt(k); resid_mix starts at sigmoid(3 (l / (n - 1) - 1/2)) on the residual stream and the rest on the embedding stream."""
    s = _variant("model.num_layers=5", "model.embed_init=overtone", "model.resid_mix_init=phase")
    m = s.model
    p = gpt.init_params(m, seed=11)
    S = torch.linalg.svdvals(p["tok_emb"])
    k = torch.arange(1, S.numel() + 1, dtype=S.dtype)
    assert torch.allclose(S, S[0] * k.rsqrt(), rtol=1e-4)
    ref = gpt.init_params(_variant("model.num_layers=5").model, seed=11)
    assert torch.allclose(torch.linalg.svdvals(ref["tok_emb"])[0], S[0], rtol=1e-5)         # the largest one is the random table's
    want = torch.sigmoid(3.0 * (torch.arange(5) / 4 - 0.5))
    assert torch.allclose(p["resid_mix"][:, 0, 0], want) and torch.allclose(p["resid_mix"][:, 1, 3], 1 - want)
    assert torch.equal(ref["resid_mix"][:, 0], torch.ones(5, m.model_dim)) and float(ref["resid_mix"][:, 1].abs().max()) == 0.0
    assert torch.equal(p["kv_bank"], ref["kv_bank"])                                          # nothing else moves


def test_gated_attention_trigram_hash_and_repeat_count():
    """GATED_ATTENTION (records/.../2026-03-23_.../train_gpt.py:629-633, :668-671), TRIGRAM (…2026-03-25_…:698-710) and blocks that
    run r times in a row (TRAINING_DEPTH_RECURRENCE of the ternary record), on the autograd model."""
    import torch.nn.functional as F
    from parameter_golf_b200.ops import reference as R
    from parameter_golf_b200.quant.calibrate import generate_autoregressive
    s = _variant("model.gated_attention=true", "model.bigram.enabled=true", "model.bigram.vocab_size=64", "model.bigram.dim=16", "model.bigram.trigram=true")
    m = s.model
    p = gpt.init_params(m, seed=2)
    assert p["gated_attn_weight"].shape == (m.num_layers, m.num_heads, m.model_dim) and float(p["gated_attn_weight"].abs().max()) == 0.0
    assert torch.equal(p["gated_attn_bias"], torch.full((m.num_layers, m.num_heads), 4.0))
    ids = torch.randint(0, m.vocab_size, (2, 20), generator=torch.Generator().manual_seed(0))
    # at initialisation every gate is sigmoid(4): the ungated model's attention output times that constant
    pd = gpt.fill_deterministic(m)
    pd["gated_attn_weight"].zero_()
    pd["gated_attn_bias"].fill_(4.0)
    plain = _variant("model.bigram.enabled=true", "model.bigram.vocab_size=64", "model.bigram.dim=16", "model.bigram.trigram=true").model
    pp = {k: v.clone() for k, v in pd.items() if not k.startswith("gated_attn")}
    pp["qo_bank"][plain.num_layers:] *= float(torch.sigmoid(torch.tensor(4.0)))                  # fold the constant gate into W_o
    assert torch.allclose(gpt.gpt_logits(m, pd, ids), gpt.gpt_logits(plain, pp, ids), atol=2e-5)
    # the trigram row: positions 0 and 1 take the sentinel row, later ones the hash of three tokens
    h3 = R.trigram_hash(ids, 64)
    assert torch.equal(h3[:, :2], torch.full((2, 2), 63)) and int(h3.max()) <= 63 and int(h3[:, 2:].min()) >= 0
    no_tri = _variant("model.gated_attention=true", "model.bigram.enabled=true", "model.bigram.vocab_size=64", "model.bigram.dim=16").model
    pd = gpt.fill_deterministic(m)
    a, b = gpt.gpt_logits(m, pd, ids), gpt.gpt_logits(no_tri, pd, ids)
    assert float((a - b).abs().max()) > 1e-4
    pz = dict(pd, bigram_embed=pd["bigram_embed"].clone())
    pz["bigram_embed"][R.trigram_hash(ids, 64).reshape(-1).unique()] = 0                           # rows the trigram path reads
    # cached decoding follows both options
    toks = generate_autoregressive(m, pd, 2, 10, seed=3)
    g = torch.Generator().manual_seed(3)
    assert torch.equal(torch.randint(0, m.vocab_size, (2,), generator=g), toks[:, 0])
    for t in range(9):
        z = gpt.gpt_logits(m, pd, toks[:, : t + 1])[:, -1]
        assert torch.equal(torch.multinomial(torch.softmax(z / 0.8, -1), 1, generator=g)[:, 0], toks[:, t + 1]), t
    # every block three times in a row
    e = family_preset("tiny_cpu")
    e.apply_env({"TRAINING_DEPTH_RECURRENCE": "3", "GATED_ATTENTION": "1", "TRIGRAM": "1", "QAT_FRACTION": "0.25", "MUON_WEIGHT_DECAY": "0.02",
                 "MTP_HEADS": "1", "SLIDING_EVAL_STRIDE": "16", "SLIDING_BATCH_SIZE": "8", "VAL_MAX_TOKENS": "0"})
    e.validate()
    assert gpt.layer_schedule(e.model) == [(0, 0), (0, 1), (0, 2), (1, 0), (1, 1), (1, 2)] and e.train.qat_fraction == 0.25
    assert e.train.muon_wd == 0.02 and e.model.mtp_num_heads == 1 and e.eval.stride == 16 and e.eval.batch_windows == 8 and e.eval.max_tokens is None
    with pytest.raises(ValueError):
        family_preset("record_11l").apply_overrides(["model.gated_attention=true"]).validate()
    with pytest.raises(ValueError):
        family_preset("record_11l").apply_overrides(["model.recurrence.enabled=true", "model.recurrence.repeat_layers=2", "model.recurrence.repeats=3"]).validate()
