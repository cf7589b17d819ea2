"""Row kernels one by one against the fp32 statements of `parameter_golf_b200.ops.reference` (autograd for the backward
forms), at the record width (d = 512, 8 query / 4 KV heads of 64, vocabulary 1024, bigram table 3072 x 128) and at a narrow
one, with row counts that are not multiples of any tile. Counterpart of the reference's per-kernel parity binary
(``parameter-golf-rs/crates/pg-bench/src/bin/parity_kernels.rs:28-66``)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def C():
    from parameter_golf_b200.ops import native
    return native.load()


def bf(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(BF)


def close(got, ref, tol, what):
    err = (got.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item()
    assert err <= tol * scale + 1e-3 * tol, (what, err, scale)


def rel(got, ref):
    return ((got.double() - ref.double()).norm() / (ref.double().norm() + 1e-12)).item()


@pytest.mark.parametrize("rows,d", [(1037, 512), (2048 + 5, 512), (333, 128)])
@pytest.mark.parametrize("variant", ["norm", "mix", "mix_skip"])
def test_mix_norm_forward_and_backward(rows, d, variant):
    from parameter_golf_b200.ops import reference as R
    s_l, eps = 0.7, 1e-6
    x, x0, skip = bf(rows, d, seed=1), bf(rows, d, seed=2), bf(rows, d, seed=3)
    mix = torch.stack([torch.rand(d, device="cuda") + 0.5, torch.rand(d, device="cuda") * 0.3])
    sw = torch.rand(d, device="cuda") * 0.5 + 0.2
    d_h, d_res = bf(rows, d, scale=0.5, seed=4), bf(rows, d, scale=0.5, seed=5)

    xf, x0f, skf = (t.float().requires_grad_(True) for t in (x, x0, skip))
    mixf, swf = mix.clone().requires_grad_(True), sw.clone().requires_grad_(True)
    if variant == "norm":
        x_in_ref = xf
    else:
        xs = xf + swf * skf if variant == "mix_skip" else xf
        x_in_ref = mixf[0] * xs + mixf[1] * x0f
    # the kernel stores x_in in bf16 and normalises the stored value, like every consumer downstream
    x_in_q = x_in_ref + (x_in_ref.detach().to(BF).float() - x_in_ref.detach())
    h_ref = R.rms_norm(x_in_q, s_l, eps)
    # d_h arrives through the norm, d_res is the gradient the residual path hands straight to x_in
    ((h_ref * d_h.float()).sum() + (x_in_q * d_res.float()).sum()).backward()

    x_in, h = torch.empty(rows, d, device="cuda", dtype=BF), torch.empty(rows, d, device="cuda", dtype=BF)
    if variant == "norm":
        C().mix_norm_fwd(x, None, None, None, None, None, h, s_l, eps)
        x_in = x
    else:
        C().mix_norm_fwd(x, x0, skip if variant == "mix_skip" else None, sw if variant == "mix_skip" else None, mix, x_in, h, s_l, eps)
        close(x_in, x_in_ref.detach(), 0.01, "x_in")
    close(h, h_ref.detach(), 0.012, "h")

    d_x = torch.empty(rows, d, device="cuda", dtype=BF)
    if variant == "norm":
        C().mix_norm_bwd(d_h, d_res, x_in, None, None, None, None, None, None, d_x, None, None, None, None, False, s_l, eps)
        torch.cuda.synchronize()
        assert rel(d_x, xf.grad) < 0.01
        return
    base0 = bf(rows, d, scale=0.1, seed=6)
    d_x0 = base0.clone()
    d_skip = torch.empty(rows, d, device="cuda", dtype=BF) if variant == "mix_skip" else None
    d_mix = torch.zeros(2, d, device="cuda")
    d_sw = torch.zeros(d, device="cuda") if variant == "mix_skip" else None
    C().mix_norm_bwd(d_h, d_res, x_in, x, x0, skip if variant == "mix_skip" else None, sw if variant == "mix_skip" else None, mix, None, d_x, d_x0,
                     d_skip, d_mix, d_sw, False, s_l, eps)
    torch.cuda.synchronize()
    assert rel(d_x, xf.grad) < 0.012
    assert rel(d_x0.float() - base0.float(), x0f.grad) < 0.03          # accumulated into a bf16 buffer that already held values
    assert rel(d_mix, mixf.grad) < 0.01
    if variant == "mix_skip":
        assert rel(d_skip, skf.grad) < 0.012
        assert rel(d_sw, swf.grad) < 0.01


@pytest.mark.parametrize("B,S,H,Hkv,rope", [(3, 128, 8, 4, 16), (1, 640, 8, 4, 64), (2, 256, 2, 1, 16), (5, 128, 4, 4, 0)])
def test_qk_norm_rope_forward_and_backward(B, S, H, Hkv, rope):
    from parameter_golf_b200.ops import reference as R
    hd, eps = 64, 1e-6
    d, kv = H * hd, Hkv * hd
    T, qkvw = B * S, H * hd + 2 * Hkv * hd
    pre = bf(T, qkvw, seed=1)
    gain = torch.rand(H, device="cuda") + 0.8
    cos, sin = R.rope_tables(S, rope, 10000.0, device="cuda") if rope else (None, None)
    post = torch.zeros(T, qkvw, device="cuda", dtype=BF)
    C().qk_norm_rope_fwd(pre, post, cos, sin, gain, H, Hkv, hd, rope, S, eps)
    qf = pre[:, :d].float().reshape(B, S, H, hd).requires_grad_(True)
    kf = pre[:, d:d + kv].float().reshape(B, S, Hkv, hd).requires_grad_(True)
    gf = gain.clone().requires_grad_(True)
    q_ref, k_ref = R.qk_norm_rope_gain(qf, kf, cos, sin, rope, gf, eps)
    close(post[:, :d], q_ref.detach().reshape(T, d), 0.01, "q")
    close(post[:, d:d + kv], k_ref.detach().reshape(T, kv), 0.01, "k")
    d_post = bf(T, qkvw, scale=0.5, seed=2)
    (q_ref * d_post[:, :d].float().reshape(B, S, H, hd)).sum().backward(retain_graph=True)
    (k_ref * d_post[:, d:d + kv].float().reshape(B, S, Hkv, hd)).sum().backward()
    d_pre = torch.zeros(T, qkvw, device="cuda", dtype=BF)
    d_gain = torch.zeros(H, device="cuda")
    C().qk_norm_rope_bwd(d_post, pre, d_pre, cos, sin, gain, d_gain, H, Hkv, hd, rope, S, eps)
    torch.cuda.synchronize()
    assert rel(d_pre[:, :d], qf.grad.reshape(T, d)) < 0.012
    assert rel(d_pre[:, d:d + kv], kf.grad.reshape(T, kv)) < 0.012
    assert rel(d_gain, gf.grad) < 0.01
    assert float(d_pre[:, d + kv:].abs().max()) == 0.0                  # the value columns belong to the attention backward


@pytest.mark.parametrize("T,H,Hkv", [(1037, 8, 4), (300, 2, 1), (129, 4, 4)])
def test_xsa_forward_and_backward(T, H, Hkv):
    from parameter_golf_b200.ops import reference as R
    hd = 64
    y = bf(T, H * hd, seed=1)
    qkv = bf(T, (H + 2 * Hkv) * hd, seed=2)
    v = qkv[:, (H + Hkv) * hd:]                     # strided view, as in the engine
    z = torch.empty_like(y)
    C().xsa_fwd(y, v, z, Hkv, H // Hkv, hd, 1e-8)
    yf = y.float().reshape(1, T, H, hd).requires_grad_(True)
    vf = v.float().reshape(1, T, Hkv, hd).requires_grad_(True)
    z_ref = R.xsa(yf, vf)
    close(z, z_ref.detach().reshape(T, H * hd), 0.012, "z")
    dz = bf(T, H * hd, scale=0.5, seed=3)
    (z_ref * dz.float().reshape(1, T, H, hd)).sum().backward()
    dy = torch.empty_like(y)
    dqkv = torch.zeros_like(qkv)
    dv = dqkv[:, (H + Hkv) * hd:]
    C().xsa_bwd(dz, y, v, dy, dv, False, Hkv, H // Hkv, hd, 1e-8)
    torch.cuda.synchronize()
    assert rel(dy, yf.grad.reshape(T, H * hd)) < 0.012
    assert rel(dv, vf.grad.reshape(T, Hkv * hd)) < 0.015


@pytest.mark.parametrize("B,S,H,Hkv", [(3, 128, 8, 4), (2, 384, 2, 1)])
def test_xsa_backward_also_yields_the_attention_backward_term(B, S, H, Hkv):
    """With `dsum` the kernel writes -rowsum(dy * y) per (batch, head, position) next to dy and dv, from the values it holds."""
    hd, T = 64, B * S
    y = bf(T, H * hd, seed=4)
    qkv = bf(T, (H + 2 * Hkv) * hd, seed=5)
    v = qkv[:, (H + Hkv) * hd:]
    dz = bf(T, H * hd, scale=0.5, seed=6)
    dy, dy2 = torch.empty_like(y), torch.empty_like(y)
    dv, dv2 = torch.zeros(T, Hkv * hd, device="cuda", dtype=BF), torch.zeros(T, Hkv * hd, device="cuda", dtype=BF)
    dsum = torch.full((B, H, S), float("nan"), device="cuda")
    C().xsa_bwd(dz, y, v, dy, dv, False, Hkv, H // Hkv, hd, 1e-8, dsum, S)
    C().xsa_bwd(dz, y, v, dy2, dv2, False, Hkv, H // Hkv, hd, 1e-8)
    torch.cuda.synchronize()
    assert torch.equal(dy, dy2) and torch.equal(dv, dv2)
    ref = -(dy.float() * y.float()).reshape(B, S, H, hd).sum(-1).permute(0, 2, 1)
    assert (dsum - ref).abs().max() < 1e-3 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("B,S,d,boundary", [(3, 128, 512, -1), (2, 257, 512, 7), (1, 640, 128, -1)])
def test_norm_smear_forward_and_backward(B, S, d, boundary):
    from parameter_golf_b200.ops import reference as R
    T = B * S
    xe = bf(T, d, seed=1)
    gate = torch.randn(d, device="cuda")
    ids = torch.randint(0, 16, (T,), device="cuda", dtype=torch.int32)
    out = torch.empty_like(xe)
    C().norm_smear_fwd(xe, gate, ids if boundary >= 0 else None, out, S, boundary, 1e-6)
    xf = xe.float().reshape(B, S, d).requires_grad_(True)
    gf = gate.clone().requires_grad_(True)
    ref = R.smear_gate(R.rms_norm(xf), gf, ids.reshape(B, S).long() if boundary >= 0 else None, boundary if boundary >= 0 else None)
    close(out, ref.detach().reshape(T, d), 0.012, "out")
    g_out = bf(T, d, scale=0.5, seed=2)
    (ref * g_out.float().reshape(B, S, d)).sum().backward()
    d_xe = torch.empty_like(xe)
    d_gate = torch.zeros(d, device="cuda")
    C().norm_smear_bwd(g_out, xe, gate, ids if boundary >= 0 else None, d_xe, d_gate, S, boundary, 1e-6)
    torch.cuda.synchronize()
    assert rel(d_xe, xf.grad.reshape(T, d)) < 0.012
    assert rel(d_gate, gf.grad) < 0.012


@pytest.mark.parametrize("rows,V", [(1037, 1024), (4099, 1024), (515, 256)])
def test_softcap_cross_entropy_loss_and_gradient(rows, V):
    from parameter_golf_b200.ops import reference as R
    cap, gscale = 30.0, 1.0 / rows
    logits = bf(rows, V, scale=6.0, seed=1)
    tgt = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
    zf = logits.float().requires_grad_(True)
    per = R.softcap_cross_entropy(zf, tgt.long(), cap, reduction="none")
    (per.sum() * gscale).backward()
    nll = torch.empty(rows, device="cuda")
    loss_sum = torch.zeros(1, device="cuda")
    dl = torch.empty_like(logits)
    C().softcap_ce(logits, tgt, nll, dl, loss_sum, cap, gscale)
    torch.cuda.synchronize()
    assert (nll - per.detach()).abs().max().item() < 2e-3
    assert abs(loss_sum.item() - per.sum().item()) < 2e-4 * rows
    assert rel(dl, zf.grad) < 0.01


@pytest.mark.parametrize("B,S", [(3, 128), (1, 1000)])
def test_embedding_gather_and_scatter_with_bigram_hash(B, S):
    from parameter_golf_b200.ops import reference as R
    V, d, buckets, bd = 1024, 512, 3072, 128
    T = B * S
    ids = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
    table, btable = bf(V, d, seed=1), bf(buckets, bd, seed=2)
    out, bout = torch.empty(T, d, device="cuda", dtype=BF), torch.empty(T, bd, device="cuda", dtype=BF)
    C().embed_gather(ids, table, out, 0, S)
    C().embed_gather(ids, btable, bout, buckets, S)
    hashed = R.bigram_hash(ids.reshape(B, S).long(), buckets).reshape(T)
    assert torch.equal(out, table[ids.long()]) and torch.equal(bout, btable[hashed])
    g, bg = bf(T, d, seed=3), bf(T, bd, seed=4)
    dt, dbt = torch.zeros(V, d, device="cuda"), torch.zeros(buckets, bd, device="cuda")
    C().embed_scatter_add(ids, g, dt, 0, S)
    C().embed_scatter_add(ids, bg, dbt, buckets, S)
    torch.cuda.synchronize()
    ref = torch.zeros(V, d, device="cuda").index_add_(0, ids.long(), g.float())
    bref = torch.zeros(buckets, bd, device="cuda").index_add_(0, hashed, bg.float())
    assert rel(dt, ref) < 1e-5 and rel(dbt, bref) < 1e-5
