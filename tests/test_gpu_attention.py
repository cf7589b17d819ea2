"""tcgen05 flash attention against the explicit fp32 attention of the oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, B, S, H, Hkv, hd):
    from parameter_golf_b200.ops.reference import causal_gqa_attention
    return causal_gqa_attention(q.float().reshape(B, S, H, hd), k.float().reshape(B, S, Hkv, hd), v.float().reshape(B, S, Hkv, hd)).reshape(B * S, H * hd)


def _ref_lse(q, k, B, S, H, Hkv, hd):
    qf = q.float().reshape(B, S, H, hd).permute(0, 2, 1, 3)
    kf = k.float().reshape(B, S, Hkv, hd).permute(0, 2, 1, 3).repeat_interleave(H // Hkv, 1)
    s = qf @ kf.transpose(-1, -2) / hd ** 0.5
    s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool, device=q.device).tril(), float("-inf"))
    return torch.logsumexp(s, -1)


@pytest.mark.parametrize("B,S,H,Hkv", [(1, 128, 2, 1), (2, 256, 4, 2), (1, 640, 8, 4), (3, 384, 2, 2), (1, 1024, 4, 1)])
def test_attention_forward(B, S, H, Hkv):
    from parameter_golf_b200.ops import native as n
    hd = 64
    torch.manual_seed(S + H)
    qkv = (torch.randn(B * S, (H + 2 * Hkv) * hd, device="cuda") * 1.5).bfloat16()       # strided views of one packed buffer
    q, k, v = qkv[:, :H * hd], qkv[:, H * hd:(H + Hkv) * hd], qkv[:, (H + Hkv) * hd:]
    y = torch.zeros(B * S, H * hd, device="cuda", dtype=torch.bfloat16)
    lse = n.attn_fwd(q, k, v, y, B, S, H, Hkv, hd)
    torch.cuda.synchronize()
    n.check_status()
    ref = _ref(q, k, v, B, S, H, Hkv, hd)
    assert (y.float() - ref).abs().max() < 0.04, (y.float() - ref).abs().max()      # one bf16 ulp of an output in [4, 8) is 0.031
    lse_nat = -lse * 0.6931471805599453               # the kernel stores -(log2-domain lse), the form its backward consumes
    assert (lse_nat - _ref_lse(q, k, B, S, H, Hkv, hd)).abs().max().item() < 0.02


@pytest.mark.parametrize("B,S,H,Hkv", [(2, 256, 4, 2), (1, 640, 8, 4), (3, 128, 2, 2)])
def test_attention_forward_with_exclusive_self_attention_output(B, S, H, Hkv):
    """The optional second output: y with its component along the token's own value vector removed, from the same kernel."""
    from parameter_golf_b200.ops import native as n
    from parameter_golf_b200.ops import reference as R
    hd = 64
    torch.manual_seed(S + 7 * H)
    qkv = (torch.randn(B * S, (H + 2 * Hkv) * hd, device="cuda") * 1.5).bfloat16()
    q, k, v = qkv[:, :H * hd], qkv[:, H * hd:(H + Hkv) * hd], qkv[:, (H + Hkv) * hd:]
    y = torch.zeros(B * S, H * hd, device="cuda", dtype=torch.bfloat16)
    z = torch.zeros_like(y)
    n.attn_fwd(q, k, v, y, B, S, H, Hkv, hd, z=z, xsa_eps=1e-8)
    torch.cuda.synchronize()
    n.check_status()
    ref = _ref(q, k, v, B, S, H, Hkv, hd)
    assert (y.float() - ref).abs().max() < 0.04
    z_ref = R.xsa(ref.reshape(B, S, H, hd), v.float().reshape(B, S, Hkv, hd)).reshape(B * S, H * hd)
    assert (z.float() - z_ref).abs().max() < 0.04, (z.float() - z_ref).abs().max()
    # z is orthogonal to the value vector of its KV group
    zz = z.float().reshape(B * S, Hkv, H // Hkv, hd)
    vv = torch.nn.functional.normalize(v.float().reshape(B * S, Hkv, 1, hd), dim=-1)
    assert (zz * vv).sum(-1).abs().max() < 0.12


def test_attention_forward_large_scores_trigger_rescale():
    """Scores that keep growing along the sequence force the lazy rescale of the accumulator."""
    from parameter_golf_b200.ops import native as n
    B, S, H, Hkv, hd = 1, 512, 2, 1, 64
    torch.manual_seed(0)
    q = torch.randn(B * S, H * hd, device="cuda")
    k = torch.randn(B * S, Hkv * hd, device="cuda") * torch.linspace(0.5, 12.0, S, device="cuda")[:, None]
    v = torch.randn(B * S, Hkv * hd, device="cuda")
    q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    y = torch.empty(B * S, H * hd, device="cuda", dtype=torch.bfloat16)
    n.attn_fwd(q, k, v, y, B, S, H, Hkv, hd)
    torch.cuda.synchronize()
    n.check_status()
    assert (y.float() - _ref(q, k, v, B, S, H, Hkv, hd)).abs().max() < 0.05


@pytest.mark.parametrize("reproducible", [False, True])
@pytest.mark.parametrize("B,S,H,Hkv", [(1, 128, 2, 1), (2, 256, 4, 2), (1, 640, 8, 4), (2, 384, 2, 2), (1, 512, 4, 1), (3, 896, 4, 2)])
def test_attention_backward(B, S, H, Hkv, reproducible):
    from parameter_golf_b200.ops import native as n
    from parameter_golf_b200.ops.reference import causal_gqa_attention
    hd = 64
    torch.manual_seed(S * 3 + H)
    qkv = (torch.randn(B * S, (H + 2 * Hkv) * hd, device="cuda") * 1.2).bfloat16()
    q, k, v = qkv[:, :H * hd], qkv[:, H * hd:(H + Hkv) * hd], qkv[:, (H + Hkv) * hd:]
    dy = (torch.randn(B * S, H * hd, device="cuda") * 0.5).bfloat16()
    y = torch.empty(B * S, H * hd, device="cuda", dtype=torch.bfloat16)
    lse = n.attn_fwd(q, k, v, y, B, S, H, Hkv, hd)
    dqkv = torch.zeros_like(qkv)
    dq, dk, dv = dqkv[:, :H * hd], dqkv[:, H * hd:(H + Hkv) * hd], dqkv[:, (H + Hkv) * hd:]
    base = (torch.randn(B * S, Hkv * hd, device="cuda") * 0.1).bfloat16()
    dv.copy_(base)
    n.attn_bwd(q, k, v, y, dy, lse, dq, dk, dv, B, S, H, Hkv, hd, accumulate_dv=True, reproducible=reproducible)
    torch.cuda.synchronize()
    n.check_status()
    qf = q.float().reshape(B, S, H, hd).requires_grad_(True)
    kf = k.float().reshape(B, S, Hkv, hd).requires_grad_(True)
    vf = v.float().reshape(B, S, Hkv, hd).requires_grad_(True)
    out = causal_gqa_attention(qf, kf, vf)
    gq, gk, gv = torch.autograd.grad(out, (qf, kf, vf), dy.float().reshape(B, S, H, hd))
    for name, got, ref in (("dq", dq, gq.reshape(B * S, -1)), ("dk", dk, gk.reshape(B * S, -1)), ("dv", dv.float() - base.float(), gv.reshape(B * S, -1))):
        err = (got.float() - ref).abs().max().item()
        scale = ref.abs().max().item()
        assert err < 0.03 * scale + 0.02, (name, err, scale)


def test_attention_backward_single_pass_many_tiles_and_clean_scratch():
    """More CTA-level items than SMs (several items per persistent CTA, both K/V buffers and every Q/dO stage reused),
    checked against the two-kernel form; the shared accumulator must be left zero, and a second call must agree."""
    from parameter_golf_b200.ops import native as n
    B, S, H, Hkv, hd = 10, 1024, 8, 4, 64
    torch.manual_seed(7)
    qkv = torch.randn(B * S, (H + 2 * Hkv) * hd, device="cuda").bfloat16()
    q, k, v = qkv[:, :H * hd], qkv[:, H * hd:(H + Hkv) * hd], qkv[:, (H + Hkv) * hd:]
    dy = (torch.randn(B * S, H * hd, device="cuda") * 0.5).bfloat16()
    y = torch.empty(B * S, H * hd, device="cuda", dtype=torch.bfloat16)
    lse = n.attn_fwd(q, k, v, y, B, S, H, Hkv, hd)
    ref = [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)]
    n.attn_bwd(q, k, v, y, dy, lse, *ref, B, S, H, Hkv, hd, reproducible=True)
    acc = n.attn_dq_scratch(q.device, B, S, H, hd)
    for _ in range(2):
        got = [torch.full_like(q, 7.0), torch.full_like(k, 7.0), torch.full_like(v, 7.0)]
        n.attn_bwd(q, k, v, y, dy, lse, *got, B, S, H, Hkv, hd)
        torch.cuda.synchronize()
        n.check_status()
        assert float(acc.abs().max()) == 0.0
        for g, r in zip(got, ref):
            err = (g.float() - r.float()).abs().max().item()
            assert err <= 0.01 * r.float().abs().max().item() + 1e-3, err
