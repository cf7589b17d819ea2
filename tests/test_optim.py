import math

import pytest
import torch

from parameter_golf_b200.optim import muon as M

torch.manual_seed(0)


@pytest.mark.parametrize("profile", ["simple", "quintic", "polar_express"])
@pytest.mark.parametrize("shape", [(24, 24), (16, 40), (40, 16)])
def test_newton_schulz_orthogonalises(profile, shape):
    g = torch.randn(*shape)
    steps = 8 if profile == "polar_express" else 5
    x = M.newton_schulz(g, steps, profile)
    assert x.shape == g.shape
    gram = x @ x.t() if shape[0] <= shape[1] else x.t() @ x
    assert (gram - torch.eye(gram.shape[0])).abs().max() < 0.5          # the reference's (loose) orthogonality bound
    norms = (x if shape[0] <= shape[1] else x.t()).norm(dim=1)
    assert norms.max() / norms.min() < 2.0
    # same singular subspace as the polar factor
    u, _, vh = torch.linalg.svd(g, full_matrices=False)
    assert torch.nn.functional.cosine_similarity((u @ vh).flatten(), x.flatten(), dim=0) > 0.9


def test_newton_schulz_batched_matches_single():
    g = torch.randn(3, 12, 20)
    xb = M.newton_schulz(g, 5, "quintic")
    for i in range(3):
        assert torch.allclose(xb[i], M.newton_schulz(g[i], 5, "quintic"), atol=1e-5)


def test_ns_coeff_tables():
    assert M.ns_coeff("simple", 3) == (3.4445, -4.7750, 2.0315)
    assert M.ns_coeff("quintic", 5) == M.ns_coeff("quintic", 0)
    assert M.ns_coeff("polar_express", 20) == M.NS_COEFFS["polar_express"][-1]


def test_muon_update_rule():
    p = torch.randn(2, 8, 4)
    g = torch.randn(2, 8, 4)
    p0 = p.clone()
    opt = M.Muon([p], lr=0.1, momentum=0.9, weight_decay=0.05, ns_profile="simple")
    opt.step([g])
    buf = g.clone()
    u = M.newton_schulz(g + 0.9 * buf, 5, "simple")
    exp = p0 * (1 - 0.1 * 0.05) - 0.1 * math.sqrt(2.0) * u
    assert torch.allclose(p, exp, atol=1e-6)
    assert torch.allclose(opt.bufs[0], buf)
    assert M.muon_scale((512, 1536)) == 1.0 and abs(M.muon_scale((1536, 512)) - math.sqrt(3)) < 1e-12


def test_adamw_converges_on_quadratic_and_decays():
    x = torch.tensor([5.0, -3.0])
    opt = M.AdamW([{"params": [x], "lr": 0.1}], betas=(0.9, 0.95), weight_decay=0.0)
    for _ in range(300):
        opt.step([[2 * x]])
    assert x.abs().max() < 1e-2
    y = torch.tensor([1.0])
    M.AdamW([{"params": [y], "lr": 0.1}], weight_decay=0.5).step([[torch.zeros(1)]])
    assert torch.allclose(y, torch.tensor([0.95]))


def test_adamw_first_step_is_sign_like():
    x = torch.tensor([1.0, 1.0])
    M.AdamW([{"params": [x], "lr": 0.01}]).step([[torch.tensor([3.0, -0.2])]])
    assert torch.allclose(x, torch.tensor([0.99, 1.01]), atol=1e-6)


def test_ema_first_call_copies_then_blends():
    e = M.Ema(0.9)
    p = {"w": torch.tensor([1.0])}
    e.update(p)
    assert e.shadow["w"].item() == 1.0
    p["w"] = torch.tensor([2.0])
    e.update(p)
    assert abs(e.shadow["w"].item() - 1.1) < 1e-6
    q = {"w": torch.zeros(1)}
    e.apply_to(q)
    assert abs(q["w"].item() - 1.1) < 1e-6


def test_swa_window_and_average():
    s = M.Swa(every=50, threshold=0.2)
    assert s.should_collect(100, 0.1) and not s.should_collect(100, 0.5) and not s.should_collect(101, 0.1)
    s.collect({"w": torch.tensor([1.0])})
    s.collect({"w": torch.tensor([3.0])})
    assert s.average()["w"].item() == 2.0


def test_lawa_keeps_the_last_k_snapshots():
    l = M.Lawa(k=3, freq=10)
    assert l.should_collect(20) and not l.should_collect(25)
    for v in (1.0, 2.0, 6.0, 7.0):
        l.collect({"w": torch.tensor([v])})
    assert l.count == 3 and l.average()["w"].item() == 5.0          # the first snapshot fell out of the window


def test_wsd_schedule():
    assert M.lr_scale(0, 20, 9000, 3500) == 0.0 and M.lr_scale(10, 20, 9000, 3500) == 0.5
    assert M.lr_scale(20, 20, 9000, 3500) == 1.0 and M.lr_scale(5499, 20, 9000, 3500) == 1.0
    assert abs(M.lr_scale(7250, 20, 9000, 3500) - 0.5) < 1e-9 and M.lr_scale(9000, 20, 9000, 3500) == 0.0
    assert M.lr_scale_with_floor(8999, 20, 9000, 3500, 0.1) == 0.1 and M.lr_scale_with_floor(5, 20, 9000, 3500, 0.1) == 0.25
    assert M.wsd_lr(9000, 1.0, 20, 9000, 3500) == 0.0


def test_wallclock_warmdown():
    # 100 ms/step, cap 600 s, 3500 warm-down steps => warm-down window is 350 s
    assert M.wallclock_lr_scale(1000, 100_000.0, 20000, 3500, 600_000.0) == 1.0
    assert abs(M.wallclock_lr_scale(4250, 425_000.0, 20000, 3500, 600_000.0) - 175_000 / 350_000) < 1e-9
    assert M.wallclock_lr_scale(10, 5.0, 20000, 0, 600_000.0) == 1.0
    assert abs(M.wallclock_lr_scale(90, 0.0, 100, 20, None) - 0.5) < 1e-9


def test_momentum_warmup_and_clip():
    assert M.muon_momentum_at(0, 0.92, 0.99, 1500) == 0.92 and abs(M.muon_momentum_at(750, 0.92, 0.99, 1500) - 0.955) < 1e-9
    assert M.muon_momentum_at(5000, 0.92, 0.99, 1500) == 0.99
    g = [torch.full((4,), 3.0), torch.full((9,), 4.0)]
    n = M.clip_grads_(g, 1.0)
    assert abs(n - math.sqrt(36 + 144)) < 1e-5
    assert abs(math.sqrt(sum(float(x.pow(2).sum()) for x in g)) - 1.0) < 1e-4


def test_fraction_warmdown_by_time_and_by_steps():
    """The last fifth of the budget: of the wall clock when there is a cap (whatever the step count), else of the steps
    (train_gpt_cuda_ternary.py lr_mul)."""
    f = M.fraction_lr_scale
    assert f(10, 100_000.0, 20000, 0.2, 600_000.0) == 1.0
    assert f(10, 480_000.0, 20000, 0.2, 600_000.0) == 1.0
    assert abs(f(10, 540_000.0, 20000, 0.2, 600_000.0) - 0.5) < 1e-12
    assert f(10, 700_000.0, 20000, 0.2, 600_000.0) == 0.0
    assert f(79, 0.0, 100, 0.2, None) == 1.0 and abs(f(90, 0.0, 100, 0.2, None) - 0.5) < 1e-12 and f(100, 0.0, 100, 0.2, None) == 0.0
    assert f(5, 0.0, 100, 0.0, 600_000.0) == 1.0
    # the bug it fixes: a 1200-step window on a run the cap ends after 900 steps decays from the very first step
    assert M.wallclock_lr_scale(1, 650.0, 20000, 1200, 600_000.0) < 1.0 and f(1, 650.0, 20000, 0.2, 600_000.0) == 1.0
