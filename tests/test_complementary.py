"""Complementary training on CPU: bigram table, weighting curves, weighted loss, trainer wiring.
Mirrors the unit tests of ``parameter-golf-rs/crates/pg-kernels/src/complementary.rs:256-431``."""
import numpy as np
import pytest
import torch

from parameter_golf_b200.ops import complementary as comp


def toy_stats():
    st = comp.BigramStats(4)
    st.add_sequence([0, 1, 0, 1, 0, 1, 0, 2, 3, 3, 3])
    return st


def test_counts_row_sums_and_smoothed_probability():
    st = toy_stats()
    assert st.count(0, 1) == 3 and st.count(0, 2) == 1 and st.count(3, 3) == 2 and st.count(2, 0) == 0
    assert st.row_sums.tolist() == [4, 3, 1, 2]
    assert st.prob(0, 1) == pytest.approx((3 + 1) / (4 + 4))
    assert st.prob(2, 1) == pytest.approx(1 / (1 + 4))
    empty = comp.BigramStats(4)
    assert empty.prob(1, 2) == pytest.approx(0.25)            # unseen row: uniform prior
    np.testing.assert_allclose(st.prob_table().sum(axis=1), 1.0, rtol=1e-6)
    assert st.prob_table()[0, 1] == pytest.approx(st.prob(0, 1))
    assert empty.row_entropy(0) == pytest.approx(np.log(4.0))
    assert st.row_entropy(0) < np.log(4.0)


def test_merge_equals_counting_the_concatenation_minus_the_seam():
    a, b = comp.BigramStats(5), comp.BigramStats(5)
    rng = np.random.default_rng(0)
    x, y = rng.integers(0, 5, 100), rng.integers(0, 5, 77)
    a.add_sequence(x)
    b.add_sequence(y)
    a.merge(b)
    whole = comp.BigramStats(5)
    whole.add_sequence(x)
    whole.add_sequence(y)
    assert np.array_equal(a.counts, whole.counts) and np.array_equal(a.row_sums, whole.row_sums)
    with pytest.raises(ValueError):
        a.merge(comp.BigramStats(4))
    with pytest.raises(ValueError):
        a.add_sequence([0, 7])


def test_byte_layout_round_trip_and_corruption():
    st = toy_stats()
    raw = st.to_bytes()
    assert len(raw) == 4 + 8 * 4 + 4 * 16
    assert raw[:4] == (4).to_bytes(4, "little")
    assert int.from_bytes(raw[4:12], "little") == 4                      # row_sums[0]
    assert int.from_bytes(raw[4 + 32 + 4:4 + 32 + 8], "little") == 3     # counts[0, 1]
    back = comp.BigramStats.from_bytes(raw)
    assert np.array_equal(back.counts, st.counts) and np.array_equal(back.row_sums, st.row_sums)
    with pytest.raises(ValueError):
        comp.BigramStats.from_bytes(raw[:-1])
    bad = bytearray(raw)
    bad[4] ^= 1
    with pytest.raises(ValueError):
        comp.BigramStats.from_bytes(bytes(bad))


def test_weight_shapes():
    p = np.array([0.0, 0.1, 0.2, 0.6, 1.0], dtype=np.float32)
    np.testing.assert_allclose(comp.apply_shape(p, 0.5, comp.WeightShape("linear")), [1.0, 0.95, 0.9, 0.7, 0.5], rtol=1e-6)
    np.testing.assert_allclose(comp.apply_shape(p, 2.0, comp.WeightShape("linear")), [1.0, 0.8, 0.6, 0.0, 0.0], atol=1e-6)
    np.testing.assert_allclose(comp.apply_shape(p, 0.5, comp.WeightShape("power", power=2.0)), 1 - 0.5 * p * p, rtol=1e-6)
    fl = comp.apply_shape(p, 1.0, comp.WeightShape())           # floor 0.2, min_w 0.25
    np.testing.assert_allclose(fl, [1.0, 1.0, 1.0, 0.5, 0.25], rtol=1e-6)
    with pytest.raises(ValueError):
        comp.WeightShape("cubic")


def test_weights_table_and_direct_agree_and_alpha_zero_is_identity():
    st = toy_stats()
    prev, curr = np.array([0, 0, 3, 2]), np.array([1, 2, 3, 0])
    w = comp.complementary_weights(prev, curr, st, 0.8)
    tab = comp.weight_table(st, 0.8)
    np.testing.assert_allclose(w, tab[prev, curr], rtol=1e-6)
    np.testing.assert_allclose(comp.complementary_weights(prev, curr, st, 0.8, table=tab), w, rtol=1e-6)
    assert w[0] < 1.0 and w[3] == 1.0                           # P(1|0)=0.5 is down-weighted, P(0|2)=0.2 is not
    assert np.all(comp.complementary_weights(prev, curr, st, 0.0) == 1.0)
    assert np.all(comp.weight_table(st, 0.0) == 1.0)


def test_weighted_mean_and_gradient_scaling():
    assert comp.weighted_mean_loss([1.0, 3.0], [1.0, 1.0]) == pytest.approx(2.0)
    assert comp.weighted_mean_loss([1.0, 3.0], [1.0, 0.0]) == pytest.approx(1.0)
    assert comp.weighted_mean_loss([1.0, 3.0], [0.0, 0.0]) == 0.0
    g = np.ones((3, 4), dtype=np.float32)
    comp.scale_grad_logits_by_weight(g, [1.0, 0.5, 0.0], 4)
    np.testing.assert_allclose(g.sum(axis=1), [4.0, 2.0, 0.0])


def test_oracle_weighted_loss_matches_manual_and_its_gradient_is_the_scaled_one():
    from parameter_golf_b200.models import gpt
    from parameter_golf_b200.spec import family_preset
    s = family_preset("tiny_cpu")
    m = s.model
    p = gpt.init_params(m, 3)
    torch.manual_seed(1)
    ids = torch.randint(0, m.vocab_size, (2, 16))
    tgt = torch.randint(0, m.vocab_size, (2, 16))
    tw = torch.rand(2, 16) + 0.1
    per = gpt.gpt_forward(m, p, ids, tgt, reduction="none")
    loss = gpt.gpt_forward(m, p, ids, tgt, token_weights=tw)
    assert float(loss) == pytest.approx(comp.weighted_mean_loss(per.numpy(), tw.numpy()), rel=1e-5)
    ones = gpt.gpt_forward(m, p, ids, tgt, token_weights=torch.ones(2, 16))
    assert float(ones) == pytest.approx(float(gpt.gpt_forward(m, p, ids, tgt)), rel=1e-6)


def test_trainer_runs_with_complementary_weights(tmp_path):
    from parameter_golf_b200.spec import family_preset
    from parameter_golf_b200.train import VariantRunner
    s = family_preset("tiny_cpu")
    s.mode = "smoke"
    s.train.complementary_alpha = 0.7
    s.train.complementary_stats_tokens = 1 << 16
    s.train.complementary_stats_path = str(tmp_path / "bigram.bin")
    s.train.artifact_path = str(tmp_path / "a.pgrs")
    s.validate()
    res = VariantRunner(s).run()
    assert res.steps > 0 and np.isfinite(res.train_loss_last)
    assert 0.25 <= res.complementary_mean_weight <= 1.0
    st = comp.BigramStats.from_bytes(open(tmp_path / "bigram.bin", "rb").read())
    assert st.vocab_size == s.model.vocab_size and int(st.row_sums.sum()) > 0
    # second run loads the saved table
    res2 = VariantRunner(s).run()
    assert res2.complementary_mean_weight == pytest.approx(res.complementary_mean_weight)
