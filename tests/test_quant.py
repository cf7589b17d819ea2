import json
import struct

import numpy as np
import pytest
import torch

from parameter_golf_b200.models import gpt
from parameter_golf_b200.quant import container as C
from parameter_golf_b200.quant import quantize as Q
from parameter_golf_b200.quant.export import build_artifact, check_budget, export_model, load_artifact
from parameter_golf_b200.quant.gptq import gptq_quantize
from parameter_golf_b200.spec import family_preset

torch.manual_seed(0)


def small_spec(**ov):
    s = family_preset("tiny_cpu")
    m = s.model
    m.vocab_size, m.num_layers, m.model_dim, m.num_heads, m.num_kv_heads = 64, 2, 32, 4, 2
    m.bigram.enabled, m.bigram.vocab_size, m.bigram.dim = True, 16, 8
    m.smear_gate = True
    s.apply_overrides([f"{k}={v}" for k, v in ov.items()])
    return s.validate()


def test_pgrs_roundtrip_and_layout():
    recs = [C.TensorRecord("a.weight", (2, 3), "i8", b"\x01\x02\x03"), C.TensorRecord("b", (2,), "f16", np.array([1, 2], "<f2").tobytes())]
    blob = C.write_pgrs(recs, '{"k":1}')
    assert blob[:4] == b"PGRS" and struct.unpack_from("<II", blob, 4) == (1, 2)
    # first record: name_len, name, ndim, dims, dtype code, data_len
    assert struct.unpack_from("<I", blob, 12)[0] == 8 and blob[16:24] == b"a.weight"
    assert struct.unpack_from("<III", blob, 24) == (2, 2, 3) and blob[36] == 3
    out, md = C.read_pgrs(blob)
    assert md == '{"k":1}' and [(r.name, r.dims, r.dtype, r.data) for r in out] == [(r.name, r.dims, r.dtype, r.data) for r in recs]


def test_pgrs_crc_detects_corruption():
    blob = bytearray(C.write_pgrs([C.TensorRecord("w", (4,), "i8", b"abcd")], "{}"))
    blob[blob.index(b"abcd") + 1] ^= 0x40
    with pytest.raises(C.ArtifactError, match="CRC"):
        C.read_pgrs(bytes(blob))
    with pytest.raises(C.ArtifactError):
        C.read_pgrs(bytes(blob[:20]))


def test_zstd_and_pergroup_roundtrip_and_sniffing():
    raw = C.write_pgrs([C.TensorRecord("w", (1000,), "i8", bytes(1000))], "{}")
    z = C.compress_payload(raw, "zstd22")
    assert z[:4] == b"\x28\xb5\x2f\xfd" and len(z) < len(raw) and C.decompress_payload(z) == raw
    g = C.compress_pergroup(raw, chunk_bytes=300)
    assert g[:4] == b"PGPG" and struct.unpack_from("<IQII", g, 4) == (1, len(raw), 300, 4)
    assert C.decompress_payload(g) == raw and C.decompress_payload(raw) == raw
    x = C.compress_payload(raw, "lzma9")
    assert x[:6] == b"\xfd7zXZ\x00" and len(x) < len(raw) and C.decompress_payload(x) == raw
    with pytest.raises(C.ArtifactError):
        C.decompress_payload(x[:-8] + b"\x00" * 8)
    with pytest.raises(C.ArtifactError):
        C.compress_payload(raw, "brotli")


@pytest.mark.parametrize("bits", [4, 5, 6, 7, 8])
def test_bitpack_lsb_first(bits):
    qmin, qmax = Q.qrange(bits)
    q = np.random.default_rng(bits).integers(qmin, qmax + 1, size=37)
    data = C.pack_bits(q, bits)
    assert len(data) == (37 * bits + 7) // 8
    assert np.array_equal(C.unpack_bits(data, 37, bits), q)
    one = C.pack_bits(np.array([qmin + 1, qmin]), bits)       # encoded values 1, 0 => only bit 0 set
    assert one[0] == 1


def test_quantizer_rule():
    assert Q.qrange(6) == (-32, 31) and Q.qrange(5) == (-16, 15)
    assert Q.round_half_away(torch.tensor([0.5, -0.5, 1.5, 2.5, -2.5])).tolist() == [1, -1, 2, 3, -3]
    w = torch.randn(8, 4096)
    w[0, 0] = 5.0                                             # an outlier makes a clipped percentile win
    q, s = Q.quantize_rows(w, 6)
    assert q.dtype == torch.int8 and q.min() >= -32 and q.max() <= 31
    srt = w[0].abs().sort().values
    assert any(abs(float(s[0]) - float(srt[min(int(4096 * p), 4095)] / 31)) < 1e-7 for p in Q.CLIP_PERCENTILES)
    assert float(s[0]) < 5.0 / 31
    for r in range(8):                                         # the chosen clip has the smallest error of the five
        errs = []
        for p in Q.CLIP_PERCENTILES:
            sc = max(float(w[r].abs().sort().values[min(int(4096 * p), 4095)]), 1e-8) / 31
            qq = Q.round_half_away(w[r] / sc).clamp(-32, 31)
            errs.append(float((w[r] - qq * sc).pow(2).sum()))
        got = float((w[r] - q[r].float() * s[r]).pow(2).sum())
        assert got <= min(errs) * (1 + 1e-5)


@pytest.mark.parametrize("scheme,compression", [("gptq_lite_int6", "zstd22"), ("mixed_int5_int6", "pergroup"), ("aggressive", "none"),
                                                ("tight_int7_int4", "zstd22")])
def test_export_load_roundtrip(scheme, compression, tmp_path):
    s = small_spec(**{"quant.scheme": scheme, "quant.compression": compression})
    p = gpt.fill_deterministic(s.model)
    blob = export_model(s, p, str(tmp_path / "a.pgrs"))
    assert (tmp_path / "a.pgrs").read_bytes() == blob
    back = load_artifact(blob, s)
    assert set(back) == set(p)
    bits = Q.scheme_bits(scheme)
    for k in p:
        tol = 0.6 * float(p[k].abs().max()) / (2 ** (min(bits.values()) - 1) - 1) if k in gpt.BANKS or k == "tok_emb" else 2e-3 * max(1.0, float(p[k].abs().max()))
        assert (back[k] - p[k]).abs().max() <= tol + 1e-6, k
    recs, md = C.read_pgrs(C.decompress_payload(blob))
    names = [r.name for r in recs]
    assert names[:4] == ["qo_bank.q.weight", "qo_bank.q.scale", "qo_bank.o.weight", "qo_bank.o.scale"]
    assert names[14:17] == ["bigram_embed", "bigram_proj", "bigram_scale"] and "blocks.1.q_gain" in names
    meta = json.loads(md)
    assert meta["format"] == "pgrs_quant" and meta["groups"] == bits and '"qo_bank.q":' in md and " " not in md
    w = next(r for r in recs if r.name == "mlp_up_bank.weight")
    assert w.dtype == "i8" and w.dims == (2 * 64, 32) and len(w.data) == (2 * 64 * 32 * bits["mlp_up_bank"] + 7) // 8


def test_load_rejects_mismatched_shape_and_corruption():
    s = small_spec()
    blob = export_model(s, gpt.fill_deterministic(s.model))
    other = small_spec(**{"model.num_layers": 3})
    with pytest.raises(C.ArtifactError, match="num_layers"):
        load_artifact(blob, other)
    raw = bytearray(C.decompress_payload(blob))
    raw[200] ^= 1
    with pytest.raises(C.ArtifactError):
        load_artifact(bytes(raw), s)


def test_lqer_reduces_error():
    s0, s1 = small_spec(**{"quant.matrix_bits": 4}), small_spec(**{"quant.matrix_bits": 4, "quant.lqer.enabled": "true", "quant.lqer.rank": 8})
    p = gpt.init_params(s0.model, seed=1)
    p["mlp_down_bank"].normal_()
    e0 = (load_artifact(export_model(s0, p), s0)["mlp_down_bank"] - p["mlp_down_bank"]).pow(2).mean()
    e1 = (load_artifact(export_model(s1, p), s1)["mlp_down_bank"] - p["mlp_down_bank"]).pow(2).mean()
    assert e1 < 0.9 * e0


def test_legacy_unsplit_names_load():
    s = small_spec()
    p = gpt.fill_deterministic(s.model)
    recs, md = C.read_pgrs(build_artifact(s, p))
    by = {r.name: r for r in recs}
    meta = json.loads(md)
    meta["groups"]["qo_bank"] = 6
    meta["groups"]["kv_bank"] = 6
    merged = []
    for bank, (a, b) in (("qo_bank", ("qo_bank.q", "qo_bank.o")), ("kv_bank", ("kv_bank.k", "kv_bank.v"))):
        qa = C.unpack_bits(by[f"{a}.weight"].data, int(np.prod(by[f"{a}.weight"].dims)), 6)
        qb = C.unpack_bits(by[f"{b}.weight"].data, int(np.prod(by[f"{b}.weight"].dims)), 6)
        rows = by[f"{a}.weight"].dims[0] + by[f"{b}.weight"].dims[0]
        merged.append(C.TensorRecord(f"{bank}.weight", (rows, by[f"{a}.weight"].dims[1]), "i8", C.pack_bits(np.concatenate([qa, qb]), 6)))
        merged.append(C.TensorRecord(f"{bank}.scale", (rows,), "f16", by[f"{a}.scale"].data + by[f"{b}.scale"].data))
    rest = [r for r in recs if not r.name.startswith(("qo_bank.", "kv_bank."))]
    back = load_artifact(C.write_pgrs(merged + rest, json.dumps(meta, separators=(",", ":"))), s)
    ref = load_artifact(build_artifact(s, p), s)
    assert torch.equal(back["qo_bank"], ref["qo_bank"]) and torch.equal(back["kv_bank"], ref["kv_bank"])


def test_prune_masks_and_ordering():
    w = torch.randn(6, 16)
    assert (Q.prune_topk_per_row(w, 0.25).sum(1) == 4).all()
    assert Q.prune_global_magnitude(w, 0.5).sum() == 48
    m24 = Q.prune_2_of_4(w).reshape(6, 4, 4)
    assert (m24.sum(-1) == 2).all()
    ab = Q.ordering_ab_test(w, 0.5, 6)
    assert set(ab) == {"prune_then_quantize_mse", "quantize_then_prune_mse"} and all(v > 0 for v in ab.values())


def test_budget_is_strict():
    assert check_budget(15_000_000, 999_999) and not check_budget(15_000_000, 1_000_000)


def test_gptq_beats_round_to_nearest_on_hessian_error():
    rows, cols = 24, 48
    W = torch.randn(rows, cols)
    X = torch.randn(400, cols) @ (torch.eye(cols) + 0.6 * torch.randn(cols, cols))      # correlated inputs
    H = X.t() @ X / 400
    q, s = gptq_quantize(W, H, bits=4, block=16)
    assert q.min() >= -8 and q.max() <= 7
    q0, s0 = Q.quantize_rows(W, 4)

    def out_err(qq, ss):
        return float(((W - qq.float() * ss.half().float()[:, None]) @ X.t()).pow(2).mean())
    assert out_err(q, s) < 0.85 * out_err(q0, s0)


def test_selective_prune_hits_target():
    q = {"a": torch.randint(-3, 4, (64, 64), dtype=torch.int8)}
    sc = {"a": torch.rand(64) + 0.1}
    size = lambda d: len(C.zstd_compress(C.pack_bits(d["a"].numpy(), 6), 3))
    full = size(q)
    out, n = Q.selective_prune_to_target(q, sc, size, int(full * 0.93))
    assert size(out) <= int(full * 0.93) and n > 0
    changed = out["a"] != q["a"]
    assert (q["a"][changed].abs() == 1).all() and (out["a"][changed] == 0).all()


def test_native_artifact_primitives_match_numpy_forms():
    """C++ bit packing, CRC-32 and PGRS container against the NumPy/zlib specification, both directions."""
    import zlib
    import numpy as np
    from parameter_golf_b200.quant import container as C
    if C._native() is None:
        pytest.skip("native extension not built")
    rng = np.random.default_rng(0)
    for bits in (4, 5, 6, 8):
        lo, hi = -(1 << (bits - 1)), (1 << (bits - 1)) - 1
        q = rng.integers(lo, hi + 1, size=1001).astype(np.int8)
        packed = C.pack_bits(q, bits, native=True)
        assert packed == C.pack_bits(q, bits, native=False)
        assert (C.unpack_bits(packed, q.size, bits, native=True) == q).all()
        assert (C.unpack_bits(packed, q.size, bits, native=False) == q).all()
    with pytest.raises(C.ArtifactError):
        C.pack_bits(np.array([40], dtype=np.int8), 6)                     # outside [-32, 31]
    blob = rng.integers(0, 256, size=100003).astype(np.uint8).tobytes()
    assert C._native().crc32(blob) == zlib.crc32(blob) & 0xFFFFFFFF
    recs = [C.TensorRecord("a.q", (3, 7), "i8", bytes(range(16))), C.TensorRecord("b", (2,), "f16", b"\x00\x3c\x00\x40")]
    raw = C.write_pgrs(recs, '{"k": 1}', native=True)
    assert raw == C.write_pgrs(recs, '{"k": 1}', native=False)
    for nat in (True, False):
        got, meta = C.read_pgrs(raw, native=nat)
        assert meta == '{"k": 1}' and [(r.name, tuple(r.dims), r.dtype, r.data) for r in got] == [(r.name, r.dims, r.dtype, r.data) for r in recs]
        bad = bytearray(raw)
        bad[40] ^= 0xFF
        with pytest.raises(C.ArtifactError):
            C.read_pgrs(bytes(bad), native=nat)


def test_int8_zlib_baseline_export_round_trip():
    """Per-row int8 with the 99.99984 % clip, small tensors kept in fp16 / control tensors in fp32, zlib-9 container."""
    import zlib
    from parameter_golf_b200.quant import int8_baseline as I8
    g = torch.Generator().manual_seed(0)
    state = {"w": torch.randn(300, 400, generator=g), "bank": torch.randn(3, 160, 200, generator=g) * 0.1,
             "small": torch.randn(8, 16, generator=g), "q_gain": torch.randn(8, generator=g), "ids": torch.arange(5)}
    q, s = I8.quantize_float_tensor(state["w"])
    ref_clip = torch.quantile(state["w"].abs(), I8.CLIP_Q, dim=1)
    ref_scale = (ref_clip / 127.0).clamp_min(1.0 / 127.0)
    assert torch.allclose(s.float(), ref_scale.to(torch.float16).float())
    ref_q = torch.clamp(torch.round(torch.maximum(torch.minimum(state["w"], ref_clip[:, None]), -ref_clip[:, None]) / ref_scale[:, None]), -127, 127)
    assert torch.equal(q, ref_q.to(torch.int8))
    obj, stats = I8.quantize_state_dict_int8(state)
    assert set(obj["quantized"]) == {"w", "bank"} and set(obj["passthrough"]) == {"small", "q_gain", "ids"}
    assert obj["passthrough"]["small"].dtype == torch.float16 and obj["passthrough"]["q_gain"].dtype == torch.float32
    assert obj["scales"]["bank"].shape == (3, 160) and obj["qmeta"]["w"]["scheme"] == "per_row"
    assert stats["param_count"] == sum(t.numel() for t in state.values())
    blob, st = I8.export_int8_zlib(state)
    assert blob[:1] == b"\x78" and zlib.decompress(blob)[:4] == I8.MAGIC and st["compressed_bytes"] == len(blob) < st["raw_bytes"]
    back = I8.load_int8_zlib(blob)
    assert torch.equal(back["ids"], state["ids"]) and torch.equal(back["q_gain"], state["q_gain"])
    assert back["small"].dtype == torch.float32 and torch.allclose(back["small"], state["small"], atol=2e-3)
    for k in ("w", "bank"):
        err = (back[k] - state[k]).abs().max() / state[k].abs().max()
        assert back[k].dtype == torch.float32 and float(err) < 0.02, (k, float(err))
    with pytest.raises(ValueError):
        I8.deserialize(b"nope" + b"\x00" * 16)


def test_int8_zlib_scheme_through_export_and_load():
    from parameter_golf_b200.models import gpt
    from parameter_golf_b200.quant.export import export_model, load_artifact
    from parameter_golf_b200.spec import family_preset
    s = family_preset("tiny_cpu")
    s.quant.scheme = "int8_zlib"
    s.validate()
    p = gpt.init_params(s.model, 1)
    blob = export_model(s, p)
    back = load_artifact(blob, s)
    assert set(back) == set(p)
    for k in p:
        assert back[k].shape == p[k].shape
        # the scale floor of 1/127 (reference rule) bounds the error of small-valued matrices by half a step
        assert float((back[k] - p[k]).abs().max()) <= 0.02 * float(p[k].abs().max()) + 0.5 / 127 + 1e-3, k


def test_ternary_quantiser_base3_packing_and_scale_fix():
    from parameter_golf_b200.quant import ternary as T3
    g = torch.Generator().manual_seed(0)
    w = torch.randn(64, 300, generator=g) * 0.05                    # 300 columns: the last group of 128 is ragged
    q, s = T3.quantize_ternary(w)
    assert q.dtype == torch.int8 and set(q.unique().tolist()) <= {-1, 0, 1} and s.shape == (64, 3)
    q0, s0 = T3.quantize_ternary(w, fix_scale=False)
    assert torch.equal(q, q0)                                        # the fix changes the scale, not the codes
    e_fix = (w - T3.dequantize_ternary(q, s)).pow(2).mean()
    e_raw = (w - T3.dequantize_ternary(q0, s0)).pow(2).mean()
    assert float(e_fix) < float(e_raw)                               # least-squares scale for the chosen codes
    # group 0 of row 0, by hand
    blk = w[0, :128]
    s_h = blk.abs().mean()
    q_h = torch.clamp(torch.round(blk / s_h), -1, 1)
    assert torch.equal(q[0, :128].float(), q_h) and float(s0[0, 0]) == pytest.approx(float(s_h), rel=1e-6)
    assert float(s[0, 0]) == pytest.approx(float(blk.abs()[q_h != 0].mean()), rel=1e-6)
    # packing: five trits per byte, exact round trip, bytes < 243
    codes = np.array([-1, 0, 1, 1, -1, 0, 1], dtype=np.int8)
    raw = T3.pack_trits(codes)
    assert len(raw) == 2 and raw[0] == 0 + 3 * 1 + 9 * 2 + 27 * 2 + 81 * 0
    assert np.array_equal(T3.unpack_trits(raw, 7), codes)
    with pytest.raises(ValueError):
        T3.pack_trits(np.array([2], dtype=np.int8))
    with pytest.raises(ValueError):
        T3.unpack_trits(bytes([250]), 5)
    blob = T3.compress(q, s)
    back = T3.decompress(blob)
    assert back.shape == w.shape and torch.allclose(back, T3.dequantize_ternary(q, s.half().float()), atol=1e-6)
    assert 1.0 < T3.bits_per_param(q, s) < 2.2                       # ~1.6 bits of entropy per weight plus scales
    with pytest.raises(ValueError):
        T3.deserialize(T3.serialize(q, s)[:-1])


def test_byte_per_code_storage_round_trips_and_prune_to_target_meets_the_budget():
    """`quant.code_storage = "bytes"` keeps one int8 per code (the container of the Python records, which lets the entropy
    coder see the code distribution); it must load to the same weights as the bit-packed form. With a byte target below the
    artifact's size the exporter zeroes the cheapest +-1 codes until the compressed artifact fits beside the code."""
    import torch
    from parameter_golf_b200.models import gpt
    from parameter_golf_b200.quant import export as E
    from parameter_golf_b200.spec import family_preset
    spec = family_preset("tiny_cpu")
    spec.quant.scheme = "gptq_lite_int6"
    spec.validate()
    torch.manual_seed(0)
    params = {k: (torch.randn_like(v) * 0.05 if v.ndim >= 2 else v.clone()) for k, v in gpt.init_params(spec.model, 0).items()}
    packed = E.load_artifact(E.export_model(spec, params), spec)
    spec.quant.code_storage = "bytes"
    blob = E.export_model(spec, params)
    loaded = E.load_artifact(blob, spec)
    for k in packed:
        assert torch.equal(packed[k], loaded[k]), k
    code = E.code_bytes()
    spec.quant.target_artifact_bytes = code + int(len(blob) * 0.992)
    small = E.export_model(spec, params)
    assert len(small) <= spec.quant.target_artifact_bytes - code < len(blob)
    assert E.export_model.last_pruned > 0
    pruned = E.load_artifact(small, spec)
    changed = sum(int((pruned[k] != loaded[k]).sum()) for k in ("qo_bank", "kv_bank", "mlp_up_bank", "mlp_down_bank"))
    assert 0 < changed and torch.equal(pruned["tok_emb"], loaded["tok_emb"])          # only matrix codes of magnitude one were dropped


def test_fp8_float_storage_round_trips_and_halves_the_float_tables():
    """quant.float_storage = fp8: the 2-D float tensors that are not coded (bigram and value-embedding tables, projections)
    are stored as e4m3 bytes and come back as the e4m3-rounded values; 1-D control tensors stay f16."""
    from parameter_golf_b200.quant import container as Cn
    from parameter_golf_b200.quant.export import build_artifact
    s = family_preset("tiny_cpu")
    s.model.bigram.enabled, s.model.bigram.vocab_size, s.model.bigram.dim = True, 64, 32
    s.model.value_embedding.enabled, s.model.value_embedding.dim, s.model.value_embedding.layers = True, 32, [1]
    s.validate()
    p = gpt.fill_deterministic(s.model)
    a16 = build_artifact(s, p)
    s.quant.float_storage = "fp8"
    s.validate()
    a8 = build_artifact(s, p)
    recs = {r.name: r for r in Cn.read_pgrs(a8)[0]}
    assert recs["bigram_embed"].dtype == "f8e4m3" and len(recs["bigram_embed"].data) == 64 * 32
    assert recs["ve_proj"].dtype == "f8e4m3" and recs["smear_gate"].dtype == "f16" if "smear_gate" in recs else True
    assert len(a8) < len(a16)
    back = load_artifact(a8, s)
    for k in ("bigram_embed", "bigram_proj", "ve_embed", "ve_proj"):
        want = p[k].clamp(-448, 448).to(torch.float8_e4m3fn).float()
        assert torch.equal(back[k], want), k
    # the python reader agrees with the native one on the new dtype code
    assert [(r.name, r.dtype, r.data) for r in Cn.read_pgrs(a8, native=False)[0]] == [(r.name, r.dtype, r.data) for r in Cn.read_pgrs(a8)[0]]


def test_fp8_qat_forward_uses_the_rounded_tables_and_passes_gradients_straight_through():
    from parameter_golf_b200.ops import reference as R
    s = family_preset("tiny_cpu")
    s.model.bigram.enabled, s.model.bigram.vocab_size, s.model.bigram.dim = True, 64, 32
    s.model.fp8_qat = True
    s.quant.float_storage = "fp8"
    s.validate()
    m = s.model
    p = gpt.fill_deterministic(m)
    ids = torch.randint(0, m.vocab_size, (2, 16))
    plain = gpt.gpt_forward(m, p, ids, ids)
    qat = gpt.gpt_forward(m, p, ids, ids, qat=True)
    rounded = dict(p, bigram_embed=p["bigram_embed"].to(torch.float8_e4m3fn).float(), bigram_proj=p["bigram_proj"].to(torch.float8_e4m3fn).float())
    m2 = family_preset("tiny_cpu").model
    m2.bigram.enabled, m2.bigram.vocab_size, m2.bigram.dim = True, 64, 32
    assert float(plain) != float(qat)
    assert torch.allclose(qat, gpt.gpt_forward(m2, rounded, ids, ids, qat=True), atol=1e-6)
    w = p["bigram_proj"].clone().requires_grad_(True)
    (g,) = torch.autograd.grad(R.fake_quant_fp8_ste(w).sum(), w)
    assert torch.equal(g, torch.ones_like(w))


def test_ternary_scheme_exports_what_ternary_qat_trains(tmp_path):
    """quant.scheme = ternary_b158 with model.qat_kind = ternary: the artifact holds base-3 packed codes and per-group fp16
    scales, reloads to exactly the weights the QAT forward used, so the loss after the round trip equals the QAT loss (the
    record's "no round-trip gap"), and costs about 1.6 bits per bank weight before compression."""
    from parameter_golf_b200.ops import reference as R
    from parameter_golf_b200.quant.export import build_artifact
    s = family_preset("tiny_cpu")
    s.apply_overrides(["quant.scheme=ternary_b158", "quant.compression=lzma9", "quant.ternary_group=64", "model.qat_kind=ternary",
                       "model.qat_ternary_group=64", "quant.prune_to_target=false"])
    s.validate()
    m = s.model
    p = gpt.fill_deterministic(m)
    blob = export_model(s, p, str(tmp_path / "t.pgrs"))
    back = load_artifact(blob, s)
    for bank in ("qo_bank", "kv_bank", "mlp_up_bank", "mlp_down_bank"):
        want = R.fake_quant_ternary_ste(p[bank], 64)
        assert torch.allclose(back[bank], want, atol=1e-7), bank
        vals = (back[bank].reshape(-1, 64) / back[bank].reshape(-1, 64).abs().amax(-1, keepdim=True).clamp_min(1e-12)).round().unique()
        assert set(vals.tolist()) <= {-1.0, 0.0, 1.0}
    ids = torch.randint(0, m.vocab_size, (2, 32))
    trained = dict(back, **{b: p[b] for b in ("qo_bank", "kv_bank", "mlp_up_bank", "mlp_down_bank")})      # the fp32 banks QAT trains
    qat_loss = gpt.gpt_forward(m, trained, ids, ids, qat=True)
    assert torch.allclose(gpt.gpt_forward(m, back, ids, ids), qat_loss, atol=1e-5)
    raw = build_artifact(s, p)
    bank_params = sum(p[b].numel() for b in ("qo_bank", "kv_bank", "mlp_up_bank", "mlp_down_bank"))
    emb_bytes = p["tok_emb"].numel() + 2 * p["tok_emb"].shape[0]
    assert (len(raw) - emb_bytes) * 8 / bank_params < 2.0            # 1.6 bits of codes + scales and small tensors
    s.quant.code_storage = "bytes"
    assert torch.equal(load_artifact(export_model(s, p), s)["qo_bank"], back["qo_bank"])
    with pytest.raises(ValueError):
        family_preset("record_11l").apply_overrides(["model.qat_kind=ternary"]).validate()
    t = family_preset("ternary_10l").validate()
    assert t.model.head_dim == 96 and t.quant.scheme == "ternary_b158" and t.train.qat_enabled and t.model.rope.mode == "yarn"


def test_binary_quantiser_bit_packing_and_scale_rule():
    """1-bit codes, absmean scale per group (the least-squares scale for sign codes), eight codes per byte with element i in bit
    i mod 8 (train_gpt_cuda_binary.py:117-127), a ragged last group scaled over the columns that exist."""
    from parameter_golf_b200.quant import binary as B1
    g = torch.Generator().manual_seed(5)
    w = torch.randn(6, 200, generator=g)
    w[0, 0] = 0.0                                        # zero codes as +1
    q, s = B1.quantize_binary(w, 64)
    assert q.shape == w.shape and s.shape == (6, 4) and set(q.unique().tolist()) == {-1, 1} and q[0, 0] == 1
    assert torch.allclose(s[:, 0], w[:, :64].abs().mean(-1)) and torch.allclose(s[:, 3], w[:, 192:].abs().mean(-1))
    base = (w - B1.dequantize_binary(q, s, 64)).pow(2).sum()
    for f in (0.9, 1.1):
        assert (w - B1.dequantize_binary(q, s * f, 64)).pow(2).sum() > base
    raw = B1.pack_signs(q.numpy())
    assert len(raw) == (q.numel() + 7) // 8
    first = q.reshape(-1)[:8].numpy()
    assert raw[0] == sum(int(first[i] > 0) << i for i in range(8))
    assert np.array_equal(B1.unpack_signs(raw, q.numel()), q.reshape(-1).numpy())
    with pytest.raises(ValueError):
        B1.pack_signs(np.array([0, 1], dtype=np.int8))
    with pytest.raises(ValueError):
        B1.unpack_signs(raw[:3], q.numel())


def test_binary_scheme_exports_what_binary_qat_trains(tmp_path):
    """quant.scheme = binary_b1 with model.qat_kind = binary: one bit per bank weight plus fp16 group scales, reloading to exactly
    the weights the QAT forward used."""
    from parameter_golf_b200.ops import reference as R
    from parameter_golf_b200.quant.export import build_artifact
    s = family_preset("tiny_cpu")
    s.apply_overrides(["quant.scheme=binary_b1", "quant.compression=lzma9", "quant.ternary_group=64", "model.qat_kind=binary",
                       "model.qat_ternary_group=64", "quant.prune_to_target=false"])
    s.validate()
    m = s.model
    p = gpt.fill_deterministic(m)
    blob = export_model(s, p, str(tmp_path / "b.pgrs"))
    back = load_artifact(blob, s)
    banks = ("qo_bank", "kv_bank", "mlp_up_bank", "mlp_down_bank")
    for bank in banks:
        assert torch.allclose(back[bank], R.fake_quant_binary_ste(p[bank], 64), atol=1e-7), bank
        grp = back[bank].reshape(-1, 64).abs()
        assert torch.allclose(grp, grp[:, :1].expand_as(grp))                    # one magnitude per group: sign codes
    ids = torch.randint(0, m.vocab_size, (2, 32))
    trained = dict(back, **{b: p[b] for b in banks})
    assert torch.allclose(gpt.gpt_forward(m, back, ids, ids), gpt.gpt_forward(m, trained, ids, ids, qat=True), atol=1e-5)
    w = p["qo_bank"].clone().requires_grad_(True)
    (gw,) = torch.autograd.grad(R.fake_quant_binary_ste(w, 64).sum(), w)
    assert torch.equal(gw, torch.ones_like(w))                                    # straight through
    raw = build_artifact(s, p)
    bank_params = sum(p[b].numel() for b in banks)
    emb_bytes = p["tok_emb"].numel() + 2 * p["tok_emb"].shape[0]
    assert (len(raw) - emb_bytes) * 8 / bank_params < 1.45                        # 1 bit of code + 0.25 of scales + the small tensors
    s.quant.code_storage = "bytes"
    assert torch.equal(load_artifact(export_model(s, p), s)["kv_bank"], back["kv_bank"])
    with pytest.raises(ValueError):
        family_preset("record_11l").apply_overrides(["model.qat_kind=binary"]).validate()
    b = family_preset("binary_15l").validate()
    assert (b.model.num_layers, b.model.head_dim, b.quant.scheme, b.model.block_smear, b.train.max_wallclock_seconds) == (15, 96, "binary_b1", True, 0.0)
    shapes = gpt.param_shapes(b.model)
    assert shapes["skip_weights"] == (7, 768)                                     # 7 blocks before the turn, 8 after


def test_fp16_embedding_and_coarse_middle_layers_in_both_exporters(tmp_path):
    """quant.embed_bits = 16 keeps the tied table as fp16 (records/.../2026-03-18_FP16Embed_WD3600); quant.coarse_layers /
    coarse_step round the codes of the listed blocks to multiples of the step (records/.../2026-03-19_10L_MixedPrecision,
    INT4_LAYERS / INT4_STEP), which shrinks the compressed artifact and costs accuracy only in those blocks."""
    from parameter_golf_b200.quant.int8_baseline import load_int8_zlib
    s = family_preset("tiny_cpu")
    s.apply_overrides(["model.num_layers=4", "quant.prune_to_target=false"])
    m = s.model
    p = gpt.init_params(m, seed=3)
    for k in ("qo_bank", "mlp_down_bank"):                       # the zero-initialised halves would hide the effect
        p[k] = torch.randn(p[k].shape, generator=torch.Generator().manual_seed(4)) * 0.05
    plain = export_model(s, p)
    s.apply_env({"INT4_LAYERS": "1,2", "INT4_STEP": "4"})
    s.quant.embed_bits = 16
    s.validate()
    blob = export_model(s, p)
    back = load_artifact(blob, s)
    assert torch.equal(back["tok_emb"], p["tok_emb"].half().float())
    base = load_artifact(plain, s)
    n = m.num_layers
    for l in range(n):
        changed = not torch.equal(back["mlp_up_bank"][l], base["mlp_up_bank"][l])
        assert changed == (l in (1, 2)), l
        assert (not torch.equal(back["kv_bank"][n + l], base["kv_bank"][n + l])) == (l in (1, 2))
    err = lambda a, l: float((a["mlp_up_bank"][l] - p["mlp_up_bank"][l]).pow(2).mean())
    assert err(back, 1) > err(base, 1) and err(back, 0) == err(base, 0)
    # the baseline trainer's int8 + zlib artifact takes the same two options
    s.quant.scheme = "int8_zlib"
    z = export_model(s, p)
    zs = load_int8_zlib(z)
    assert zs["tok_emb"].dtype == torch.float32 and torch.equal(zs["tok_emb"], p["tok_emb"].half().float())
    s.quant.embed_bits = 8
    zc = export_model(s, p)
    s.quant.coarse_layers = []
    z0 = export_model(s, p)
    assert len(zc) < 0.97 * len(z0) and len(z) > len(zc)        # coarser codes in two of four blocks compress better; the fp16 table costs bytes
    z0s = load_int8_zlib(z0)
    for l in range(n):
        assert (not torch.equal(zs["qo_bank"][l], z0s["qo_bank"][l])) == (l in (1, 2))
        assert (not torch.equal(zs["qo_bank"][n + l], z0s["qo_bank"][n + l])) == (l in (1, 2))
    with pytest.raises(ValueError):
        family_preset("tiny_cpu").apply_overrides(["quant.coarse_layers=[7]"]).validate()
