import os

import numpy as np
import pytest

from parameter_golf_b200.data import shards as S
from parameter_golf_b200.data.bpb import BpbLuts, compute_bpb


def _mk(tmp_path, n_files=2, n=1000, vocab=64):
    for i in range(n_files):
        S.write_shard(str(tmp_path / f"t_train_{i:06d}.bin"), (np.arange(n) + 1000 * i) % vocab)
    return str(tmp_path / "t_train_*.bin")


def test_shard_roundtrip_and_header(tmp_path):
    p = str(tmp_path / "a.bin")
    toks = np.arange(777, dtype=np.uint16)
    S.write_shard(p, toks)
    assert (tmp_path / "a.bin").stat().st_size == 1024 + 2 * 777
    hdr = np.fromfile(p, dtype="<i4", count=3)
    assert list(hdr) == [20240520, 1, 777]
    assert np.array_equal(np.asarray(S.open_shard(p)), toks)


def test_shard_rejects_bad_files(tmp_path):
    p = tmp_path / "a.bin"
    S.write_shard(str(p), np.arange(10))
    raw = bytearray(p.read_bytes())
    (tmp_path / "short.bin").write_bytes(raw[:-2])
    with pytest.raises(S.ShardError):
        S.open_shard(str(tmp_path / "short.bin"))
    raw[0] ^= 0xFF
    (tmp_path / "magic.bin").write_bytes(raw)
    with pytest.raises(S.ShardError):
        S.open_shard(str(tmp_path / "magic.bin"))
    with pytest.raises(FileNotFoundError):
        S.TokenStream(str(tmp_path / "none_*.bin"))


def test_stream_wraps_and_skips(tmp_path):
    pat = _mk(tmp_path, 2, 100, 1 << 16)
    st = S.TokenStream(pat)
    a = st.take(150)
    assert a[99] == 99 and a[100] == 1000
    st.skip(50)
    assert st.take(3).tolist() == [0, 1, 2]      # wrapped to the first shard


@pytest.mark.parametrize("world,accum", [(1, 1), (2, 1), (4, 2), (8, 1)])
def test_loader_spans_are_the_reference_slicing(tmp_path, world, accum):
    pat = _mk(tmp_path, 3, 5000, 1 << 16)
    global_tokens, seq = 64 * world * accum, 16
    ref = S.TokenStream(pat)
    loaders = [S.DistributedTokenLoader(pat, r, world) for r in range(world)]
    for _ in range(5):
        L = global_tokens // (world * accum)
        chunk = ref.take((L + 1) * world)
        for r, ld in enumerate(loaders):
            x, y = ld.next_batch(global_tokens, seq, accum)
            span = chunk[r * (L + 1):(r + 1) * (L + 1)].astype(np.int64)
            assert np.array_equal(x.reshape(-1), span[:-1]) and np.array_equal(y.reshape(-1), span[1:])
            assert x.shape == (L // seq, seq)


def test_loader_state_restore(tmp_path):
    pat = _mk(tmp_path, 2, 3000, 1 << 16)
    a = S.DistributedTokenLoader(pat, 1, 2)
    a.next_batch(256, 16)
    st = a.state()
    x1, _ = a.next_batch(256, 16)
    b = S.DistributedTokenLoader(pat, 1, 2)
    b.restore(st)
    x2, _ = b.next_batch(256, 16)
    assert np.array_equal(x1, x2)


def test_markov_generator_is_seeded_and_zipfian():
    a = S.generate_markov_tokens(50000, 1024, seed=3)
    assert np.array_equal(a, S.generate_markov_tokens(50000, 1024, seed=3))
    assert not np.array_equal(a, S.generate_markov_tokens(50000, 1024, seed=4))
    assert a.dtype == np.uint16 and a.max() < 1024
    # order-1 structure: the conditional entropy is far below the marginal entropy
    pair = np.bincount(a[:-1].astype(np.int64) * 1024 + a[1:], minlength=1024 * 1024).reshape(1024, 1024).astype(np.float64)
    rowp = pair / np.clip(pair.sum(1, keepdims=True), 1, None)
    h_cond = -(pair / pair.sum() * np.log(np.clip(rowp, 1e-12, None))).sum()
    marg = np.bincount(a, minlength=1024) / a.size
    h_marg = -(marg * np.log(np.clip(marg, 1e-12, None))).sum()
    assert h_cond < 0.8 * h_marg


def test_validation_loader_truncates(tmp_path):
    S.write_shard(str(tmp_path / "v_val_000000.bin"), np.arange(1000) % 50)
    v = S.load_validation_tokens(str(tmp_path / "v_val_*.bin"), 64)
    assert v.shape[0] == 15 * 64 + 1
    assert S.load_validation_tokens(str(tmp_path / "v_val_*.bin"), 64, max_tokens=200).shape[0] == 3 * 64 + 1


def test_bpb_formula_and_luts():
    luts = BpbLuts.from_pieces(["<s>", "▁the", "cat", "<0x41>", "▁"], 5, control={0})
    assert luts.base_bytes.tolist() == [0, 3, 3, 1, 0]
    prev, tgt = np.array([0, 1, 2]), np.array([1, 2, 1])
    # "▁the" after a boundary token: no space byte; after "cat": +1
    assert luts.token_bytes(prev, tgt).tolist() == [3, 3, 4]
    loss, bpb = compute_bpb(loss_sum_nats=np.log(2.0) * 10, token_count=10, byte_count=40)
    assert abs(loss - np.log(2.0)) < 1e-12 and abs(bpb - 0.25) < 1e-12
    s = BpbLuts.seeded(1024)
    assert s.base_bytes.min() >= 1 and s.base_bytes.max() <= 6 and np.array_equal(s.base_bytes, BpbLuts.seeded(1024).base_bytes)
    assert BpbLuts.placeholder(8).base_bytes.tolist() == [4] * 8


# ---- native (C++) loader --------------------------------------------------------------------------------------------

def _native_or_skip():
    from parameter_golf_b200.ops import native
    try:
        native.load_raw()
    except Exception as e:          # no compiler / no torch headers on this machine
        pytest.skip(f"extension unavailable: {e}")
    from parameter_golf_b200.data.native_loader import NativeTokenLoader
    return NativeTokenLoader


def _write_three_shards(tmp_path):
    import numpy as np
    from parameter_golf_b200.data.shards import write_shard
    rng = np.random.default_rng(3)
    sizes = [1000, 0, 777]
    for i, n in enumerate(sizes):
        write_shard(str(tmp_path / f"tok_train_{i:06d}.bin"), rng.integers(0, 1024, size=n, dtype=np.uint16))
    return str(tmp_path / "tok_train_*.bin")


@pytest.mark.parametrize("world", [1, 2, 3])
def test_native_loader_matches_python_loader(tmp_path, world):
    import numpy as np
    from parameter_golf_b200.data.shards import DistributedTokenLoader
    Native = _native_or_skip()
    pattern = _write_three_shards(tmp_path)
    for rank in range(world):
        a, b = DistributedTokenLoader(pattern, rank, world), Native(pattern, rank, world)
        for step in range(9):                        # crosses shard ends, the empty shard and the wrap-around
            x = a.next_span_u16(384, 2)
            y = b.next_span_u16(384, 2)
            assert np.array_equal(x, y), (rank, step)
        assert a.stream.state() == b.state()


def test_native_loader_prefetch_and_restore(tmp_path):
    import numpy as np
    from parameter_golf_b200.data.shards import DistributedTokenLoader
    Native = _native_or_skip()
    pattern = _write_three_shards(tmp_path)
    ref = DistributedTokenLoader(pattern, 1, 2)
    nat = Native(pattern, 1, 2)
    nat.start_prefetch(256, 2)
    got = []
    for _ in range(6):
        got.append(nat.next_prefetched().numpy().view(np.uint16).copy())
    want = [ref.next_span_u16(256, 2).copy() for _ in range(6)]
    for x, y in zip(want, got):
        assert np.array_equal(x, y)
    st = nat.state()
    assert st == ref.stream.state()                  # spans the worker fetched ahead do not count
    more_ref = [ref.next_span_u16(256, 2).copy() for _ in range(3)]
    nat.restore(st)                                   # restarts the worker from the consumed position
    more = [nat.next_prefetched().numpy().view(np.uint16).copy() for _ in range(3)]
    for x, y in zip(more_ref, more):
        assert np.array_equal(x, y)
    nat.stop_prefetch()
    z = nat.next_span_u16(256, 2)                     # synchronous path resumes where the consumer stopped
    assert np.array_equal(z, ref.next_span_u16(256, 2))


def test_native_loader_rejects_bad_shards(tmp_path):
    import numpy as np
    Native = _native_or_skip()
    p = tmp_path / "bad_train_000000.bin"
    hdr = np.zeros(256, dtype="<i4")
    hdr[0], hdr[1], hdr[2] = 20240520, 1, 10
    p.write_bytes(hdr.tobytes() + b"\x00" * 18)       # one token short
    with pytest.raises(RuntimeError, match="does not match"):
        Native(str(tmp_path / "bad_train_*.bin"))


def test_byte_sidecar_is_filtered_from_tokens_and_drives_the_byte_count(tmp_path):
    """Sidecar shards share the directory and the format of the token shards; they must not be read as tokens, and when
    attached to the byte tables the byte count of a scored token is the sidecar entry at its position."""
    import torch
    from parameter_golf_b200.data.bpb import BpbLuts
    from parameter_golf_b200.data.shards import (is_byte_sidecar_path, load_validation_byte_sidecar, load_validation_tokens,
                                                 write_shard)
    from parameter_golf_b200.eval.sliding import eval_contiguous, eval_sliding
    rng = np.random.default_rng(0)
    toks = rng.integers(0, 64, 16 * 8 + 1).astype(np.uint16)
    side = rng.integers(1, 9, toks.shape[0]).astype(np.uint16)
    write_shard(str(tmp_path / "fineweb_val_000000.bin"), toks)
    write_shard(str(tmp_path / "fineweb_val_bytes_000000.bin"), side)
    assert is_byte_sidecar_path("x/fineweb_val_bytes_000000.bin") and is_byte_sidecar_path("val_bytes.bin")
    assert not is_byte_sidecar_path("x/fineweb_val_000000.bin")
    got = load_validation_tokens(str(tmp_path / "fineweb_val_*.bin"), 16)
    assert np.array_equal(got, toks)                                   # the sidecar matched the glob and was left out
    sc = load_validation_byte_sidecar(str(tmp_path / "fineweb_val_bytes_*.bin"))
    assert sc.dtype == np.float32 and np.array_equal(sc, side.astype(np.float32))
    luts = BpbLuts.seeded(64).with_sidecar(sc)
    nll = lambda x, y: torch.ones(x.shape, dtype=torch.float32)
    loss, bpb = eval_contiguous(nll, got, 16, luts)
    want = (1.0 / np.log(2.0)) * (128 / side[1:129].sum())
    assert loss == pytest.approx(1.0) and bpb == pytest.approx(want, rel=1e-6)
    from parameter_golf_b200.eval.sliding import scored_range, window_starts
    nbytes = ntok = 0.0                                                # the tail windows re-score their last tokens, as in the reference
    for ws in window_starts(128, 16, 4):
        s0, wlen = scored_range(ws, 128, 16, 4)
        nbytes += side[ws + 1 + s0: ws + 1 + wlen].sum()
        ntok += wlen - s0
    loss2, bpb2 = eval_sliding(nll, got, 16, 4, luts)
    assert bpb2 == pytest.approx((1.0 / np.log(2.0)) * (ntok / nbytes), rel=1e-6)
    with pytest.raises(ValueError):
        luts.token_bytes(np.array([1]), np.array([2]))


def test_synthetic_validation_shard_follows_the_training_chain(tmp_path):
    """Training and validation shards are different draws from ONE Markov chain: the most likely successor of a token is the
    same in both (a model fitted to the training shard must be scorable on the validation shard)."""
    root = str(tmp_path / "d")
    S.write_synthetic_dataset(root, vocab=64, train_tokens=1 << 18, val_tokens=1 << 17, train_shards=2, seed=5)

    def top_successor(path):
        t = S.open_shard(path).astype(np.int64)
        counts = np.zeros((64, 64), dtype=np.int64)
        np.add.at(counts, (t[:-1], t[1:]), 1)
        return counts.argmax(1)

    a = top_successor(os.path.join(root, "fineweb_train_000000.bin"))
    b = top_successor(os.path.join(root, "fineweb_train_000001.bin"))
    v = top_successor(os.path.join(root, "fineweb_val_000000.bin"))
    assert (a == v).mean() > 0.9 and (a == b).mean() > 0.9
    assert not np.array_equal(S.open_shard(os.path.join(root, "fineweb_train_000000.bin"))[:1000], S.open_shard(os.path.join(root, "fineweb_val_000000.bin"))[:1000])


# ---- local text -> tokenizer -> shards (data/text_shards.py) -----------------------------------------------------------------

def _corpus(n=400, seed=3):
    rng = np.random.default_rng(seed)
    words = ["alpha", "beta", "gamma", "delta", "tensor", "memory", "kernel", "golf", "parameter", "stream", "42", "2048", "the", "of", "and"]
    return [" ".join(rng.choice(words, size=int(rng.integers(5, 40)))) + "." for _ in range(n)]


def test_sentencepiece_training_and_shard_export_round_trip(tmp_path):
    """A BPE tokenizer trained on local documents with the reference's settings, exported to shards: documents start with
    BOS, the first documents form the validation split, the text comes back from the ids, and the byte sidecar adds up to
    the UTF-8 size of the validation text."""
    import json
    from parameter_golf_b200.data import text_shards as T
    from parameter_golf_b200.data.bpb import BpbLuts
    docs = _corpus()
    jl = tmp_path / "docs.jsonl"
    jl.write_text("\n".join(json.dumps({"text": d}) for d in docs) + "\n")
    assert list(T.iter_documents(str(jl))) == docs
    model = T.train_sentencepiece(T.iter_documents(str(jl)), 320, str(tmp_path / "tok" / "sp320"))
    tok = T.load_sentencepiece(model)
    assert tok.vocab_size <= 320 and tok.bos_id == 1 and tok.eos_id == 2
    stats = T.export_shards(T.iter_documents(str(jl)), tok, str(tmp_path / "out"), num_val_docs=50, shard_tokens=4000)
    assert stats["docs_val"] == 50 and stats["docs_train"] == 350 and stats["files_train"] >= 2
    val = S.load_validation_tokens(str(tmp_path / "out" / "fineweb_val_*.bin"), 16)           # sidecars matched by the pattern are left out
    side = S.load_validation_byte_sidecar(str(tmp_path / "out" / "fineweb_val_bytes_*.bin"))
    allval = np.concatenate([np.asarray(S.open_shard(f)) for f in sorted((tmp_path / "out").glob("fineweb_val_0*.bin"))])
    assert len(side) == len(allval) == stats["tokens_val"] and np.array_equal(val, allval[:len(val)])
    starts = np.flatnonzero(allval == tok.bos_id)
    assert len(starts) == 50 and starts[0] == 0
    first = allval[starts[0] + 1:starts[1]]
    assert tok.decode(first) == docs[0]
    assert int(side.sum()) == stats["bytes_val"] == sum(len(d.encode()) for d in docs[:50])
    # the table rule gives the same byte counts as the sidecar
    luts = BpbLuts.from_sentencepiece(model, tok.vocab_size)
    assert np.array_equal(luts.token_bytes(allval[:-1], allval[1:]), side[1:])
    train = np.concatenate([np.asarray(S.open_shard(f)) for f in sorted((tmp_path / "out").glob("fineweb_train_*.bin"))])
    assert len(train) == stats["tokens_train"] and int((train == tok.bos_id).sum()) == 350 and int(train.max()) < tok.vocab_size
    assert json.load(open(tmp_path / "out" / "manifest.json"))["vocab_size"] == tok.vocab_size


def test_byte_tokenizer_export_and_the_vocabulary_guard(tmp_path):
    from parameter_golf_b200.data import text_shards as T
    txt = tmp_path / "notes.txt"
    txt.write_text("first block\nstill first\n\nsecond block with an accent: café\n\n\nthird\n")
    docs = list(T.iter_documents(str(tmp_path)))
    assert docs == ["first block\nstill first", "second block with an accent: café", "third"]
    tok = T.ByteTokenizer().as_tokenizer()
    stats = T.export_shards(docs, tok, str(tmp_path / "b"), num_val_docs=2, shard_tokens=1000, append_eos=True)
    val = np.asarray(S.open_shard(str(tmp_path / "b" / "fineweb_val_000000.bin")))
    side = np.asarray(S.open_shard(str(tmp_path / "b" / "fineweb_val_bytes_000000.bin")))
    assert val[0] == 1 and int((val == 2).sum()) == 2 and stats["bytes_val"] == int(side.sum()) == sum(len(d.encode()) for d in docs[:2])
    assert T.ByteTokenizer().decode(val[1:1 + len(docs[0].encode())]) == docs[0]
    bad = T.Tokenizer("bad", 10, 1, 2, lambda texts: [np.array([3, 11]) for _ in texts], lambda ids: "", tok.luts)
    with pytest.raises(ValueError, match="outside declared vocab_size"):
        T.export_shards(["x"], bad, str(tmp_path / "c"))
    assert T._main(["--docs", str(txt), "--out", str(tmp_path / "cli"), "--tokenizer", "bytes", "--val-docs", "1", "--shard-tokens", "64"]) == 0
    assert (tmp_path / "cli" / "fineweb_train_000000.bin").exists()


def test_export_from_a_tokenizer_config_uses_the_reference_layout(tmp_path):
    """A tokenizer config in the format of the reference's data/tokenizer_specs.json: one dataset per entry under
    datasets/fineweb10B_<suffix>/, tokenizer models under tokenizers/, a manifest listing both."""
    import json
    from parameter_golf_b200.data import text_shards as T
    jl = tmp_path / "docs.jsonl"
    jl.write_text("\n".join(json.dumps({"text": d}) for d in _corpus(200)) + "\n")
    cfg = tmp_path / "specs.json"
    cfg.write_text(json.dumps({"tokenizers": [{"name": "sp_bpe_320", "dataset_suffix": "sp320", "vocab_size": 320},
                                              {"name": "pure_byte_260", "dataset_suffix": "byte260", "kind": "byte"}]}))
    assert T._main(["--docs", str(jl), "--out", str(tmp_path / "root"), "--tokenizer-config", str(cfg), "--val-docs", "20", "--shard-tokens", "5000"]) == 0
    root = tmp_path / "root"
    man = json.load(open(root / "manifest.json"))
    assert [d["name"] for d in man["datasets"]] == ["fineweb10B_sp320", "fineweb10B_byte260"]
    assert [t["kind"] for t in man["tokenizers"]] == ["sentencepiece_bpe", "byte"] and man["tokenizers"][0]["model_path"] == "tokenizers/fineweb_320_bpe.model"
    assert (root / "tokenizers" / "fineweb_320_bpe.model").exists() and (root / "tokenizer_config.export.json").exists()
    for d in man["datasets"]:
        assert d["stats"]["docs_val"] == 20 and d["stats"]["docs_train"] == 180
        toks = S.load_validation_tokens(str(root / d["val_glob"]), 8)
        assert int(toks.max()) < d["vocab_size"] and toks[0] == d["bos_id"]
        assert len(list((root / d["path"]).glob("fineweb_train_*.bin"))) >= 1
    assert T.tokenizer_kind({"vocab_size": 1024}) == "sentencepiece_bpe" and T.tokenizer_kind({"dataset_suffix": "byte260"}) == "byte"
    with pytest.raises(ValueError):
        T.tokenizer_kind({"name": "x"})


def test_fetch_from_a_local_mirror_follows_the_manifest(tmp_path):
    """export (tokenizer config) -> mirror -> fetch: the validation split with its sidecars, the first N training shards and the
    tokenizer files land under the destination; a second call writes nothing; asking for more shards than exist is refused."""
    import json
    from parameter_golf_b200.data import fetch_cached as F
    from parameter_golf_b200.data import text_shards as T
    jl = tmp_path / "docs.jsonl"
    jl.write_text("\n".join(json.dumps({"text": d}) for d in _corpus(300)) + "\n")
    cfg = tmp_path / "specs.json"
    cfg.write_text(json.dumps({"tokenizers": [{"name": "sp_bpe_320", "dataset_suffix": "sp320", "vocab_size": 320}]}))
    mirror = tmp_path / "mirror"
    T.export_from_config(str(jl), str(mirror), str(cfg), val_docs=20, shard_tokens=1500)
    have = json.load(open(mirror / "manifest.json"))["datasets"][0]["stats"]["files_train"]
    assert have >= 3
    dest = tmp_path / "data"
    assert F.main(["--source", str(mirror), "--dest", str(dest), "--variant", "sp320", "--train-shards", "2"]) == 0
    got = sorted(p.name for p in (dest / "datasets" / "fineweb10B_sp320").iterdir())
    assert [g for g in got if "train" in g] == ["fineweb_train_000000.bin", "fineweb_train_000001.bin"]
    assert any(g.startswith("fineweb_val_bytes_") for g in got) and any(g.startswith("fineweb_val_0") for g in got)
    assert (dest / "tokenizers" / "fineweb_320_bpe.model").exists() and (dest / "manifest.json").exists()
    out = F.fetch_variant(F.local_getter(str(mirror)), str(dest), "sp320", 3)
    assert out["written"] == ["datasets/fineweb10B_sp320/fineweb_train_000002.bin"]           # only what was missing
    assert F.fetch_variant(F.local_getter(str(mirror)), str(dest), "sp320", 3)["written"] == []
    toks = S.load_validation_tokens(str(dest / "datasets" / "fineweb10B_sp320" / "fineweb_val_*.bin"), 8)
    assert toks[0] == 1 and int(toks.max()) < 320
    with pytest.raises(ValueError, match="training shards"):
        F.fetch_variant(F.local_getter(str(mirror)), str(dest), "sp320", have + 1)
    with pytest.raises(ValueError):
        F.dataset_dir_for_variant("gpt2")
    with pytest.raises(ValueError, match="not in the manifest"):
        F.fetch_variant(F.local_getter(str(mirror)), str(dest), "sp1024", 1)
