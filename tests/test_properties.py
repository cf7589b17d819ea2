"""Property tests (hypothesis) of the pure data transformations: bit / trit / sign packing, shard slicing across ranks, sliding
windows and document chunk windows. Each property is a statement that must hold for every input, not a list of examples."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from parameter_golf_b200.quant import container as C

FAST = settings(max_examples=60, deadline=None)


@FAST
@given(bits=st.integers(2, 8), data=st.data())
def test_bit_packing_round_trips_and_has_the_exact_length(bits, data):
    n = data.draw(st.integers(0, 300))
    lo, hi = -(1 << (bits - 1)), (1 << (bits - 1)) - 1
    q = np.array(data.draw(st.lists(st.integers(lo, hi), min_size=n, max_size=n)), dtype=np.int8)
    raw = C.pack_bits(q, bits)
    assert len(raw) == (n * bits + 7) // 8
    assert np.array_equal(C.unpack_bits(raw, n, bits), q.astype(np.int32))


@FAST
@given(st.lists(st.sampled_from([-1, 0, 1]), max_size=200))
def test_trit_packing_round_trips(codes):
    from parameter_golf_b200.quant.ternary import pack_trits, unpack_trits
    q = np.array(codes, dtype=np.int8)
    raw = pack_trits(q)
    assert len(raw) == (len(codes) + 4) // 5 and all(b < 243 for b in raw)
    assert np.array_equal(unpack_trits(raw, len(codes)), q)


@FAST
@given(st.lists(st.sampled_from([-1, 1]), max_size=200))
def test_sign_packing_round_trips(codes):
    from parameter_golf_b200.quant.binary import pack_signs, unpack_signs
    q = np.array(codes, dtype=np.int8)
    raw = pack_signs(q)
    assert len(raw) == (len(codes) + 7) // 8
    assert np.array_equal(unpack_signs(raw, len(codes)), q)


@FAST
@given(slots=st.integers(1, 64), world=st.integers(1, 16))
def test_bank_slots_are_owned_exactly_once(slots, world):
    from parameter_golf_b200.optim.muon import shard_range
    owned = []
    for r in range(world):
        a, b = shard_range(slots, r, world)
        assert 0 <= a <= b <= slots and b - a <= -(-slots // world)
        owned.extend(range(a, b))
    assert owned == list(range(slots))


@FAST
@given(total=st.integers(1, 3000), window=st.integers(2, 256), stride_div=st.integers(1, 8))
def test_sliding_windows_cover_every_token_and_full_windows_score_each_once(total, window, stride_div):
    """The Python records' rule (…2026-03-23…/train_gpt.py:1027-1046): window 0 scores all of its positions, every later one its
    last ``stride``; no token is skipped, and tokens that only full-length windows reach are scored exactly once (the shortened
    windows at the very end of the stream score some of their tokens again, in the reference as here)."""
    from parameter_golf_b200.eval.sliding import scored_range, window_starts
    stride = max(window // stride_div, 1)
    seen = np.zeros(total, dtype=np.int32)
    for ws in window_starts(total, window, stride):
        s, wlen = scored_range(ws, total, window, stride)
        assert 0 <= s < wlen <= window and ws + wlen <= total
        seen[ws + s: ws + wlen] += 1
    assert np.all(seen >= 1)
    first_short = next((ws for ws in window_starts(total, window, stride) if ws + window > total), total)
    assert np.all(seen[: min(first_short + window - stride, total) if first_short < total else total][: max(total - window, 0)] == 1)


@FAST
@given(pred_len=st.integers(1, 2000), chunk=st.integers(1, 300), window=st.integers(1, 600))
def test_document_chunks_tile_the_predictions_and_windows_end_with_their_chunk(pred_len, chunk, window):
    from parameter_golf_b200.eval.doc_lora import chunk_window
    window = max(window, chunk)
    n = -(-pred_len // chunk)
    covered = 0
    for ci in range(n):
        w0, wl, co, cl = chunk_window(ci, pred_len, n, chunk, window)
        assert w0 >= 0 and 0 < wl <= window and co + cl == wl and cl > 0          # the window ends where the chunk ends
        assert w0 + co == covered                                                  # chunks follow one another without gaps
        covered += cl
    assert covered == pred_len


@FAST
@given(world=st.integers(1, 8), seqs_per_rank=st.integers(1, 4), seq_len=st.sampled_from([4, 8, 16]), steps=st.integers(1, 3))
def test_rank_spans_are_disjoint_and_follow_the_stream_in_order(tmp_path_factory, world, seqs_per_rank, seq_len, steps):
    """Each global batch takes world * (L + 1) tokens off the stream, L = local tokens; rank r reads the r-th span of L + 1 tokens
    (the extra token turns a span into inputs and targets), so spans never overlap and nothing is read twice
    (train_gpt.py:486-494, pg-data/src/token_stream.rs:222-248)."""
    from parameter_golf_b200.data.shards import DistributedTokenLoader, write_shard
    d = tmp_path_factory.mktemp("p")
    L = seqs_per_rank * seq_len
    stream = (np.arange(world * (L + 1) * steps) % 60000).astype(np.uint16)
    write_shard(str(d / "fineweb_train_000000.bin"), stream)
    loaders = [DistributedTokenLoader(str(d / "fineweb_train_*.bin"), r, world) for r in range(world)]
    for s in range(steps):
        for r, ld in enumerate(loaders):
            x, y = ld.next_batch(world * L, seq_len, 1)
            lo = (s * world + r) * (L + 1)
            want = stream[lo: lo + L + 1].astype(np.int64)
            assert np.array_equal(x.reshape(-1), want[:-1]) and np.array_equal(y.reshape(-1), want[1:])
