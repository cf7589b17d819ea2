import math

import numpy as np
import pytest
import torch

from parameter_golf_b200.data.bpb import BpbLuts
from parameter_golf_b200.eval import sliding as S
from parameter_golf_b200.eval import ttt as T
from parameter_golf_b200.models import gpt
from parameter_golf_b200.models.runner import OracleRunner
from parameter_golf_b200.spec import family_preset


def spec(**ov):
    s = family_preset("tiny_cpu")
    m = s.model
    m.vocab_size, m.num_layers, m.model_dim, m.num_heads, m.num_kv_heads, m.eval_seq_len = 32, 2, 16, 4, 2, 16
    s.eval.stride, s.eval.chunk_tokens, s.eval.ttt_batch_seqs, s.eval.batch_windows = 4, 32, 2, 8
    s.apply_overrides([f"{k}={v}" for k, v in ov.items()])
    return s.validate()


def test_window_rule():
    starts = S.window_starts(100, 16, 4)
    assert starts[:3] == [0, 4, 8] and starts[-1] == 96
    assert S.scored_range(0, 100, 16, 4) == (0, 16) and S.scored_range(8, 100, 16, 4) == (12, 16)
    assert S.scored_range(96, 100, 16, 4) == (0, 4) and S.scored_range(90, 100, 16, 4) == (6, 10)
    covered = np.zeros(100, int)
    for ws in starts:
        s, w = S.scored_range(ws, 100, 16, 4)
        covered[ws + s: ws + w] += 1
    assert covered.min() >= 1 and (covered[:84] == 1).all()      # every token scored; exactly once away from the tail


def test_chunk_assignment_by_first_scored_token():
    chunks = S.build_ttt_chunks(100, 16, 4, 32)
    assert len(chunks) == 4 and chunks[0][0] == 0
    for ci, ws_list in enumerate(chunks):
        for ws in ws_list:
            s, _ = S.scored_range(ws, 100, 16, 4)
            assert min((ws + s) // 32, 3) == ci
    assert sum(len(c) for c in chunks) == len(S.window_starts(100, 16, 4, min_len=4))


def test_sliding_equals_contiguous_when_stride_is_window_and_rank_split():
    s = spec()
    p = gpt.fill_deterministic(s.model)
    r = OracleRunner(s.model, p)
    toks = np.random.default_rng(0).integers(0, 32, 16 * 6 + 1).astype(np.uint16)
    luts = BpbLuts.seeded(32)
    a = S.eval_sliding(r.nll, toks, 16, 16, luts)
    b = S.eval_contiguous(r.nll, toks, 16, luts)
    assert abs(a[0] - b[0]) < 1e-6 and abs(a[1] - b[1]) < 1e-6
    starts = S.window_starts(96, 16, 4)
    parts = S.ScoreSums()
    for rank in range(3):
        lo, hi = S.rank_slice(len(starts), rank, 3)
        parts.add(S.score_windows(r.nll, toks, starts[lo:hi], 16, 4, luts, 4))
    whole = S.score_windows(r.nll, toks, starts, 16, 4, luts, 8)
    assert abs(parts.loss - whole.loss) < 1e-4 and parts.tokens == whole.tokens and parts.bytes == whole.bytes


def test_more_context_scores_better_on_markov_data():
    from parameter_golf_b200.data.shards import generate_markov_tokens
    s = spec()
    p = gpt.fill_deterministic(s.model)
    toks = generate_markov_tokens(200, 32, seed=1)
    luts = BpbLuts.placeholder(32)
    loss, bpb = S.eval_sliding(OracleRunner(s.model, p).nll, toks, 16, 4, luts)
    assert math.isfinite(loss) and abs(bpb - loss / math.log(2) / 4) < 1e-9


@pytest.mark.parametrize("mode", ["full_sgd", "q_only", "lact"])
def test_score_first_ttt_runs_and_masks(mode):
    s = spec()
    s.eval.ttt_lr, s.eval.ttt_epochs = 0.05, 1
    p = gpt.fill_deterministic(s.model)
    before = {k: v.clone() for k, v in p.items()}
    toks = np.random.default_rng(1).integers(0, 32, 16 * 8 + 1).astype(np.uint16)
    loss, bpb = T.eval_score_first_ttt(OracleRunner(s.model, p), toks, s.model, s.eval, BpbLuts.seeded(32), mode=mode)
    assert math.isfinite(loss) and math.isfinite(bpb)
    n = s.model.num_layers
    assert not torch.equal(p["qo_bank"][:n], before["qo_bank"][:n])
    if mode == "q_only":
        assert torch.equal(p["qo_bank"][n:], before["qo_bank"][n:]) and torch.equal(p["kv_bank"], before["kv_bank"])
        assert torch.equal(p["tok_emb"], before["tok_emb"])
    else:
        assert not torch.equal(p["kv_bank"], before["kv_bank"])


def test_first_chunk_score_is_unadapted_and_last_chunk_not_trained():
    s = spec()
    s.eval.ttt_lr = 0.05
    toks = np.random.default_rng(2).integers(0, 32, 32 + 1).astype(np.uint16)       # exactly one chunk
    p = gpt.fill_deterministic(s.model)
    ref = S.eval_sliding(OracleRunner(s.model, {k: v.clone() for k, v in p.items()}).nll, toks, 16, 4, BpbLuts.seeded(32))
    before = {k: v.clone() for k, v in p.items()}
    got = T.eval_score_first_ttt(OracleRunner(s.model, p), toks, s.model, s.eval, BpbLuts.seeded(32))
    assert all(torch.equal(p[k], before[k]) for k in p)                                  # a single (= last) chunk is never trained on
    chunks = S.build_ttt_chunks(32, 16, 4, 32)
    assert sum(len(c) for c in chunks) == len(S.window_starts(32, 16, 4, min_len=4)) and math.isfinite(got[0]) and math.isfinite(ref[0])


def test_mutation_guard_trips():
    s = spec()
    p = gpt.fill_deterministic(s.model)
    r = OracleRunner(s.model, p)
    orig = r.nll

    def evil(ids, tg):
        p["qo_bank"].add_(1e-3)
        return orig(ids, tg)
    r.nll = evil
    toks = np.random.default_rng(3).integers(0, 32, 16 * 4 + 1).astype(np.uint16)
    with pytest.raises(RuntimeError, match="mutation"):
        T.eval_score_first_ttt(r, toks, s.model, s.eval, BpbLuts.seeded(32))


def test_freeze_blocks_and_cosine():
    s = spec()
    g = {k: torch.ones_like(v) for k, v in gpt.fill_deterministic(s.model).items()}
    T.mask_grads(s.model, g, "full_sgd", freeze_blocks=1)
    assert g["qo_bank"][0].abs().max() == 0 and g["qo_bank"][2].abs().max() == 0 and g["qo_bank"][1].abs().max() == 1
    assert g["mlp_up_bank"][0].abs().max() == 0 and g["tok_emb"].abs().max() == 1
    assert S.cosine_over_chunks(1.0, 0, 11) == 1.0 and abs(S.cosine_over_chunks(1.0, 10, 11)) < 1e-12


def test_lora_phased_ttt_and_deadline():
    s = spec()
    s.eval.lora_rank, s.eval.phased_ttt_phases, s.eval.ttt_lr = 4, 2, 0.05
    p = gpt.fill_deterministic(s.model)
    before = {k: v.clone() for k, v in p.items()}
    toks = np.random.default_rng(4).integers(0, 32, 16 * 8 + 1).astype(np.uint16)
    logs = []
    loss, bpb = T.eval_lora_phased_ttt(OracleRunner(s.model, p), toks, s.model, s.eval, BpbLuts.seeded(32), log=logs.append)
    assert math.isfinite(loss) and all(torch.equal(p[k], before[k]) for k in p)          # base weights untouched
    assert any(l.startswith("ttt_audit_json=") for l in logs)
    s.eval.max_eval_seconds = 1e-9
    logs.clear()
    T.eval_lora_phased_ttt(OracleRunner(s.model, p), toks, s.model, s.eval, BpbLuts.seeded(32), log=logs.append)
    assert any("deadline" in l for l in logs)


def test_prefix_doc_schedule():
    toks = np.array([5, 1, 7, 7, 1, 9, 9, 9, 1, 3] * 10, dtype=np.uint16)
    assert T.schedule_prefix_docs(toks, 1, 2, 8) == 8 and T.schedule_prefix_docs(toks, 1, 0, 8) == 0
    assert T.schedule_prefix_docs(toks, None, 2, 8) == 0


def test_slot_limits():
    tab = T.BigramCounts(8)
    prev, cur = np.array([1, 1, 1, 2]), np.array([3, 3, 4, 5])
    tab.update(prev, cur)
    logits = torch.randn(4, 8)
    neural = -torch.log_softmax(logits.double(), -1)[torch.arange(4), torch.from_numpy(cur)].numpy()
    assert np.allclose(T.slot_nll(logits, prev, cur, tab, alpha=1.0), neural)
    bg = -np.log(tab.row_probs(prev)[np.arange(4), cur])
    assert np.allclose(T.slot_nll(logits, prev, cur, tab, alpha=0.0), bg)
    assert abs(tab.row_probs(np.array([1]))[0, 3] - 3 / 11) < 1e-12                     # add-one smoothing
    mid = T.slot_nll(logits, prev, cur, tab, alpha=0.5, adaptive=True)
    assert np.isfinite(mid).all()


def test_temperature_scaling_and_its_grid_search():
    """eval.temperature divides the capped logits when scoring; the grid search scores training tokens once per temperature and
    keeps the best. A model whose logits are too flat by a known factor gets that factor back."""
    import torch.nn.functional as F
    from parameter_golf_b200.eval.sliding import find_temperature
    from parameter_golf_b200.models import gpt
    from parameter_golf_b200.models.runner import OracleRunner
    from parameter_golf_b200.spec import family_preset
    s = family_preset("tiny_cpu")
    s.model.vocab_size, s.model.num_layers, s.model.model_dim, s.model.num_heads, s.model.num_kv_heads = 32, 1, 16, 2, 1
    m = s.validate().model
    p = gpt.fill_deterministic(m)
    r = OracleRunner(m, p)
    ids = torch.randint(0, 32, (3, 12))
    tgt = torch.randint(0, 32, (3, 12))
    base = r.nll(ids, tgt)
    r.temperature = 0.5
    want = F.cross_entropy((gpt.gpt_logits(m, p, ids) / 0.5).reshape(-1, 32), tgt.reshape(-1), reduction="none").reshape(3, 12)
    assert torch.allclose(r.nll(ids, tgt), want, atol=1e-5) and not torch.allclose(base, want)
    # targets drawn from softmax(logits / 0.7): the log-likelihood is maximised near T = 0.7
    g = torch.Generator().manual_seed(0)
    stream = torch.randint(0, 32, (4097,), generator=g)
    x = stream[:-1].reshape(-1, 64)
    probs = torch.softmax(gpt.gpt_logits(m, p, x) / 0.7, -1)
    y = torch.multinomial(probs.reshape(-1, 32), 1, generator=g).reshape(x.shape)
    toks = np.concatenate([x.reshape(-1).numpy()[:1], y.reshape(-1).numpy()])          # a stream whose shift-by-one targets are y

    class Fixed:                                      # a runner that scores x against y at the current temperature
        temperature = 1.0
        def nll(self, a, b):
            rr = OracleRunner(m, p)
            rr.temperature = self.temperature
            return rr.nll(x[: a.shape[0]], y[: a.shape[0]])
    best, table = find_temperature(Fixed(), toks, 64, [0.5, 0.7, 1.0, 1.4], batch_seqs=64)
    assert best == 0.7 and table[0.7] < table[1.0] < table[1.4]


def _doc_stream(vocab, n_docs, rng, lo=20, hi=90):
    """Documents that each repeat a short private pattern (so an adapter trained on the start of a document helps on its end),
    every one opened by the boundary token 1."""
    out = []
    for _ in range(n_docs):
        pat = rng.integers(2, vocab, size=5)
        ln = int(rng.integers(lo, hi))
        out.append(np.concatenate([[1], np.tile(pat, ln // 5 + 1)[:ln]]))
    return np.concatenate(out).astype(np.uint16)


def test_documents_and_chunk_windows():
    from parameter_golf_b200.eval import doc_lora as D
    toks = np.array([9, 9, 1, 5, 6, 7, 1, 8, 1, 1, 4, 4, 4], dtype=np.uint16)
    # a document takes the next boundary token as its last target; the last one runs to the end of the stream
    assert D.find_documents(toks, 1) == [(2, 5), (6, 3), (8, 2), (9, 4)]
    assert D.find_documents(toks, 1, include_next_boundary=False) == [(2, 4), (6, 2), (9, 4)]
    assert sum(ln - 1 for _, ln in D.find_documents(toks, 1)) == len(toks) - 1 - 2            # every target after the first boundary, once
    # chunk 2 of 3 with chunks of 4 in a window of 6: ends at 10 predictions, reaches back 6, the chunk sits at offset 4
    assert D.chunk_window(2, 10, 3, 4, 6) == (4, 6, 4, 2)
    assert D.chunk_window(0, 10, 3, 4, 6) == (0, 4, 0, 4) and D.chunk_window(1, 10, 3, 4, 6) == (2, 6, 2, 4)


def test_doc_isolated_scoring_without_adapters_equals_per_document_forward():
    """rank 0 adapters: every document scored alone, each token with all of its document's earlier tokens (up to the window)."""
    from parameter_golf_b200.eval.doc_lora import eval_doc_lora_ttt, find_documents
    s = spec()
    m = s.model
    m.eval_seq_len = 64
    p = gpt.fill_deterministic(m)
    rng = np.random.default_rng(0)
    toks = _doc_stream(m.vocab_size, 7, rng, 20, 60)
    luts = BpbLuts.seeded(m.vocab_size)
    s.eval.doc_lora_rank, s.eval.doc_chunk_size, s.eval.doc_batch_size = 0, 16, 3
    loss, bpb = eval_doc_lora_ttt(p, m, toks, s.eval, luts)
    tot, nb, cnt = 0.0, 0.0, 0
    for d0, ln in find_documents(toks, 1):
        ids = torch.from_numpy(toks[d0: d0 + ln].astype(np.int64))[None]
        nll = gpt.gpt_forward(m, p, ids[:, :-1], ids[:, 1:], reduction="none")[0]
        tot += float(nll.double().sum())
        nb += float(luts.token_bytes(ids[0, :-1].numpy(), ids[0, 1:].numpy()).sum())
        cnt += ln - 1
    assert abs(loss - tot / cnt) < 1e-5 and abs(bpb - tot / math.log(2) / nb) < 1e-5
    # ranks take contiguous slices of the documents and their sums add up to the same result
    parts = []
    for r in range(2):
        got = {}
        eval_doc_lora_ttt(p, m, toks, s.eval, luts, rank=r, world=2, all_reduce=lambda t, got=got: got.setdefault("s", t.clone()))
        parts.append(got["s"])
    both = parts[0] + parts[1]
    assert abs(float(both[0] / both[2]) - loss) < 1e-6 and int(both[2]) == cnt


def test_doc_lora_ttt_scores_before_it_trains_and_never_crosses_documents():
    from parameter_golf_b200.eval import doc_lora as D
    s = spec()
    m = s.model
    m.eval_seq_len = 64
    p = gpt.init_params(m, seed=5)
    rng = np.random.default_rng(1)
    toks = _doc_stream(m.vocab_size, 6, rng, 60, 100)
    luts = BpbLuts.seeded(m.vocab_size)
    s.eval.doc_chunk_size, s.eval.doc_batch_size, s.eval.doc_lora_lr = 16, 4, 0.02
    s.eval.doc_lora_rank = 0
    base_loss, _ = D.eval_doc_lora_ttt(p, m, toks, s.eval, luts)
    s.eval.doc_lora_rank = 4
    before = {k: v.clone() for k, v in p.items()}
    loss, bpb = D.eval_doc_lora_ttt(p, m, toks, s.eval, luts)
    assert all(torch.equal(before[k], p[k]) for k in p)                      # the model itself never changes
    assert loss < base_loss - 0.02 and bpb > 0                               # repeated patterns: adapting inside a document helps
    # the first chunk of every document is scored by fresh adapters (B = 0): same numbers as without adapters
    docs = D.find_documents(toks, 1)
    short = np.concatenate([toks[d0: d0 + 16] for d0, _ in docs] + [[1]]).astype(np.uint16)      # 16 predictions = one chunk per document
    s.eval.doc_lora_rank = 0
    a, _ = D.eval_doc_lora_ttt(p, m, short, s.eval, luts)
    s.eval.doc_lora_rank = 4
    b, _ = D.eval_doc_lora_ttt(p, m, short, s.eval, luts)
    assert abs(a - b) < 1e-5
    # a document's score does not depend on which documents share its batch or come before it
    s.eval.doc_batch_size = 1
    one, _ = D.eval_doc_lora_ttt(p, m, toks, s.eval, luts, seed=0)
    s.eval.doc_batch_size = 4
    rev = np.concatenate([toks[d0: d0 + ln - (1 if i + 1 < len(docs) else 0)] for i, (d0, ln) in reversed(list(enumerate(docs)))]).astype(np.uint16)
    # (adapter A matrices are drawn per batch, so equality across batchings is statistical, not bitwise: compare the gain instead)
    two, _ = D.eval_doc_lora_ttt(p, m, rev, s.eval, luts, seed=3)
    assert abs(one - loss) < 0.05 and abs(two - loss) < 0.05 and one < base_loss and two < base_loss
    e = family_preset("tiny_cpu")
    e.apply_env({"TTT_LORA_RANK": "8", "TTT_LORA_LR": "0.01", "TTT_CHUNK_SIZE": "256", "TTT_BATCH_SIZE": "64", "TTT_EVAL_SEQ_LEN": "1024"})
    assert (e.eval.doc_lora_rank, e.eval.doc_chunk_size, e.eval.doc_batch_size, e.model.eval_seq_len) == (8, 256, 64, 1024)


def test_phases_and_the_prefix_document_warm_up_schedule():
    """pg-eval/src/gpu_lora_ttt.rs:688-750: without a prefix chunk i is in phase i * P / n; with one, the leading documents'
    chunks are phase 0 and the rest spreads over phases 1 .. P-1; the adapter's B restarts at every phase change."""
    import json
    assert T.chunk_phases(6, 3) == [0, 0, 1, 1, 2, 2] and T.chunk_phases(5, 1) == [0] * 5 and T.chunk_phases(4, 8) == [0, 2, 4, 6]
    assert T.chunk_phases(7, 3, prefix_chunks=2) == [0, 0, 1, 1, 1, 2, 2] and T.chunk_phases(4, 1, prefix_chunks=2) == [0] * 4
    assert T.chunk_phases(3, 2, prefix_chunks=9) == [0, 0, 0]
    s = spec()
    s.eval.lora_rank, s.eval.phased_ttt_phases, s.eval.ttt_lr, s.eval.chunk_tokens = 4, 3, 0.05, 32
    s.eval.phased_ttt_prefix_docs, s.eval.doc_boundary_token_id = 2, 1
    p = gpt.fill_deterministic(s.model)
    rng = np.random.default_rng(6)
    body = rng.integers(2, 32, 32 * 6 + 1).astype(np.uint16)
    body[[0, 20, 50, 90, 140]] = 1                                   # document starts: the first two documents end before token 51
    logs = []
    loss, _ = T.eval_lora_phased_ttt(OracleRunner(s.model, p), body, s.model, s.eval, BpbLuts.seeded(32), log=logs.append)
    audits = [json.loads(l.split("=", 1)[1]) for l in logs if l.startswith("ttt_audit_json=")]
    start = audits[0]
    assert start["event"] == "lora_phased_ttt_start" and start["prefix_docs"] == 2 and start["prefix_token_end"] == 32 and start["ttt_beta2"] == 0.99
    per_chunk = [a for a in audits[1:] if "chunk" in a]
    assert T.chunk_phases(6, 3, prefix_chunks=1) == [0, 1, 1, 1, 2, 2]
    assert [a["phase"] for a in per_chunk] == [0, 1, 1, 1, 2]            # the last chunk is scored and never trained on: no line
    assert [a["prefix_warmup"] for a in per_chunk] == [True] + [False] * 4 and math.isfinite(loss)


def test_replica_agreement_check_catches_a_diverged_adapter():
    lora = {"a": torch.ones(2, 3, 4), "b": torch.full((2, 4, 3), 0.5)}
    same = lambda vals, op, world, device: list(vals)
    T.replicas_agree(lora, 2, "cpu", agree_fn=same)
    other = lambda vals, op, world, device: [vals[0] + (1e-3 if op == "max" else 0.0)]          # some rank holds different factors
    with pytest.raises(RuntimeError, match="diverged"):
        T.replicas_agree(lora, 2, "cpu", agree_fn=other)


def test_evaluation_depth_recurrence_repeats_every_block():
    s = spec()
    m = s.model
    assert m.for_evaluation(0) is m and m.for_evaluation(1) is m
    e = m.for_evaluation(3)
    assert gpt.layer_schedule(e) == [(0, 0), (0, 1), (0, 2), (1, 0), (1, 1), (1, 2)] and gpt.layer_schedule(m) == [(0, 0), (1, 0)]
    assert gpt.param_shapes(e) == gpt.param_shapes(m)                      # the same weights, run more often
    p = gpt.fill_deterministic(m)
    ids = torch.randint(0, 32, (2, 16), generator=torch.Generator().manual_seed(0))
    assert float((gpt.gpt_logits(e, p, ids) - gpt.gpt_logits(m, p, ids)).abs().max()) > 1e-4
    f = family_preset("tiny_cpu").apply_env({"EVAL_DEPTH_RECURRENCE": "2"})
    assert f.eval.depth_recurrence == 2
