"""Score-first ("legal") test-time training and its variants, over the runner interface.

Every variant scores a chunk's windows with the current weights *before* any update that could have
seen those tokens, then adapts on the chunk; the last chunk is never trained on.

* `eval_score_first_ttt` — full-parameter SGD with momentum, cosine LR over chunks, gradient clip,
  rank-split sequences with gradient averaging
  (``records/track_10min_16mb/2026-03-23_LeakyReLU_LegalTTT_ParallelMuon/train_gpt.py:1074-1229``).
* ``mode="q_only"`` — only the Q half of ``qo_bank`` and ``q_gain`` receive updates
  (``parameter-golf-rs/crates/pg-eval/src/qttt.rs:151-216``).
* ``mode="lact"`` — gradients accumulated over the chunk's non-overlapping sequences, one step per epoch
  (``pg-eval/src/lact.rs:110-184,313-396``).
* `eval_lora_phased_ttt` — rank-r LoRA on the Q projection (A warm-started, B zero), B reset at phase
  changes, packed gradient all-reduce, SGD with weight decay, wallclock deadline, score-phase mutation
  guard (``pg-eval/src/gpu_lora_ttt.rs:340-682``).
* `slot_nll` — blend of the neural distribution with an add-one bigram row, fixed or entropy-adaptive
  weight (``pg-eval/src/slot.rs:35-60,119-165``).
"""
from __future__ import annotations

import json
import os
import math
import time
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np
import torch

from ..data.bpb import BpbLuts
from ..parallel.agree import agree
from ..spec import EvalSpec, ModelSpec
from .sliding import ScoreSums, build_ttt_chunks, cosine_over_chunks, rank_slice, score_windows


def _dist():
    import torch.distributed as dist
    return dist if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1 else None


def packed_all_reduce_mean(grads: Dict[str, torch.Tensor], names: List[str], all_reduce: Optional[Callable] = None):
    """Average gradients over ranks with ONE collective on a packed fp32 buffer."""
    dist = _dist()
    if dist is None and all_reduce is None:
        return
    flat = torch.cat([grads[n].reshape(-1).float() for n in names])
    if all_reduce is not None:
        all_reduce(flat)
    else:
        dist.all_reduce(flat)
        flat /= dist.get_world_size()
    off = 0
    for n in names:
        k = grads[n].numel()
        grads[n] = flat[off:off + k].reshape(grads[n].shape).to(grads[n].dtype)
        off += k


def trainable_names(model: ModelSpec, params: Dict[str, torch.Tensor], mode: str, freeze_blocks: int = 0) -> List[str]:
    if mode == "q_only":
        return ["qo_bank", "q_gain"]
    return list(params)


def mask_grads(model: ModelSpec, grads: Dict[str, torch.Tensor], mode: str, freeze_blocks: int = 0):
    n = model.num_layers
    if mode == "q_only":
        grads["qo_bank"][n:] = 0          # O half is frozen
    if freeze_blocks > 0:
        fb = min(freeze_blocks, n)
        for k, g in grads.items():
            if k in ("qo_bank", "kv_bank"):
                g[:fb] = 0
                g[n:n + fb] = 0
            elif k in ("mlp_up_bank", "mlp_down_bank", "attn_scale", "mlp_scale", "resid_mix", "q_gain",
                       "attn_gate_weight", "attn_gate_bias", "sparse_attn_gate_weight", "vr_lambda", "dtg_gate_weight", "dtg_gate_bias",
                       "block_smear_gate"):
                g[:fb] = 0


def snapshot_checksum(params: Dict[str, torch.Tensor], names: List[str]) -> float:
    return float(sum(params[n].double().sum() for n in names))


def eval_score_first_ttt(runner, tokens: np.ndarray, model: ModelSpec, ev: EvalSpec, luts: BpbLuts, rank: int = 0, world: int = 1,
                         mode: str = "full_sgd", device="cpu", log: Callable = lambda s: None,
                         all_reduce: Optional[Callable] = None) -> Tuple[float, float]:
    window, stride = model.eval_seq_len, ev.stride
    total = tokens.shape[0] - 1
    chunks = build_ttt_chunks(total, window, stride, ev.chunk_tokens)
    names = trainable_names(model, runner.params, mode, ev.ttt_freeze_blocks)
    mom = {n: torch.zeros_like(runner.params[n], dtype=torch.float32) for n in names}
    sums = ScoreSums()
    t0 = time.perf_counter()
    tok64 = tokens.astype(np.int64)
    # The adapt phase contains a collective (the packed gradient all-reduce), so every rank must skip it on the same
    # chunk: the decision is taken on the slowest rank's elapsed time, not on each rank's own.
    deadline = (lambda: agree([time.perf_counter() - t0], "max", world, device)[0] > ev.max_eval_seconds) if ev.max_eval_seconds > 0 else None
    for ci, windows in enumerate(chunks):
        if not windows:
            continue
        # ---- score (no parameter may change here) ----------------------------------------------
        before = snapshot_checksum(runner.params, names)
        a, b = rank_slice(len(windows), rank, world)
        sums.add(score_windows(runner.nll, tokens, windows[a:b], window, stride, luts, ev.batch_windows, device))
        if snapshot_checksum(runner.params, names) != before:
            raise RuntimeError("score-phase mutation detected: parameters changed while scoring")
        # ---- adapt ----------------------------------------------------------------------------------
        last = ci == len(chunks) - 1
        if last or ev.ttt_epochs <= 0 or (deadline is not None and deadline()):
            continue
        c0, c1 = ci * ev.chunk_tokens, min((ci + 1) * ev.chunk_tokens, total)
        n_seq = (c1 - c0) // window
        if n_seq <= 0:
            continue
        lr = cosine_over_chunks(ev.ttt_lr, ci, len(chunks))
        sa, sb = rank_slice(n_seq, rank, world)
        for _ in range(ev.ttt_epochs):
            acc: Optional[Dict[str, torch.Tensor]] = None
            n_acc = 0
            for bs in range(sa, max(sb, sa + 1), ev.ttt_batch_seqs):
                be = min(bs + ev.ttt_batch_seqs, sb)
                if be > bs:
                    span = tok64[c0 + bs * window: c0 + be * window + 1]
                    x = torch.from_numpy(span[:-1].reshape(-1, window)).to(device)
                    y = torch.from_numpy(span[1:].reshape(-1, window)).to(device)
                    _, grads = runner.loss_and_grads(x, y, names=names)
                else:       # a rank with no sequence still joins the collective with zero gradients
                    grads = {n: torch.zeros_like(runner.params[n]) for n in names}
                if mode == "lact":
                    acc = grads if acc is None else {n: acc[n] + grads[n] for n in names}
                    n_acc += 1
                    continue
                _apply_sgd(runner, model, grads, names, mom, lr, ev, mode, all_reduce)
            if mode == "lact" and acc is not None:
                _apply_sgd(runner, model, {n: acc[n] / n_acc for n in names}, names, mom, lr, ev, mode, all_reduce)
        if rank == 0 and (ci % 10 == 0 or last):
            l, bpb = ScoreSums(sums.loss, sums.tokens, sums.bytes).result()
            log(f"ttt_chunk [{ci + 1}/{len(chunks)}] bpb={bpb:.6f} time={time.perf_counter() - t0:.1f}s")
    return sums.all_reduce(device).result()


def _apply_sgd(runner, model, grads, names, mom, lr, ev: EvalSpec, mode, all_reduce):
    packed_all_reduce_mean(grads, names, all_reduce)
    mask_grads(model, grads, mode, ev.ttt_freeze_blocks)
    if ev.ttt_grad_clip > 0:
        tot = math.sqrt(sum(float(grads[n].float().pow(2).sum()) for n in names))
        f = min(1.0, ev.ttt_grad_clip / (tot + 1e-6))
    else:
        f = 1.0
    with torch.no_grad():
        for n in names:
            g = grads[n].float() * f
            if mom[n].device != g.device:          # the runner moves its parameters to the device on first use
                mom[n] = mom[n].to(g.device)
            mom[n].mul_(ev.ttt_momentum).add_(g)
            runner.params[n].add_(mom[n].to(runner.params[n].dtype), alpha=-lr)
    if hasattr(runner, "params_changed"):
        runner.params_changed()


# ---- LoRA phased TTT ----------------------------------------------------------------------------------------------------

def init_q_lora(model: ModelSpec, rank: int, alpha: float, device="cpu") -> dict:
    """A warm start: a fixed pseudo-random sign pattern scaled by 1/sqrt(d); B = 0 so the adapted model
    starts identical to the base model."""
    n, d = model.num_layers, model.model_dim
    idx = torch.arange(n * rank * d, dtype=torch.int64)
    h = (idx * 2654435761 + 40503) % 4294967296
    a = (((h >> 13) & 1).float() * 2 - 1).reshape(n, rank, d) / math.sqrt(d)
    return {"a": a.to(device), "b": torch.zeros(n, d, rank, device=device), "alpha": float(alpha), "trainable": True}


def schedule_prefix_docs(tokens: np.ndarray, boundary_id: Optional[int], prefix_docs: int, chunk_tokens: int) -> int:
    """Number of leading tokens covered by the first ``prefix_docs`` documents (split at
    ``boundary_id``), rounded up to whole chunks; 0 when no prefix phase is requested."""
    if prefix_docs <= 0 or boundary_id is None:
        return 0
    pos = np.flatnonzero(tokens == boundary_id)
    if pos.size < prefix_docs:
        return 0
    end = int(pos[prefix_docs - 1]) + 1
    return min(-(-end // chunk_tokens) * chunk_tokens, tokens.shape[0] - 1)


def replicas_agree(lora: dict, world: int, device, agree_fn=agree) -> None:
    """Debugging aid (``PGB_DEBUG_TTT_SYNC=1``; the reference's PG_DEBUG_DISTRIBUTED_TTT_SYNC, pg-eval/src/gpu_lora_ttt.rs:570-592):
    after an adapter update every rank must hold the same factors, since all of them applied the same averaged gradient. Compares a
    checksum of A and B across ranks (max against min) and raises on the rank(s) that see a difference."""
    cs = float(lora["a"].double().sum()) + 3.0 * float(lora["b"].double().sum()) + float(lora["b"].double().abs().sum())
    hi, lo = agree_fn([cs], "max", world, device)[0], agree_fn([cs], "min", world, device)[0]
    if abs(hi - lo) > 1e-9 * max(1.0, abs(hi)):
        raise RuntimeError(f"test-time-training replicas diverged: adapter checksum {cs!r} here, range over ranks [{lo!r}, {hi!r}]")


def chunk_phases(num_chunks: int, phases: int, prefix_chunks: int = 0) -> List[int]:
    """Phase of every chunk (``pg-eval/src/gpu_lora_ttt.rs:688-750``): without a prefix, chunk ``i`` is in phase
    ``i * phases / num_chunks``; with one, the chunks of the leading documents form phase 0 (the warm-up) and the rest is spread
    evenly over phases 1 .. phases-1."""
    phases = max(phases, 1)
    if prefix_chunks <= 0:
        return [min(i * phases // max(num_chunks, 1), phases - 1) for i in range(num_chunks)]
    prefix_chunks = min(prefix_chunks, num_chunks)
    rest = max(num_chunks - prefix_chunks, 1)
    tail = [0 if phases <= 1 else 1 + min(i * (phases - 1) // rest, phases - 2) for i in range(num_chunks - prefix_chunks)]
    return [0] * prefix_chunks + tail


def eval_lora_phased_ttt(runner, tokens: np.ndarray, model: ModelSpec, ev: EvalSpec, luts: BpbLuts, rank: int = 0, world: int = 1,
                         device="cpu", log: Callable = lambda s: None, all_reduce: Optional[Callable] = None) -> Tuple[float, float]:
    """Phased Q-LoRA test-time training: score a chunk with the adapter as it stands (guarded against mutation), then one
    pass of SGD with weight decay on the adapter only, its gradients averaged over ranks with one packed collective
    (``all_reduce``: an in-place mean over ranks, e.g. `PeerAllReduce.mean_`; default the process group); B is reset at every
    phase change. Runs on any runner, the CUDA engine included (``parameter-golf-rs/crates/pg-eval/src/gpu_lora_ttt.rs:258-568``)."""
    window, stride = model.eval_seq_len, ev.stride
    total = tokens.shape[0] - 1
    chunks = build_ttt_chunks(total, window, stride, ev.chunk_tokens)
    runner.lora = init_q_lora(model, ev.lora_rank, ev.lora_alpha, device)
    prefix_end = schedule_prefix_docs(tokens[: total + 1], ev.doc_boundary_token_id, ev.phased_ttt_prefix_docs, ev.chunk_tokens)
    phase_of = chunk_phases(len(chunks), ev.phased_ttt_phases, -(-prefix_end // ev.chunk_tokens))
    if rank == 0:
        log("ttt_audit_json=" + json.dumps({"event": "lora_phased_ttt_start", "chunks": len(chunks), "phases": max(ev.phased_ttt_phases, 1),
                                            "prefix_docs": ev.phased_ttt_prefix_docs, "prefix_token_end": prefix_end,
                                            "boundary_token_id": ev.doc_boundary_token_id, "lora_rank": ev.lora_rank, "lora_alpha": ev.lora_alpha,
                                            "weight_decay": ev.phased_ttt_weight_decay, "ttt_beta2": ev.ttt_beta2, "score_first": True}))
    sums = ScoreSums()
    t0 = time.perf_counter()
    tok64 = tokens.astype(np.int64)
    for ci, windows in enumerate(chunks):
        if ev.max_eval_seconds > 0 and agree([time.perf_counter() - t0], "max", world, device)[0] > ev.max_eval_seconds:
            log(f"ttt_deadline_reached chunk={ci}")
            break
        if ci > 0 and phase_of[ci] != phase_of[ci - 1]:
            runner.lora["b"].zero_()                         # phase change resets B
        if not windows:
            continue
        guard = float(runner.lora["b"].double().sum()) + float(runner.lora["a"].double().sum())
        a, b = rank_slice(len(windows), rank, world)
        sums.add(score_windows(runner.nll, tokens, windows[a:b], window, stride, luts, ev.batch_windows, device))
        if float(runner.lora["b"].double().sum()) + float(runner.lora["a"].double().sum()) != guard:
            raise RuntimeError("score-phase mutation detected: LoRA factors changed while scoring")
        if ci == len(chunks) - 1:
            continue
        c0, c1 = ci * ev.chunk_tokens, min((ci + 1) * ev.chunk_tokens, total)
        n_seq = (c1 - c0) // window
        sa, sb = rank_slice(n_seq, rank, world)
        lr = cosine_over_chunks(ev.ttt_lr, ci, len(chunks))
        for bs in range(sa, max(sb, sa + 1), ev.ttt_batch_seqs):
            be = min(bs + ev.ttt_batch_seqs, sb)
            if be > bs:
                span = tok64[c0 + bs * window: c0 + be * window + 1]
                x = torch.from_numpy(span[:-1].reshape(-1, window)).to(device)
                y = torch.from_numpy(span[1:].reshape(-1, window)).to(device)
                _, g = runner.loss_and_grads(x, y, names=[])
            else:
                g = {"lora.a": torch.zeros_like(runner.lora["a"]), "lora.b": torch.zeros_like(runner.lora["b"])}
            packed_all_reduce_mean(g, ["lora.a", "lora.b"], all_reduce)
            with torch.no_grad():
                for key, gk in (("a", "lora.a"), ("b", "lora.b")):
                    if ev.phased_ttt_weight_decay > 0:
                        runner.lora[key].mul_(1.0 - lr * ev.phased_ttt_weight_decay)
                    runner.lora[key].add_(g[gk], alpha=-lr)
            if world > 1 and os.environ.get("PGB_DEBUG_TTT_SYNC") == "1":
                replicas_agree(runner.lora, world, device)
        if rank == 0:
            log("ttt_audit_json=" + json.dumps({"chunk": ci, "phase": phase_of[ci], "prefix_warmup": ci * ev.chunk_tokens < prefix_end, "windows": len(windows), "lr": lr,
                                                "elapsed_s": round(time.perf_counter() - t0, 3)}))
    runner.lora = None
    return sums.all_reduce(device).result()


# ---- SLOT ------------------------------------------------------------------------------------------------------------------

class BigramCounts:
    """Add-one smoothed bigram table built from already-scored tokens."""

    def __init__(self, vocab: int):
        self.vocab = vocab
        self.counts = np.zeros((vocab, vocab), dtype=np.float64)

    def update(self, prev: np.ndarray, cur: np.ndarray):
        np.add.at(self.counts, (prev, cur), 1.0)

    def row_probs(self, prev: np.ndarray) -> np.ndarray:
        rows = self.counts[prev] + 1.0
        return rows / rows.sum(-1, keepdims=True)


def slot_nll(logits: torch.Tensor, prev: np.ndarray, targets: np.ndarray, table: BigramCounts, alpha: float = 0.9,
             adaptive: bool = False) -> np.ndarray:
    """Per-token NLL of ``alpha * softmax(logits) + (1-alpha) * bigram_row``; with ``adaptive`` the neural
    weight is ``alpha`` scaled by ``1 - H/ln V`` (low-entropy predictions keep more neural mass).
    ``alpha = 1`` is the neural model, ``alpha = 0`` the bigram model."""
    p = torch.softmax(logits.double(), dim=-1).cpu().numpy().reshape(-1, logits.shape[-1])
    bg = table.row_probs(prev.reshape(-1))
    if adaptive:
        ent = -(p * np.log(np.clip(p, 1e-30, None))).sum(-1)
        a = np.clip(alpha * (1.0 - ent / math.log(p.shape[-1])), 0.0, 1.0)[:, None]
    else:
        a = alpha
    mix = a * p + (1.0 - a) * bg
    return -np.log(np.clip(mix[np.arange(mix.shape[0]), targets.reshape(-1)], 1e-30, None))
