"""Run orchestration: validation gates, batch plan, step loop with wallclock cap, export, evaluation.

The flow mirrors ``VariantRunner::run`` (``parameter-golf-rs/crates/pg-train/src/lib.rs:864-1781``) and the
Python trainer's loop (``train_gpt.py:966-1060``): gates → model → loader → for each step
{wallclock check, LR scale, momentum warm-up, micro-batches, optimizer} → EMA/SWA application → export →
artifact budget check → evaluation → ``key=value`` result lines and one ``record_audit_json=`` line.

Backends: ``cpu`` runs the autograd oracle (one process, or gloo ranks for control-plane tests);
``cuda_single`` / ``cuda_distributed`` run the sm_100a engine (`parameter_golf_b200.models.engine`), one process
per GPU.

Command line: ``python -m parameter_golf_b200.train run [--spec file.toml | --family name] [--mode smoke|proxy|
record_shaped_proxy|record] [--env] [key=value …]`` and ``… train sweep --families a,b``.
"""
from __future__ import annotations

import argparse
import contextlib
import copy
import json
import math
import os
import sys
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np
import torch

from .data.bpb import BpbLuts
from .data.shards import DistributedTokenLoader, load_validation_tokens, write_synthetic_dataset
from .eval.sliding import eval_contiguous, eval_sliding
from .eval.ttt import eval_lora_phased_ttt, eval_score_first_ttt
from .models import gpt
from .models.runner import OracleRunner
from .parallel.agree import agree
from .optim.muon import AdamW, Ema, Lawa, Muon, ShardedMuon, Swa, clip_grads_, fraction_lr_scale, lr_scale_with_floor, muon_momentum_at, wallclock_lr_scale
from .quant.export import check_budget, code_bytes, export_model, load_artifact
from .spec import RunSpec, family_preset
from .utils.checkpoint import load_checkpoint, save_checkpoint
from .utils.logging import RunLog, StageTimers


def split_param_groups(spec: RunSpec, params: Dict[str, torch.Tensor]):
    """Optimizer grouping of the Python records (``…03-23…/train_gpt.py:1517-1529``): banks → Muon;
    embedding tables → Adam at the (tied) embedding LR; everything else → Adam at the scalar LR."""
    t = spec.train
    banks = [k for k in gpt.BANKS if k in params]
    emb = [k for k in ("tok_emb", "bigram_embed", "ve_embed") if k in params]
    head = [k for k in ("lm_head",) if k in params]
    scalars = [k for k in params if k not in banks and k not in emb and k not in head]
    emb_lr = t.tied_embed_lr if spec.model.tie_embeddings else t.embed_lr
    groups = [{"names": emb, "lr": emb_lr}, {"names": scalars, "lr": t.scalar_lr}]
    if head:
        groups.append({"names": head, "lr": t.head_lr})
    if t.matrix_optimizer == "adamw":           # the ternary script's MATRIX_OPTIMIZER=adam: no Muon, the matrices are one more AdamW group
        groups.append({"names": banks, "lr": t.adam_matrix_lr})
        banks = []
    return banks, groups


def step_batch_plan(spec: RunSpec, mode: str):
    """(global tokens per step, micro-batches per rank). Smoke and proxy modes shrink the batch
    (``pg-train/src/lib.rs:5932-5971``); the record modes keep the real arithmetic."""
    t = spec.train
    seq = t.seq_len
    world = t.world_size
    tokens = t.batch_tokens
    if mode == "smoke":
        tokens = min(tokens, world * seq * 2)
    elif mode == "proxy":
        tokens = min(tokens, world * seq * 8)
    if t.grad_accum_steps > 0:
        accum = t.grad_accum_steps
    elif t.backend == "cpu" or world > 8 or 8 % world or tokens % (8 * seq):
        accum = 1
    else:
        accum = 8 // world          # the reference's rule: the micro-batch is always 1/8 of the global batch
    return tokens, accum


def mode_max_steps(spec: RunSpec, mode: str) -> int:
    return {"smoke": min(4, spec.train.total_iterations), "proxy": min(32, spec.train.total_iterations),
            "record_shaped_proxy": min(8, spec.train.total_iterations)}.get(mode, spec.train.total_iterations)


class OracleBackend:
    """CPU / reference training backend on the autograd model with the torch optimizers."""

    def __init__(self, spec: RunSpec, params: Dict[str, torch.Tensor]):
        self.spec = spec
        self.params = params
        self.runner = OracleRunner(spec.model, params)
        self.token_weight_table = None      # [V, V] fp32 loss weights per (input token, target), see `set_token_weight_table`
        t = spec.train
        self.bank_names, self.adam_groups = split_param_groups(spec, params)
        import torch.distributed as dist
        self.sharded = (t.distributed_optimizer_backend == "sharded_parallel_muon" and dist.is_available() and dist.is_initialized()
                        and dist.get_world_size() > 1)
        if self.sharded:
            # CPU ranks: the same split of the banks as the CUDA path, with gloo reduces and all-gathers in place of the peer kernels
            self.muon = ShardedMuon([params[k] for k in self.bank_names], t.matrix_lr, t.muon_momentum, t.muon_ns_steps, t.muon_ns_profile,
                                    t.muon_wd)
        else:
            self.muon = Muon([params[k] for k in self.bank_names], t.matrix_lr, t.muon_momentum, t.muon_ns_steps,
                             t.muon_ns_profile, t.muon_wd)
        self.adam = AdamW([{"params": [params[k] for k in g["names"]], "lr": g["lr"]} for g in self.adam_groups],
                          (t.adam_beta1, t.adam_beta2), t.adam_eps, t.adam_wd)

    def train_step(self, batches, lr_scale: float, momentum: float, qat: bool) -> float:
        import torch.distributed as dist
        total: Optional[Dict[str, torch.Tensor]] = None
        loss_sum = 0.0
        for ids, tgt in batches:
            tw = None
            if self.token_weight_table is not None:
                tw = torch.from_numpy(self.token_weight_table[ids.numpy().astype(np.int64), tgt.numpy().astype(np.int64)])
            loss, g = self.runner.loss_and_grads(ids, tgt, qat=qat, token_weights=tw, mtp=self.spec.model.mtp_num_heads > 0, train=True)
            loss_sum += float(loss)
            total = g if total is None else {k: total[k] + g[k] for k in g}
        inv = 1.0 / len(batches)
        grads = {k: v * inv for k, v in total.items()}
        if self.sharded:
            return self._sharded_update(grads, lr_scale, momentum, loss_sum * inv)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            flat = torch.cat([grads[k].reshape(-1) for k in sorted(grads)])
            dist.all_reduce(flat)
            flat /= dist.get_world_size()
            off = 0
            for k in sorted(grads):
                n = grads[k].numel()
                grads[k] = flat[off:off + n].reshape(grads[k].shape)
                off += n
        if self.spec.train.grad_clip_norm > 0:
            clip_grads_(list(grads.values()), self.spec.train.grad_clip_norm)
        self.adam.step([[grads[k] for k in g["names"]] for g in self.adam_groups], lr_scale)
        self.muon.step([grads[k] for k in self.bank_names], lr=self.spec.train.matrix_lr * lr_scale, momentum=momentum)
        return loss_sum * inv

    def _sharded_update(self, grads, lr_scale: float, momentum: float, loss: float) -> float:
        """Sharded Parallel Muon on CPU ranks: the replicated (non-bank) gradients are averaged with one all-reduce, every bank
        slot's gradient goes to its owner, the clip factor comes from one scalar all-reduce in which each rank contributes
        ||replicated||^2 / world + ||own slots||^2 (``pg-train/src/lib.rs:3495-3559``), AdamW runs replicated and Muon on the
        owned slots, whose new values are then all-gathered."""
        import torch.distributed as dist
        world = dist.get_world_size()
        small = sorted(k for k in grads if k not in self.bank_names)
        flat = torch.cat([grads[k].reshape(-1) for k in small])
        dist.all_reduce(flat)
        flat /= world
        off = 0
        for k in small:
            n = grads[k].numel()
            grads[k] = flat[off:off + n].reshape(grads[k].shape)
            off += n
        own = self.muon.reduce_to_owners([grads[k] for k in self.bank_names])
        clip = self.spec.train.grad_clip_norm
        if clip > 0:
            sq = (flat.float().pow(2).sum() / world + self.muon.own_sumsq(own)).reshape(1)
            dist.all_reduce(sq)
            norm = float(sq.sqrt())
            if norm > clip:
                f = clip / (norm + 1e-6)
                flat.mul_(f)
                own = [g * f for g in own]
        self.adam.step([[grads[k] for k in g["names"]] for g in self.adam_groups], lr_scale)
        self.muon.step(own, lr=self.spec.train.matrix_lr * lr_scale, momentum=momentum)
        return loss

    def set_token_weight_table(self, table) -> None:
        self.token_weight_table = None if table is None else np.ascontiguousarray(table, dtype=np.float32)

    def state_dict(self):
        return {"muon": self.muon.state_dict(), "adam": self.adam.state_dict()}

    def load_state_dict(self, st):
        self.muon.load_state_dict(st["muon"])
        self.adam.load_state_dict(st["adam"])

    def sync_params(self) -> Dict[str, torch.Tensor]:
        return self.params


def complementary_table(spec: RunSpec, log=None) -> np.ndarray:
    """``[V, V]`` loss-weight table of complementary training: bigram counts over the first
    ``train.complementary_stats_tokens`` training tokens (every rank reads the same shards, so the tables agree without
    a collective), loaded from / saved to ``train.complementary_stats_path`` in the reference's byte layout when set."""
    from .ops import complementary as comp
    t, V = spec.train, spec.model.vocab_size
    stats = None
    path = t.complementary_stats_path
    if path and os.path.exists(path):
        with open(path, "rb") as f:
            stats = comp.BigramStats.from_bytes(f.read())
        if stats.vocab_size != V:
            raise RuntimeError(f"bigram table at {path} has vocab {stats.vocab_size}, the model {V}")
    if stats is None:
        stats = comp.stats_from_stream(t.train_data_pattern, V, t.complementary_stats_tokens)
        if path and t.rank == 0:
            tmp = path + ".tmp"
            with open(tmp, "wb") as f:
                f.write(stats.to_bytes())
            os.replace(tmp, path)
    shape = comp.WeightShape(t.complementary_shape, t.complementary_power, t.complementary_floor, t.complementary_min_w)
    table = comp.weight_table(stats, t.complementary_alpha, shape)
    if log is not None:
        log.info(f"complementary_training: alpha:{t.complementary_alpha} shape:{t.complementary_shape} "
                 f"pairs:{int(stats.row_sums.sum())} mean_weight:{float(table.mean()):.4f}")
    return table


@dataclass
class VariantResult:
    name: str = ""
    mode: str = ""
    backend: str = ""
    fingerprint: str = ""
    steps: int = 0
    train_loss_first: float = float("nan")
    train_loss_last: float = float("nan")
    train_ms: float = 0.0
    step_avg_ms: float = 0.0
    measured_ms_per_step: float = 0.0       # step time without the first train.timing_skip_steps steps
    tokens_per_step: int = 0
    tokens_per_s: float = 0.0
    stopped_early: bool = False
    artifact_bytes: int = 0
    code_bytes: int = 0
    budget_ok: bool = True
    prequant_val_loss: float = float("nan")
    prequant_val_bpb: float = float("nan")
    val_loss: float = float("nan")
    val_bpb: float = float("nan")
    eval_ms: float = 0.0
    eval_kind: str = "none"
    peak_mem_mib: int = 0
    complementary_mean_weight: float = 1.0
    eval_temperature: float = 1.0           # the logit temperature the final evaluation used (eval.temperature, or the grid's best)
    churn_history: list = field(default_factory=list)    # (step, fraction of discrete codes that changed) at every train.churn_log_every steps
    val_history: list = field(default_factory=list)      # (step, val_loss, val_bpb) of the periodic validations (train.val_loss_every)
    timers: dict = field(default_factory=dict)
    reference_keys: dict = field(default_factory=dict)   # the same facts under the names the reference trainer prints (pg-train/src/main.rs:218-431)

    def key_value_lines(self) -> List[str]:
        out = []
        for k, v in self.__dict__.items():
            if isinstance(v, list):
                continue
            if k == "reference_keys":
                out.extend(f"{kk}={vv}" for kk, vv in v.items())
                continue
            if isinstance(v, dict):
                out.extend(f"{k}.{kk}={vv}" for kk, vv in v.items())
            else:
                out.append(f"{k}={v}")
        if self.steps:
            out.append(f"train_ms_per_step={self.train_ms / self.steps:.3f}")
            # per-step derivatives of the stage totals, under the reference's naming (pg-train/src/main.rs:432-690)
            out.extend(f"timing_{k}_per_step={v / self.steps:.3f}" for k, v in self.timers.items() if k in ("data_ms", "train_step_ms", "ema_ms"))
        return out


def record_gaps(spec: RunSpec, mode: str) -> List[str]:
    """Fail-closed checklist for a record attempt (``pg-train/src/lib.rs:5533-5635``)."""
    gaps = []
    t = spec.train
    if mode == "record":
        if t.backend != "cuda_distributed":
            gaps.append("record needs the cuda_distributed backend")
        if not t.train_data_pattern or not t.validation_data_pattern:
            gaps.append("record needs real train/validation shards")
        if spec.eval.max_tokens is not None:
            gaps.append("record needs the full validation set")
        if t.world_size != 8:
            gaps.append("record is defined on 8 GPUs")
    return gaps


def code_churn(m, params: Dict[str, torch.Tensor], prev: Optional[dict]):
    """``(fraction of bank codes that differ from the previous call, the codes of this call)``: the discrete weights a ternary or
    binary QAT run would export now, compared with those of the last look
    (records/track_non_record_16mb/2026-03-24_106M_Binary_.../train_gpt_cuda_binary.py:246-261). 0 on the first call."""
    from .quant.binary import quantize_binary
    from .quant.ternary import quantize_ternary
    quant = quantize_binary if m.qat_kind == "binary" else quantize_ternary
    cur, changed, total = {}, 0, 0
    for name in gpt.BANKS:
        w = params[name].detach().float().cpu()
        cur[name] = quant(w.reshape(-1, w.shape[-1]), m.qat_ternary_group)[0]
        if prev is not None:
            changed += int((cur[name] != prev[name]).sum())
            total += cur[name].numel()
    return changed / max(total, 1), cur


def frontier_algorithm_notes(spec: RunSpec) -> List[str]:
    """Where a spec departs from the reference's late-frontier algorithm target (``pg-train/src/lib.rs:5637-5665``): CaseOps with a
    byte sidecar, SparseAttnGate of width 12, boundary-masked SmearGate, LQER. Informational: the audit line carries the list,
    nothing is refused because of it (the benchmark configurations are the Python records, which predate that target)."""
    m, notes = spec.model, []
    if not (m.caseops.enabled and m.caseops.byte_sidecar):
        notes.append("no CaseOps byte sidecar")
    elif not spec.eval.caseops_byte_sidecar_pattern:
        notes.append("CaseOps byte sidecar enabled but eval.caseops_byte_sidecar_pattern is not set")
    if not m.sparse_attn_gate.enabled:
        notes.append("no SparseAttnGate")
    elif m.sparse_attn_gate.width != 12:
        notes.append("SparseAttnGate width is not 12")
    if not m.smear_gate:
        notes.append("no SmearGate")
    elif m.smear_gate_boundary_token_id is None:
        notes.append("SmearGate is not masked at document boundaries: the previous-token mix can cross packed documents")
    if not spec.quant.lqer.enabled:
        notes.append("no LQER correction")
    return notes


def preflight(spec: RunSpec) -> Tuple[List[str], bool]:
    """``(key=value lines, ok)``: what can be verified about a run before any process group or device exists, for every rank at once
    (the reference keeps a metadata-only communicator so that its CPU build can do this per-rank data check,
    pg-core/src/nccl.rs:125-134, pg-train/src/lib.rs:879-886): spec validation and record gates, the training and validation
    shards (headers, token counts, how often the run would wrap around its data, per-rank span arithmetic), tokenizer and byte
    sidecar, the engine's memory estimate against one GPU, the artifact directory and the counted code size."""
    import glob as _glob
    from .data.shards import is_byte_sidecar_path, read_shard_header
    out, problems = [], []
    t, m, e = spec.train, spec.model, spec.eval
    try:
        spec.validate()
    except ValueError as exc:
        problems.append(str(exc))
    gaps = record_gaps(spec, spec.mode)
    out.append(f"preflight.mode={spec.mode}")
    out.append(f"preflight.record_gaps={json.dumps(gaps)}")
    if gaps and not spec.allow_unsupported_variants:
        problems.append("record gates: " + "; ".join(gaps))
    tokens_per_step, accum = step_batch_plan(spec, spec.mode)
    steps = mode_max_steps(spec, spec.mode)
    world = max(t.world_size, 1)
    if tokens_per_step % (world * accum * t.seq_len):
        problems.append(f"{tokens_per_step} tokens per step do not split into whole sequences of {t.seq_len} over {world} ranks x {accum} micro-batches")
    out += [f"preflight.tokens_per_step={tokens_per_step}", f"preflight.grad_accum={accum}", f"preflight.steps={steps}",
            f"preflight.local_sequences_per_micro_batch={tokens_per_step // max(world * accum * t.seq_len, 1)}"]
    for kind, pattern in (("train", t.train_data_pattern), ("val", t.validation_data_pattern)):
        if not pattern:
            out.append(f"preflight.{kind}_data=synthetic (generated by rank 0 at start-up)")
            continue
        files = sorted(f for f in _glob.glob(pattern) if not is_byte_sidecar_path(f))
        total = 0
        for f in files:
            try:
                total += read_shard_header(f)
            except Exception as exc:            # noqa: BLE001 - every bad shard is reported
                problems.append(f"{f}: {exc}")
        out += [f"preflight.{kind}_shards={len(files)}", f"preflight.{kind}_tokens={total}"]
        if not files:
            problems.append(f"no {kind} shard matches {pattern!r}")
        elif kind == "train":
            need = steps * (tokens_per_step + world * accum)          # every rank and micro-batch reads one token more than it trains on
            out += [f"preflight.train_tokens_needed={need}", f"preflight.train_data_passes={need / max(total, 1):.3f}"]
            if total < tokens_per_step + world * accum:
                problems.append(f"the training shards hold {total} tokens, one step needs {tokens_per_step + world * accum}")
        elif total < m.eval_seq_len + 1:
            problems.append(f"the validation shards hold {total} tokens, one window needs {m.eval_seq_len + 1}")
    if e.tokenizer_vocab_path and not os.path.isfile(e.tokenizer_vocab_path):
        problems.append(f"eval.tokenizer_vocab_path {e.tokenizer_vocab_path!r} does not exist")
    if e.caseops_byte_sidecar_pattern:
        side = sorted(_glob.glob(e.caseops_byte_sidecar_pattern))
        out.append(f"preflight.byte_sidecar_shards={len(side)}")
        if not side:
            problems.append(f"no byte sidecar matches {e.caseops_byte_sidecar_pattern!r}")
    if t.backend != "cpu" and not problems:
        from .plan import HBM_BYTES_B200, estimate_engine_memory
        mem = estimate_engine_memory(spec, tokens_per_step // (world * accum)).total
        out.append(f"preflight.engine_memory_gib={mem / 2 ** 30:.2f}")
        if mem > 0.95 * HBM_BYTES_B200:
            problems.append(f"the engine's buffers are estimated at {mem / 2 ** 30:.1f} GiB, more than one GPU holds")
    art_dir = os.path.dirname(os.path.abspath(t.artifact_path))
    probe = art_dir
    while not os.path.isdir(probe):
        probe = os.path.dirname(probe)
    if not os.access(probe, os.W_OK):
        problems.append(f"the artifact directory {art_dir!r} cannot be written")
    cb = code_bytes()
    out += [f"preflight.code_bytes={cb}", f"preflight.artifact_budget_bytes={spec.quant.target_artifact_bytes - cb}"]
    if spec.quant.target_artifact_bytes - cb <= 0:
        problems.append("the counted source alone exceeds quant.target_artifact_bytes (set PG_SUBMISSION_CODE_BYTES to the submission's real code size)")
    out += [f"preflight.problem={p}" for p in problems]
    out.append(f"preflight.ok={str(not problems).lower()}")
    return out, not problems


def check_record_step_time(mode: str, steps: int, measured_ms_per_step: float, limit_ms: float) -> None:
    """A record run whose measured step time is above the limit is refused before export (``pg-train/src/lib.rs:1514-1521``)."""
    if mode == "record" and limit_ms > 0 and steps > 0 and measured_ms_per_step > limit_ms:
        raise RuntimeError(f"record run is too slow for a submission: measured_ms_per_step={measured_ms_per_step:.3f} "
                           f"max_ms_per_step={limit_ms:.3f} (train.record_max_ms_per_step=0 only for debugging)")


class VariantRunner:
    def __init__(self, spec: RunSpec, log: Optional[RunLog] = None, backend_factory: Optional[Callable] = None):
        self.spec = spec.validate()
        self.log = log or RunLog(spec.name)
        self.backend_factory = backend_factory
        self.clock: Callable[[], float] = time.perf_counter      # seconds; the training loop's only time source

    def _make_backend(self, params):
        if self.backend_factory is not None:
            return self.backend_factory(self.spec, params)
        if self.spec.train.backend == "cpu":
            return OracleBackend(self.spec, params)
        from .models.engine import EngineBackend       # needs the CUDA extension
        return EngineBackend(self.spec, params)

    def run(self, mode: Optional[str] = None) -> VariantResult:
        spec = self.spec
        mode = mode or spec.mode
        t, m = spec.train, spec.model
        log = self.log
        gaps = record_gaps(spec, mode)
        if gaps and not spec.allow_unsupported_variants:
            raise RuntimeError("record gate failed: " + "; ".join(gaps))
        res = VariantResult(name=spec.name, mode=mode, backend=t.backend, fingerprint=f"{spec.fingerprint():016x}")
        timers = StageTimers()
        torch.manual_seed(t.seed)
        np.random.seed(t.seed)
        device = "cpu" if t.backend == "cpu" else f"cuda:{int(os.environ.get('LOCAL_RANK', 0))}"

        # ---- data ----------------------------------------------------------------------------------
        synthetic_data = not t.train_data_pattern
        if not t.train_data_pattern:
            root = os.path.join(os.environ.get("PGB_DATA_ROOT", "/tmp/pgb200_synth"), f"v{m.vocab_size}_s{t.seed}")
            # One writer: rank 0 generates (each shard is written to a temporary name and renamed), the others wait at a
            # barrier before any of them opens a shard.
            if t.rank == 0:
                write_synthetic_dataset(root, m.vocab_size, train_tokens=max(4 * t.batch_tokens, 1 << 20),
                                        val_tokens=max(4 * m.eval_seq_len * 8 + 1, 1 << 16), seed=t.seed)
            if t.world_size > 1:
                import torch.distributed as dist
                if dist.is_available() and dist.is_initialized():
                    dist.barrier()
                elif not os.path.exists(os.path.join(root, "fineweb_val_000000.bin")):
                    raise RuntimeError("synthetic data is generated by rank 0; the other ranks need a process group to wait for it")
            t.train_data_pattern = os.path.join(root, "fineweb_train_*.bin")
            t.validation_data_pattern = os.path.join(root, "fineweb_val_*.bin")
        loader = DistributedTokenLoader(t.train_data_pattern, t.rank, t.world_size)
        tokens_per_step, accum = step_batch_plan(spec, mode)
        res.tokens_per_step = tokens_per_step

        # ---- model + backend ------------------------------------------------------------------------
        params = gpt.init_params(m, t.seed, device="cpu")
        backend = self._make_backend(params)
        if t.complementary_alpha > 0:
            table = complementary_table(spec, log)
            backend.set_token_weight_table(table)
            res.complementary_mean_weight = float(table.mean())
        fused_ema = getattr(backend, "fused_ema", False)       # CUDA engine: EMA is updated inside the optimizer kernels
        ema = Ema(t.ema_decay) if (t.ema_decay > 0 and not fused_ema) else None
        swa = Swa(t.swa_every, t.swa_threshold) if t.swa_enabled else None
        lawa = Lawa(t.lawa_k, t.lawa_freq) if t.lawa_enabled else None
        step0 = 0
        if t.resume_from:
            ck = load_checkpoint(t.resume_from)
            if ck["fingerprint"] != res.fingerprint:
                raise RuntimeError("checkpoint fingerprint does not match this run spec")
            for k, v in ck["params"].items():
                backend.sync_params()[k].copy_(v)
            backend.load_state_dict(ck["optim"])
            loader.restore(ck["loader"])
            step0 = int(ck["step"])
            if ema is not None and ck.get("ema") is not None:
                ema.shadow = ck["ema"]
            torch.set_rng_state(ck["rng"])
            if hasattr(backend, "params_changed"):
                backend.params_changed()
            log.info(f"resumed from {t.resume_from} at step {step0}")
        if hasattr(backend, "train_step_spans"):
            # CUDA backends read through the C++ loader: a worker thread keeps page-locked spans ahead of the step loop
            from .data.native_loader import NativeTokenLoader
            fast = NativeTokenLoader(t.train_data_pattern, t.rank, t.world_size)
            fast.restore(loader.stream.state())
            fast.start_prefetch(tokens_per_step, accum)
            loader = fast

        max_steps = mode_max_steps(spec, mode)
        max_ms = 1000.0 * t.max_wallclock_seconds if t.max_wallclock_seconds > 0 else None
        qat = t.qat_enabled
        if t.prime_steps > 0 and t.backend != "cpu":
            log.info(f"warmup_steps:{t.prime_steps} skipped: the CUDA engine compiles nothing at run time")
        if t.prime_steps > 0 and step0 == 0 and t.backend == "cpu":
            # priming: real steps whose every effect is undone afterwards (train_gpt.py:937-961)
            keep_p = {k: v.detach().clone() for k, v in backend.sync_params().items()}
            keep_o, keep_l, keep_r = copy.deepcopy(backend.state_dict()), loader.state(), torch.get_rng_state()
            for ws in range(t.prime_steps):
                prime = [tuple(torch.from_numpy(a) for a in loader.next_batch(tokens_per_step, t.seq_len, accum)) for _ in range(accum)]
                backend.train_step(prime, 1.0, t.muon_momentum_warmup_start, qat)
                log.info(f"warmup_step:{ws + 1}/{t.prime_steps}")
            for k, v in keep_p.items():
                backend.sync_params()[k].copy_(v)
            backend.load_state_dict(keep_o)
            loader.restore(keep_l)
            torch.set_rng_state(keep_r)
        log.info(f"model_params:{gpt.count_params(m)} world_size:{t.world_size} grad_accum_steps:{accum} "
                 f"train_batch_tokens:{tokens_per_step} train_seq_len:{t.seq_len} iterations:{max_steps}")
        train_ms = 0.0
        step = step0
        t_start = self.clock()
        # curriculum: shorter sequences / a smaller global batch until a fraction of the budget has passed
        unit = t.world_size * accum
        cur_seq = t.seq_len_start if 0 < t.seq_len_start < t.seq_len else t.seq_len
        cur_tokens = tokens_per_step
        if 0 < t.batch_tokens_start < tokens_per_step:
            cur_tokens = max(t.batch_tokens_start // (unit * t.seq_len), 1) * unit * t.seq_len     # whole sequences of either length per micro-batch
        health = None
        if t.world_size > 1:
            from .parallel.health import RankHealth
            health = RankHealth.from_process_group(timeout_s=float(os.environ.get("PGB_HEALTH_TIMEOUT_S", "120")))
        val_cache = {}
        churn_prev = None
        skipped_ms = 0.0

        def validate_now():
            """Periodic validation of the baseline trainer (train_gpt.py:964-994): the current weights on non-overlapping
            validation sequences, every rank on its slice; its time does not count as training time."""
            nonlocal train_ms, t_start
            train_ms += 1000.0 * (self.clock() - t_start)
            t_val = time.perf_counter()
            if not val_cache:
                limit = spec.eval.max_tokens if mode == "record" else min(spec.eval.max_tokens or (1 << 62), 8 * m.eval_seq_len)
                val_cache["tokens"] = load_validation_tokens(t.validation_data_pattern, m.eval_seq_len, limit)
                val_cache["luts"] = (BpbLuts.from_sentencepiece(spec.eval.tokenizer_vocab_path, m.vocab_size) if spec.eval.tokenizer_vocab_path
                                     else BpbLuts.seeded(m.vocab_size, spec.eval.byte_table_seed))
            # CUDA backends: a host copy with the sharded banks gathered from their owners (a collective: every rank is at this step)
            cur = backend.final_params(ema=False) if fused_ema else backend.sync_params()
            if t.backend == "cpu":
                runner_v, vdev = OracleRunner(m, cur), "cpu"
            else:
                from .models.engine import EngineRunner
                runner_v, vdev = EngineRunner(spec, cur, device, train=False), device
            # sequences per forward: the baseline's VAL_BATCH_SIZE split over ranks and micro-batches (train_gpt.py:238-247), never
            # more than the evaluation batch the spec allows
            seqs = max(min(t.val_batch_size // max(t.world_size * accum * m.eval_seq_len, 1), spec.eval.batch_windows), 1)
            vl, vb = eval_contiguous(runner_v.nll, val_cache["tokens"], m.eval_seq_len, val_cache["luts"], t.rank, t.world_size, seqs, vdev)
            del runner_v
            res.val_history.append((step, vl, vb))
            log.info(f"step:{step}/{max_steps} val_loss:{vl:.4f} val_bpb:{vb:.4f} train_time:{train_ms:.0f}ms "
                     f"step_avg:{train_ms / max(step - step0, 1):.2f}ms eval_time:{1000.0 * (time.perf_counter() - t_val):.0f}ms")
            t_start = self.clock()

        while step < max_steps:
            if health is not None:
                health.check()        # a peer that failed or went silent ends this rank on the host, before its next launch
            elapsed = train_ms + 1000.0 * (self.clock() - t_start)
            if max_ms is not None and t.world_size > 1:
                # Every rank acts on the slowest rank's clock: the stop, the wall-clock learning-rate scale and the switches
                # driven by it (late QAT, SWA) then flip on the same step everywhere (train_gpt.py:1049-1053 reduces its
                # reached_cap flag the same way). A rank that left the loop alone would strand its peers' collectives.
                elapsed = agree([elapsed], "max", t.world_size, device)[0]
            if max_ms is not None and elapsed >= max_ms:
                res.stopped_early = True
                log.info(f"stopping_early: wallclock_cap train_time:{elapsed:.0f}ms step:{step}/{max_steps}")
                break
            if t.wallclock_warmdown and max_ms is not None and t.warmdown_frac > 0:
                scale = fraction_lr_scale(step, elapsed, max_steps, t.warmdown_frac, max_ms)    # the last fraction of the time budget
            elif t.wallclock_warmdown and max_ms is not None:
                scale = wallclock_lr_scale(step, elapsed, max_steps, t.warmdown_iters, max_ms)
            else:
                # counted against the configured run length, not the (shorter) length of a smoke or proxy run, as the reference
                # does (pg-train/src/lib.rs:1105-1111; warm-down length from the fraction as in pg-model/src/spec.rs:527-531)
                total = max(t.total_iterations, max_steps)
                wd = int(round(total * t.warmdown_frac)) if t.warmdown_frac > 0 else min(t.warmdown_iters, total)
                scale = lr_scale_with_floor(step, t.warmup_steps, total, wd, t.min_lr_scale) if (wd or t.warmup_steps) else 1.0
            if t.qat_fraction > 0 and not qat and (elapsed / max_ms if max_ms is not None else step / max(max_steps, 1)) >= 1.0 - t.qat_fraction:
                qat = True
                log.info(f"late_qat:enabled step:{step} by qat_fraction:{t.qat_fraction}")
            if t.late_qat_threshold > 0 and scale < t.late_qat_threshold and not qat:
                qat = True
                log.info(f"late_qat:enabled step:{step} scale:{scale:.4f}")
            mom = muon_momentum_at(step, t.muon_momentum_warmup_start, t.muon_momentum, t.muon_momentum_warmup_steps)
            progress = elapsed / max_ms if max_ms is not None else step / max(max_steps, 1)
            if cur_seq != t.seq_len and progress >= t.seq_schedule_fraction:
                log.info(f"step:{step} seq_len_switch:{cur_seq}->{t.seq_len}")
                cur_seq = t.seq_len
            if cur_tokens != tokens_per_step and progress >= t.batch_schedule_fraction:
                log.info(f"step:{step} batch_switch:{cur_tokens}->{tokens_per_step}")
                cur_tokens = tokens_per_step
            with timers.time("data"):
                batches, spans = [], None
                if hasattr(backend, "train_step_spans"):
                    spans = [loader.next_prefetched() for _ in range(accum)]     # page-locked uint16 spans (2 bytes per token over PCIe)
                else:
                    for _ in range(accum):
                        x, y = loader.next_batch(cur_tokens, cur_seq, accum)
                        batches.append((torch.from_numpy(x), torch.from_numpy(y)))
            with timers.time("train_step"), (health.guard() if health is not None else contextlib.nullcontext()):
                loss = backend.train_step_spans(spans, scale, mom, qat) if spans is not None else backend.train_step(batches, scale, mom, qat)
            step += 1
            if step - step0 == t.timing_skip_steps and step < max_steps:
                skipped_ms = train_ms + 1000.0 * (self.clock() - t_start)
            if health is not None:
                health.beat(step)
            if step == step0 + 1:
                res.train_loss_first = loss
            res.train_loss_last = loss
            if ema is not None and progress >= t.ema_start_fraction:
                with timers.time("ema"):
                    ema.update(backend.sync_params())
            if swa is not None and swa.should_collect(step, scale):
                swa.collect(backend.final_params(ema=False) if fused_ema else backend.sync_params())
            if lawa is not None and lawa.should_collect(step):
                lawa.collect(backend.final_params(ema=False) if fused_ema else backend.sync_params())
            now_ms = train_ms + 1000.0 * (self.clock() - t_start)
            if t.train_log_every > 0 and (step <= 10 or step % t.train_log_every == 0 or step == max_steps):
                log.info(f"step:{step}/{max_steps} train_loss:{loss:.4f} train_time:{now_ms:.0f}ms step_avg:{now_ms / (step - step0):.2f}ms")
            if t.churn_log_every > 0 and step % t.churn_log_every == 0 and t.backend == "cpu" and m.qat_kind in ("ternary", "binary"):
                frac, churn_prev = code_churn(m, backend.sync_params(), churn_prev)
                log.info(f"step:{step} churn:{frac:.4f}")
                res.churn_history.append((step, frac))
            if t.val_loss_every > 0 and t.validation_data_pattern and (step % t.val_loss_every == 0 or step == max_steps):
                validate_now()
            if t.checkpoint_every > 0 and t.checkpoint_path and step % t.checkpoint_every == 0:
                # Every rank takes part: the sharded optimizer gathers its state from the slot owners (a collective), rank 0
                # writes, and the others wait for the write at a host barrier instead of starting a step whose device-side
                # waits would run out while rank 0 is still in fsync.
                opt_state = backend.state_dict()
                if t.rank == 0:
                    save_checkpoint(t.checkpoint_path, res.fingerprint, step, backend.sync_params(), opt_state,
                                    loader.state(), ema.shadow if ema else None)
                if t.world_size > 1:
                    import torch.distributed as dist
                    if dist.is_available() and dist.is_initialized():
                        dist.barrier()
        train_ms += 1000.0 * (self.clock() - t_start)
        if hasattr(loader, "stop_prefetch"):
            loader.stop_prefetch()
        res.steps = step - step0
        res.train_ms = train_ms
        res.step_avg_ms = train_ms / max(res.steps, 1)
        # the measured step time leaves out the first timing_skip_steps steps (pg-train/src/lib.rs:4129-4134, :1509-1521)
        timed_steps = res.steps - min(t.timing_skip_steps, max(res.steps - 1, 0))
        res.measured_ms_per_step = (train_ms - skipped_ms) / max(timed_steps, 1)
        if not spec.allow_unsupported_variants:          # the development switch that waives the other record gates waives this one too
            check_record_step_time(mode, res.steps, res.measured_ms_per_step, t.record_max_ms_per_step)
        res.tokens_per_s = tokens_per_step * res.steps / max(train_ms / 1000.0, 1e-9)
        if torch.cuda.is_available() and t.backend != "cpu":
            res.peak_mem_mib = torch.cuda.max_memory_allocated() // (1 << 20)
            log.info(f"peak memory allocated: {res.peak_mem_mib} MiB")

        # ---- weight averaging, export, budget ---------------------------------------------------------
        if fused_ema:
            final = backend.final_params(ema=t.ema_decay > 0)
            if t.ema_decay > 0:
                log.info("ema:applying EMA weights")
        else:
            final = {k: v.detach().cpu().float().clone() for k, v in backend.sync_params().items()}
        if lawa is not None and lawa.count > 1:
            log.info(f"lawa:applying LAWA averaging k={lawa.count}")
            final = lawa.average()
        elif swa is not None and swa.count > 1:
            log.info(f"swa:applying {swa.count} snapshots")
            final = {k: v.cpu() for k, v in swa.average().items()}
        elif ema is not None and ema.shadow is not None:
            log.info("ema:applying EMA weights")
            final = {k: v.cpu().clone() for k, v in ema.shadow.items()}
        # ---- diagnostic before quantisation: the averaged fp32 weights on non-overlapping validation sequences ----------
        # (the reference logs the same right after applying EMA, train_gpt.py of the 2026-03-23 record: "post-EMA diagnostic")
        if mode == "record" and t.validation_data_pattern:
            with timers.time("prequant_eval"):
                t_diag = time.perf_counter()
                val_d = load_validation_tokens(t.validation_data_pattern, m.eval_seq_len, spec.eval.max_tokens)
                luts_d = (BpbLuts.from_sentencepiece(spec.eval.tokenizer_vocab_path, m.vocab_size) if spec.eval.tokenizer_vocab_path
                          else BpbLuts.seeded(m.vocab_size, spec.eval.byte_table_seed))
                if t.backend == "cpu":
                    runner_d, ddev = OracleRunner(m, final), "cpu"
                else:
                    from .models.engine import EngineRunner
                    runner_d, ddev = EngineRunner(spec, final, device, train=False), device
                res.prequant_val_loss, res.prequant_val_bpb = eval_contiguous(runner_d.nll, val_d, m.eval_seq_len, luts_d, t.rank, t.world_size,
                                                                              spec.eval.batch_windows, ddev)
                del runner_d
                log.info(f"prequant_diagnostic val_loss:{res.prequant_val_loss:.4f} val_bpb:{res.prequant_val_bpb:.4f} "
                         f"eval_time:{1000.0 * (time.perf_counter() - t_diag):.0f}ms")
        with timers.time("export"):
            precomputed = None
            if spec.quant.scheme == "full_gptq_int6" and spec.quant.calibration == "self_generated":
                from .quant.calibrate import self_generated_hessians
                from .quant.gptq import gptq_quantize_model
                hess = self_generated_hessians(spec, final, device=device if t.backend != "cpu" else "cpu",
                                               num_seqs=spec.quant.gptq_calibration_batches if mode == "record" else 2,
                                               seq_len=m.train_seq_len if mode == "record" else min(m.train_seq_len, 64))
                precomputed = gptq_quantize_model(spec, final, hess, device=device if t.backend != "cpu" else None)
            blob = export_model(spec, final, t.artifact_path if t.rank == 0 else None, precomputed) if spec.quant.scheme != "none" else b""
        res.artifact_bytes = len(blob)
        res.code_bytes = code_bytes()
        res.budget_ok = check_budget(res.artifact_bytes, res.code_bytes, spec.quant.target_artifact_bytes)
        log.info(f"artifact_bytes:{res.artifact_bytes} code_bytes:{res.code_bytes} budget_ok:{res.budget_ok}")
        if mode == "record" and not res.budget_ok:
            raise RuntimeError("artifact + code exceed the byte budget")

        # ---- evaluation on the round-tripped artifact ---------------------------------------------------
        with timers.time("eval"):
            t_eval = time.perf_counter()
            eval_params = load_artifact(blob, spec) if blob else final
            val = load_validation_tokens(t.validation_data_pattern, m.eval_seq_len, spec.eval.max_tokens if mode == "record" else
                                         min(spec.eval.max_tokens or (1 << 62), 8 * m.eval_seq_len))
            luts = (BpbLuts.from_sentencepiece(spec.eval.tokenizer_vocab_path, m.vocab_size) if spec.eval.tokenizer_vocab_path
                    else BpbLuts.seeded(m.vocab_size, spec.eval.byte_table_seed))
            if spec.eval.caseops_byte_sidecar_pattern:
                from .data.shards import load_validation_byte_sidecar
                luts = luts.with_sidecar(load_validation_byte_sidecar(spec.eval.caseops_byte_sidecar_pattern)[: val.shape[0]])
            if t.backend == "cpu":
                runner = OracleRunner(m.for_evaluation(spec.eval.depth_recurrence), eval_params)
                runner.temperature = spec.eval.temperature
                edev = "cpu"
                if spec.eval.auto_temperature:
                    # the ternary / binary scripts' TEMP_SCALING: the grid is scored on training tokens with the round-tripped
                    # model, the best value scales the logits of the final evaluation (train_gpt_cuda_ternary.py find_temp)
                    from .eval.sliding import find_temperature
                    calib = load_validation_tokens(t.train_data_pattern, m.eval_seq_len, min(spec.eval.temperature_calibration_tokens,
                                                                                             8 * m.eval_seq_len if mode != "record" else 1 << 62))
                    best, table = find_temperature(runner, calib, m.eval_seq_len, spec.eval.temperature_grid)
                    runner.temperature = res.eval_temperature = best
                    log.info("temperature_search:" + json.dumps({str(k): round(v, 6) for k, v in table.items()}) + f" optimal_T:{best}")
            else:
                if spec.eval.temperature != 1.0:
                    raise RuntimeError("eval.temperature != 1 is scored by the autograd runner (train.backend=cpu or evalcli --device cpu)")
                from .models.engine import EngineRunner
                runner = EngineRunner(spec, eval_params, device)
                edev = device
            ab = spec.eval.adaptation_backend
            if spec.eval.legal_score_first and ab in ("full_sgd", "cpu_q_only", "lact"):
                emode = {"full_sgd": "full_sgd", "cpu_q_only": "q_only", "lact": "lact"}[ab]
                res.val_loss, res.val_bpb = eval_score_first_ttt(runner, val, m, spec.eval, luts, t.rank, t.world_size, emode, edev, log.info)
                res.eval_kind = f"score_first_{emode}"
            elif spec.eval.legal_score_first and ab == "gpu_lora_phased":
                res.val_loss, res.val_bpb = eval_lora_phased_ttt(runner, val, m, spec.eval, luts, t.rank, t.world_size, edev, log.info)
                res.eval_kind = "lora_phased"
            elif spec.eval.legal_score_first and ab == "doc_lora":
                from .eval.doc_lora import eval_doc_lora_ttt
                hook = None
                if t.world_size > 1:
                    import torch.distributed as dist

                    def hook(x):
                        dev_x = x.to(edev) if edev != "cpu" else x
                        dist.all_reduce(dev_x)
                        x.copy_(dev_x.cpu())
                res.val_loss, res.val_bpb = eval_doc_lora_ttt(runner.params, m, val, spec.eval, luts, t.rank, t.world_size, edev, log.info,
                                                              all_reduce=hook, betas=(t.adam_beta1, t.adam_beta2))
                res.eval_kind = "doc_lora"
            else:
                res.val_loss, res.val_bpb = eval_sliding(runner.nll, val, m.eval_seq_len, spec.eval.stride, luts, t.rank, t.world_size,
                                                         spec.eval.batch_windows, edev)
                res.eval_kind = "sliding"
            res.eval_ms = 1000.0 * (time.perf_counter() - t_eval)
        log.info(f"final_{res.eval_kind}_roundtrip val_loss:{res.val_loss:.4f} val_bpb:{res.val_bpb:.4f} eval_time:{res.eval_ms:.0f}ms")
        log.info(f"final_{res.eval_kind}_roundtrip_exact val_loss:{res.val_loss:.8f} val_bpb:{res.val_bpb:.8f}")     # train_gpt.py:1119
        res.timers = timers.summary()
        tm = res.timers
        res.reference_keys = {
            "run_name": spec.name, "train_backend": t.backend, "variant_fingerprint": res.fingerprint, "steps_completed": res.steps,
            "train_loss": f"{res.train_loss_last:.6f}", "train_loss_source": "last_step_mean_over_local_microbatches",
            "ms_per_step": f"{res.measured_ms_per_step:.3f}", "wallclock_seconds": f"{res.train_ms / 1000.0:.3f}",
            "timing_steps": max(res.steps - min(t.timing_skip_steps, max(res.steps - 1, 0)), 0), "rank": t.rank, "world_size": t.world_size,
            "seq_len": t.seq_len, "global_batch_tokens": tokens_per_step, "tokens_seen_global": tokens_per_step * res.steps,
            "distributed_sync": "none" if t.world_size == 1 else t.distributed_optimizer_backend,
            "attention_backend": "autograd_reference" if t.backend == "cpu" else "native_tcgen05_flash",
            "eval_adaptation_backend": spec.eval.adaptation_backend, "frontier_record_ready": str(not gaps).lower(),
            "bank_update_backend": "torch" if t.backend == "cpu" else "fused_kernels",
            "train_data_source": "shards" if not synthetic_data else "synthetic_zipf_markov",
            "bpb_byte_source": ("caseops_sidecar" if spec.eval.caseops_byte_sidecar_pattern else "tokenizer" if spec.eval.tokenizer_vocab_path
                                else "seeded_table"),
            "timing_backend": "host_perf_counter" if t.backend == "cpu" else "cuda_events_max_over_ranks",
            "timing_train_step_ms": tm.get("train_step_ms", 0.0), "timing_data_sampling_ms": tm.get("data_ms", 0.0),
            "timing_artifact_export_ms": tm.get("export_ms", 0.0), "timing_eval_ms": tm.get("eval_ms", 0.0)}
        if t.rank == 0:
            def finite(x):          # strict JSON has no NaN: a value that was not measured is null
                if isinstance(x, float) and not math.isfinite(x):
                    return None
                if isinstance(x, dict):
                    return {k: finite(v) for k, v in x.items()}
                if isinstance(x, (list, tuple)):
                    return [finite(v) for v in x]
                return x
            log.raw("record_audit_json=" + json.dumps(finite({
                "name": spec.name, "mode": mode, "fingerprint": res.fingerprint, "backend": t.backend,
                "distributed_optimizer_backend": t.distributed_optimizer_backend, "world_size": t.world_size,
                "tokens_per_step": tokens_per_step, "grad_accum": accum, "seq_len": t.seq_len, "steps": res.steps,
                "step_avg_ms": round(res.step_avg_ms, 3), "ns_profile": t.muon_ns_profile, "grad_wire_dtype": t.grad_wire_dtype,
                "quant_scheme": spec.quant.scheme, "compression": spec.quant.compression, "artifact_bytes": res.artifact_bytes,
                "eval_kind": res.eval_kind, "gaps": gaps, "frontier_algorithm_notes": frontier_algorithm_notes(spec), "timing_backend": "host_perf_counter" if t.backend == "cpu" else "cuda_events_max_over_ranks",
                # everything that shaped the run, so that a result can be traced to its configuration from the log alone
                # (the reference's audit line carries every switch, pg-train/src/lib.rs:4227-4824)
                "measured_ms_per_step": round(res.measured_ms_per_step, 3), "tokens_per_s": round(res.tokens_per_s, 1), "stopped_early": res.stopped_early,
                "train_loss_first": res.train_loss_first, "train_loss_last": res.train_loss_last, "val_loss": res.val_loss, "val_bpb": res.val_bpb,
                "prequant_val_bpb": res.prequant_val_bpb, "code_bytes": res.code_bytes, "budget_ok": res.budget_ok, "peak_mem_mib": res.peak_mem_mib,
                "model_params": gpt.count_params(m), "bank_shapes": {k: list(gpt.param_shapes(m)[k]) for k in gpt.BANKS},
                "layer_schedule": gpt.layer_schedule(m), "xsa_layers": m.xsa_layers(), "parallel_residual": m.parallel,
                "torch": torch.__version__, "cuda": torch.version.cuda, "spec": spec.to_dict()}), default=str, allow_nan=False))
        return res


# The reference trainer's command-line flags (pg-train/src/main.rs:58-122) and the spec keys they set. Every one of them can
# also be given as a ``section.key=value`` override; the flags are for scripts written against that binary.
REFERENCE_FLAGS = {
    "--train-data": "train.train_data_pattern", "--val-data": "train.validation_data_pattern", "--rank": "train.rank",
    "--world-size": "train.world_size", "--batch-tokens": "train.batch_tokens", "--seq-len": "train.seq_len",
    "--total-iterations": "train.total_iterations", "--max-steps": "train.total_iterations",
    "--max-wallclock-seconds": "train.max_wallclock_seconds", "--min-lr-scale": "train.min_lr_scale",
    "--tokenizer-vocab": "eval.tokenizer_vocab_path", "--caseops-byte-sidecar": "eval.caseops_byte_sidecar_pattern",
    "--eval-max-tokens": "eval.max_tokens", "--eval-stride": "eval.stride", "--distributed-optimizer": "train.distributed_optimizer_backend",
    "--eval-adaptation": "eval.adaptation_backend", "--attn-out-gate-width": "model.attn_out_gate.width", "--quant-scheme": "quant.scheme",
    "--prune-keep-ratio": "quant.prune_keep_ratio",
}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="parameter_golf_b200.train")
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("keys", help="list every spec key (type, default) and the train_gpt.py environment names that map onto them")
    for name in ("run", "sweep", "plan", "preflight", "spec"):
        sp = sub.add_parser(name)
        sp.add_argument("--spec")
        sp.add_argument("--family", "--builtin", dest="family", default=None)
        for flag, key in REFERENCE_FLAGS.items():
            sp.add_argument(flag, dest="ref_" + key.replace(".", "__"), default=None, help=f"sets {key}")
        sp.add_argument("--attn-out-gate", action="store_true", help="sets model.attn_out_gate.enabled=true")
        sp.add_argument("--allow-unsupported-variants", action="store_true")
        sp.add_argument("--attention-backend", default=None, help="accepted for compatibility: there is one attention path")
        sp.add_argument("--fast-bank-updates", action="store_true", help="accepted for compatibility: bank updates are always fused")
        sp.add_argument("--families", default="tiny_cpu")
        sp.add_argument("--mode", default=None)
        sp.add_argument("--arch", default=None, help="one of the sweep architectures (spec.ARCH_VARIANTS) instead of a family")
        sp.add_argument("--log-dir", default=None, help="also write the run log to <dir>/<run name>.txt (or set PGB_LOG_DIR)")
        sp.add_argument("--env", action="store_true", help="overlay train_gpt.py environment variable names")
        sp.add_argument("--backend", default=None)
        sp.add_argument("--artifact", default=None)
        sp.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    if a.cmd == "keys":
        spec = RunSpec()
        by_key: dict = {}
        for env_name, keys in RunSpec.env_names().items():
            for k in keys:
                by_key.setdefault(k, []).append(env_name)
        flags = {v: k for k, v in REFERENCE_FLAGS.items()}
        for key, tname, default in spec.describe_keys():
            extra = "".join(f"  env {n}" for n in by_key.get(key, [])) + (f"  flag {flags[key]}" if key in flags else "")
            print(f"{key} ({tname}) = {default!r}{extra}")
        return 0
    fams = [a.family] if (a.cmd != "sweep" and a.family) else ([None] if a.cmd != "sweep" else a.families.split(","))
    rc = 0
    for fam in fams:
        if a.arch:
            from .spec import arch_variant
            spec = arch_variant(a.arch)
        else:
            spec = RunSpec.load(a.spec) if a.spec else family_preset(fam or "tiny_cpu")
        if a.env:
            spec.apply_env()
        if "RANK" in os.environ:
            spec.train.rank, spec.train.world_size = int(os.environ["RANK"]), int(os.environ.get("WORLD_SIZE", 1))
        if a.backend:
            spec.train.backend = a.backend
        if a.artifact:
            spec.train.artifact_path = a.artifact
        ref = [f"{k[4:].replace('__', '.')}={v}" for k, v in vars(a).items() if k.startswith("ref_") and v is not None]
        if a.attn_out_gate:
            ref.append("model.attn_out_gate.enabled=true")
        if a.attention_backend and a.attention_backend.replace("-", "_") in ("native", "naive_f32", "flash_f32", "cudnn_sdpa_bf16"):
            # recorded in the spec (and so in its fingerprint), never dispatched on; other spellings are ignored, as the reference's
            # parser does (pg-train/src/main.rs:981-988)
            ref.append(f"model.attention_backend={a.attention_backend.replace('-', '_')}")
        if a.fast_bank_updates:
            ref.append("train.fast_bank_updates=true")
        spec.apply_overrides(ref)
        if any(o.startswith("train.seq_len=") for o in ref):          # the binary's --seq-len sets the model's lengths too
            spec.model.train_seq_len = spec.model.eval_seq_len = spec.train.seq_len
        if a.allow_unsupported_variants:
            spec.allow_unsupported_variants = True
        spec.apply_overrides(a.overrides)
        if a.mode:
            spec.mode = a.mode
        if spec.train.world_size > 1 and a.cmd not in ("plan", "preflight", "spec"):
            import torch.distributed as dist
            if not dist.is_initialized():
                dist.init_process_group("gloo" if spec.train.backend == "cpu" else "nccl")
        if a.cmd == "spec":              # the resolved spec as a TOML file: every key, after the family, file, environment and overrides
            spec.validate()
            print(spec.to_toml(), end="")
            continue
        if a.cmd == "preflight":         # everything that can be checked about a planned run without a device
            lines, ok = preflight(spec)
            print("\n".join(lines))
            rc |= 0 if ok else 1
            continue
        if a.cmd == "plan":              # print the execution plan (layout, block schedule, memory estimate) and stop
            from .plan import ExecutionPlan
            print("\n".join(ExecutionPlan.from_run_spec(spec).summary_lines()))
            continue
        log_dir = a.log_dir or os.environ.get("PGB_LOG_DIR")
        run_log = RunLog(spec.name, directory=log_dir, rank=spec.train.rank)
        if run_log.path:
            # the file starts with what produced the run, as the Python trainer's log starts with its source and the GPU list
            # (train_gpt.py:777-794): here the resolved spec and the environment summary
            from .doctor import collect
            env = collect()
            head = ["=" * 100, spec.to_toml().rstrip(), "=" * 100] + [f"{k}={v}" for k, v in env.items() if k != "gpus"]
            head += [f"gpu{g['index']}={g['name']} sm_{g['capability'].replace('.', '')} {g['memory_gib']}GiB" for g in env["gpus"]] + ["=" * 100]
            with open(run_log.path, "a", encoding="utf-8") as f:
                f.write("\n".join(head) + "\n")
        res = VariantRunner(spec, run_log).run()
        if spec.train.rank == 0:
            print("\n".join(res.key_value_lines()))
            if run_log.path:
                with open(run_log.path, "a", encoding="utf-8") as f:
                    f.write("\n".join(res.key_value_lines()) + "\n")
        rc |= 0 if (res.budget_ok or spec.mode != "record") else 1
    return rc


if __name__ == "__main__":
    sys.exit(main())
