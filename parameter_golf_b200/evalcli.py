"""Evaluation entry point: ``python -m parameter_golf_b200.evalcli --artifact a.pgrs [--spec s.toml | --family f] [--leaderboard] …``.

Flow (``parameter-golf-rs/crates/pg-eval/src/bin/run.rs:6-214``): flags → spec → leaderboard-mode validation → artifact + code byte
budget → load artifact into a fresh model → validation tokens → byte counts (SentencePiece LUT | seeded table | placeholder)
→ dispatch (sliding | score-first TTT variants | LoRA phased) → timing and one ``eval_audit_json=`` line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

from .data.bpb import BpbLuts
from .data.shards import load_validation_tokens
from .eval.sliding import eval_sliding
from .eval.ttt import eval_lora_phased_ttt, eval_score_first_ttt
from .quant.export import check_budget, code_bytes, load_artifact
from .spec import RunSpec, family_preset


def leaderboard_violations(spec: RunSpec, args) -> list:
    """Fail-closed rules for a leaderboard evaluation (``run.rs:238-306``)."""
    bad = []
    if spec.eval.max_tokens is not None:
        bad.append("leaderboard evaluation must cover the full validation set (eval.max_tokens is set)")
    if spec.eval.adaptation_backend != "none" and not spec.eval.legal_score_first:
        bad.append("test-time adaptation must be score-first")
    if not spec.eval.legal_score_first:
        bad.append("leaderboard evaluation requires eval.legal_score_first=true")
    if (spec.eval.adaptation_backend == "gpu_lora_phased" and spec.eval.phased_ttt_prefix_docs > 0
            and spec.model.smear_gate_boundary_token_id is None):
        bad.append("prefix-document TTT needs the document boundary token (model.smear_gate_boundary_token_id)")
    if spec.eval.adaptation_backend == "gpu_lora_phased" and int(os.environ.get("WORLD_SIZE", 1)) < max(spec.train.world_size, 1):
        bad.append("leaderboard LoRA-phased evaluation runs on the configured world size, not on fewer ranks")
    if spec.model.caseops.enabled and spec.model.caseops.byte_sidecar:
        if not spec.eval.caseops_byte_sidecar_pattern:
            bad.append("leaderboard evaluation with CaseOps needs --caseops-byte-sidecar")
    elif args.bytes == "tokenizer" and not spec.eval.tokenizer_vocab_path:
        bad.append("leaderboard evaluation with --bytes tokenizer needs --tokenizer-vocab")
    # (--bytes seeded, the fixed 1-6 byte table that stands in for a tokenizer on synthetic data, is accepted; the reference
    # insists on a tokenizer here, pg-eval/src/bin/run.rs:296-301)
    if args.bytes == "placeholder":
        bad.append("leaderboard evaluation needs real byte counts, not the 4-bytes-per-token placeholder")
    if not args.val_pattern:
        bad.append("leaderboard evaluation needs --val-pattern")
    return bad


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="parameter_golf_b200.evalcli")
    ap.add_argument("--artifact", required=True)
    ap.add_argument("--spec")
    ap.add_argument("--family", "--builtin", dest="family", default="record_11l")
    ap.add_argument("--val-pattern", "--val-data", dest="val_pattern", help="validation shards (default: the spec's train.validation_data_pattern)")
    # the reference binary's flag names (pg-eval/src/bin/run.rs:19-27); each one overrides the spec key it names
    ap.add_argument("--stride", type=int)
    ap.add_argument("--tokenizer-vocab")
    ap.add_argument("--caseops-byte-sidecar")
    ap.add_argument("--find-temperature", action="store_true",
                    help="pick eval.temperature from eval.temperature_grid on the first training tokens before scoring (autograd runner)")
    ap.add_argument("--bytes", choices=["tokenizer", "seeded", "placeholder"], default="seeded")
    ap.add_argument("--leaderboard", action="store_true")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--max-tokens", type=int)
    ap.add_argument("overrides", nargs="*")
    a = ap.parse_args(argv)
    spec = RunSpec.load(a.spec) if a.spec else family_preset(a.family)
    spec.apply_overrides(a.overrides)
    if a.max_tokens is not None:
        spec.eval.max_tokens = a.max_tokens
    if a.stride is not None:
        spec.eval.stride = a.stride
    if a.tokenizer_vocab:
        spec.eval.tokenizer_vocab_path = a.tokenizer_vocab
        if a.bytes == "seeded":
            a.bytes = "tokenizer"              # a tokenizer given on the command line is meant to be used
    if a.caseops_byte_sidecar:
        spec.eval.caseops_byte_sidecar_pattern = a.caseops_byte_sidecar
    if not a.val_pattern:
        a.val_pattern = spec.train.validation_data_pattern
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if a.device == "cuda":                        # one process per GPU: each rank evaluates on its own device
        import torch
        a.device = f"cuda:{int(os.environ.get('LOCAL_RANK', 0))}"
        torch.cuda.set_device(a.device)
    if world > 1:
        import torch
        import torch.distributed as dist
        if a.device == "cpu":
            dist.init_process_group("gloo")
        else:
            dist.init_process_group("nccl", device_id=torch.device(a.device))
    if a.leaderboard:
        bad = leaderboard_violations(spec, a)
        if bad:
            print("leaderboard validation failed: " + "; ".join(bad), file=sys.stderr)
            return 2
    blob = open(a.artifact, "rb").read()
    cb = code_bytes()
    ok = check_budget(len(blob), cb, spec.quant.target_artifact_bytes)
    print(f"artifact_bytes={len(blob)}\ncode_bytes={cb}\nbudget_ok={ok}")
    if a.leaderboard and not ok:
        return 3
    m = spec.model
    params = load_artifact(blob, spec)
    if not a.val_pattern:
        raise SystemExit("--val-pattern (or train.validation_data_pattern in the spec) is required")
    val = load_validation_tokens(a.val_pattern, m.eval_seq_len, spec.eval.max_tokens)
    luts = {"tokenizer": lambda: BpbLuts.from_sentencepiece(spec.eval.tokenizer_vocab_path, m.vocab_size),
            "seeded": lambda: BpbLuts.seeded(m.vocab_size, spec.eval.byte_table_seed),
            "placeholder": lambda: BpbLuts.placeholder(m.vocab_size)}[a.bytes]()
    if spec.eval.caseops_byte_sidecar_pattern:     # byte counts per validation position instead of per token surface
        from .data.shards import load_validation_byte_sidecar
        side = load_validation_byte_sidecar(spec.eval.caseops_byte_sidecar_pattern)
        if side.shape[0] < val.shape[0]:
            raise SystemExit(f"byte sidecar has {side.shape[0]} entries, the validation split {val.shape[0]} tokens")
        luts = luts.with_sidecar(side[: val.shape[0]])
    if a.device == "cpu":
        from .models.runner import OracleRunner
        runner = OracleRunner(m.for_evaluation(spec.eval.depth_recurrence), params)
        runner.temperature = spec.eval.temperature
        if a.find_temperature:
            from .eval.sliding import find_temperature
            if not spec.train.train_data_pattern:
                raise SystemExit("--find-temperature needs train.train_data_pattern (the grid is scored on training tokens)")
            calib = load_validation_tokens(spec.train.train_data_pattern, m.eval_seq_len, spec.eval.temperature_calibration_tokens)
            best, table = find_temperature(runner, calib, m.eval_seq_len, spec.eval.temperature_grid)
            if rank == 0:
                print("temperature_search=" + json.dumps({str(k): round(v, 6) for k, v in table.items()}) + f"\ntemperature={best}")
    else:
        if spec.eval.temperature != 1.0 or a.find_temperature:
            raise SystemExit("temperature scaling is scored by the autograd runner: use --device cpu")
        from .models.engine import EngineRunner
        runner = EngineRunner(spec, params, a.device)
    t0 = time.perf_counter()
    ab = spec.eval.adaptation_backend
    if spec.eval.legal_score_first and ab in ("full_sgd", "cpu_q_only", "lact"):
        mode = {"full_sgd": "full_sgd", "cpu_q_only": "q_only", "lact": "lact"}[ab]
        hook = None
        if world > 1 and a.device != "cpu":       # packed gradient all-reduce on the peer-memory kernels instead of NCCL
            from .models import gpt
            from .parallel.peer_allreduce import PeerAllReduce
            hook = PeerAllReduce(gpt.count_params(m) + 64).mean_
        loss, bpb = eval_score_first_ttt(runner, val, m, spec.eval, luts, rank, world, mode, a.device, print, all_reduce=hook)
        kind = f"score_first_{mode}"
    elif spec.eval.legal_score_first and ab == "gpu_lora_phased":
        hook = None
        if world > 1 and a.device != "cpu":       # packed adapter-gradient all-reduce on the peer-memory kernels
            from .parallel.peer_allreduce import PeerAllReduce
            hook = PeerAllReduce(2 * m.num_layers * m.model_dim * spec.eval.lora_rank + 64).mean_
        loss, bpb = eval_lora_phased_ttt(runner, val, m, spec.eval, luts, rank, world, a.device, print, all_reduce=hook)
        kind = "lora_phased"
    elif spec.eval.legal_score_first and ab == "doc_lora":
        from .eval.doc_lora import eval_doc_lora_ttt
        hook = None
        if world > 1:
            import torch.distributed as dist

            def hook(t):           # three float64 sums: the process group's own all-reduce (gloo on cpu)
                dev_t = t.to(a.device) if a.device != "cpu" else t
                dist.all_reduce(dev_t)
                t.copy_(dev_t.cpu())
        loss, bpb = eval_doc_lora_ttt(runner.params, m, val, spec.eval, luts, rank, world, a.device, print, all_reduce=hook,
                                      betas=(spec.train.adam_beta1, spec.train.adam_beta2))
        kind = "doc_lora"
    else:
        loss, bpb = eval_sliding(runner.nll, val, m.eval_seq_len, spec.eval.stride, luts, rank, world, spec.eval.batch_windows, a.device)
        kind = "sliding"
    ms = 1000.0 * (time.perf_counter() - t0)
    if rank == 0:
        print(f"val_loss={loss}\nval_bpb={bpb}\neval_ms={ms:.1f}\neval_kind={kind}")
        # the same facts under the names the reference evaluator prints (pg-eval/src/bin/run.rs:96-214)
        print(f"eval_loss={loss}\neval_bpb={bpb}\neval_wallclock_seconds={ms / 1000.0:.3f}\neval_max_wallclock_seconds={spec.eval.max_eval_seconds}\n"
              f"eval_status={'ok' if ms / 1000.0 <= spec.eval.max_eval_seconds or spec.eval.max_eval_seconds <= 0 else 'over_budget'}\n"
              f"eval_stride={spec.eval.stride}\neval_tokens={int(val.shape[0] - 1)}\neval_gpu_world_size={world if a.device != 'cpu' else 0}\n"
              f"legal_score_first={str(spec.eval.legal_score_first).lower()}\nqttt={str(spec.eval.qttt).lower()}\nlora_rank={spec.eval.lora_rank}\n"
              f"lora_alpha={spec.eval.lora_alpha}\nphased_ttt_phases={spec.eval.phased_ttt_phases}\nvariant_fingerprint={spec.fingerprint():016x}\n"
              f"submission_code_bytes={cb}\nsubmission_total_bytes={cb + len(blob)}")
        print("eval_audit_json=" + json.dumps({"artifact": a.artifact, "artifact_bytes": len(blob), "eval_kind": kind, "stride": spec.eval.stride,
                                               "window": m.eval_seq_len, "tokens": int(val.shape[0] - 1), "world_size": world, "bytes": a.bytes,
                                               "fingerprint": f"{spec.fingerprint():016x}", "eval_ms": round(ms, 1),
                                               "within_budget_s": ms / 1000.0 <= spec.eval.max_eval_seconds}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
