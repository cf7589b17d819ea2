"""Post-training export and evaluation of the 11-layer record model on one or more GPUs, stage by stage.

    python bench/export_eval_bench.py [--calib-seqs 64] [--eval-tokens 2097152] [--ttt-chunks 4]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench/export_eval_bench.py ...

Stages (random-init weights, synthetic Zipf/Markov validation tokens, seeded 1-6 byte table):
  1. calibration: ``--calib-seqs`` x 2048 tokens generated autoregressively by the model at temperature 0.8, then the
     Hessians of every linear input;
  2. full-Hessian GPTQ int6 of every bank matrix with the CUDA row kernel, bit packing, zstd level 22 -> artifact bytes;
  3. artifact load + sliding-window evaluation (stride 64, window 2048) of ``--eval-tokens`` held-out tokens on the CUDA
     engine, windows split over ranks; reports tokens/s and the time the full 62 M-token evaluation would take at that
     rate on this many GPUs;
  4. score-first test-time training: ``--ttt-chunks`` chunks of 32,768 tokens, each scored first and then trained on for
     one SGD epoch; reports seconds per chunk and the projection for 1,893 chunks.

The reference's envelope for stages 3 and 4 is 74 s and 410 s on 8 x H100
(records/track_10min_16mb/2026-03-23_LeakyReLU_LegalTTT_ParallelMuon/train_seed1337.log:77, :274).
"""
import argparse
import json
import os
import sys
import tempfile
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--calib-seqs", type=int, default=64)
    ap.add_argument("--eval-tokens", type=int, default=1 << 21)
    ap.add_argument("--ttt-chunks", type=int, default=4)
    ap.add_argument("--skip-export", action="store_true")
    a = ap.parse_args()
    import torch.distributed as dist
    from parameter_golf_b200.data.bpb import BpbLuts
    from parameter_golf_b200.data.shards import generate_markov_tokens
    from parameter_golf_b200.eval.sliding import eval_sliding
    from parameter_golf_b200.eval.ttt import eval_score_first_ttt
    from parameter_golf_b200.models import gpt
    from parameter_golf_b200.models.engine import EngineRunner
    from parameter_golf_b200.ops import native
    from parameter_golf_b200.quant.calibrate import self_generated_hessians
    from parameter_golf_b200.quant.export import export_model, load_artifact
    from parameter_golf_b200.quant.gptq import gptq_quantize_model
    from parameter_golf_b200.spec import family_preset

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    dev = f"cuda:{torch.cuda.current_device()}"
    spec = family_preset("record_11l")
    spec.quant.scheme = "full_gptq_int6"
    spec.quant.calibration = "self_generated"
    spec.eval.legal_score_first = True
    spec.eval.adaptation_backend = "full_sgd"
    spec.eval.ttt_epochs = 1
    m = spec.model
    params = gpt.init_params(m, seed=1337)
    out = {"bench": "export_eval", "gpus": world}

    def tick():
        torch.cuda.synchronize()
        return time.perf_counter()

    path = os.path.join(tempfile.gettempdir(), "pgb200_export_eval.bin")
    if not a.skip_export and rank == 0:
        l0 = native.launch_count()
        t0 = tick()
        hess = self_generated_hessians(spec, params, device=dev, num_seqs=a.calib_seqs, seq_len=m.train_seq_len)
        t1 = tick()
        pre = gptq_quantize_model(spec, params, hess, device=dev)
        t2 = tick()
        blob = export_model(spec, params, path, pre)
        t3 = tick()
        out.update({"calibration_s": round(t1 - t0, 2), "gptq_s": round(t2 - t1, 2), "pack_compress_s": round(t3 - t2, 2),
                    "artifact_bytes": len(blob), "within_16MB": len(blob) <= 16_000_000, "gptq_kernel_launches": native.launch_count() - l0})
        print(f"[export] calibration {t1 - t0:.1f}s  gptq {t2 - t1:.1f}s  pack+zstd {t3 - t2:.1f}s  artifact {len(blob)} bytes", flush=True)
    if world > 1:
        dist.barrier()
    if os.path.exists(path):
        params = load_artifact(open(path, "rb").read(), spec)
    val = generate_markov_tokens(a.eval_tokens + 1, m.vocab_size, seed=99991)
    luts = BpbLuts.seeded(m.vocab_size, spec.eval.byte_table_seed)
    runner = EngineRunner(spec, params, dev)
    eval_sliding(runner.nll, val[: 64 * m.eval_seq_len + 1], m.eval_seq_len, spec.eval.stride, luts, rank, world, spec.eval.batch_windows, dev)   # warm-up
    t0 = tick()
    loss, bpb = eval_sliding(runner.nll, val, m.eval_seq_len, spec.eval.stride, luts, rank, world, spec.eval.batch_windows, dev)
    t1 = tick()
    rate = a.eval_tokens / (t1 - t0)
    out.update({"sliding_tokens": a.eval_tokens, "sliding_s": round(t1 - t0, 2), "sliding_scored_tokens_per_s": round(rate), "val_loss": loss, "val_bpb": bpb,
                "sliding_62M_projection_s": round(62e6 / rate, 1)})
    if rank == 0:
        print(f"[sliding] {a.eval_tokens} tokens in {t1 - t0:.2f}s -> {rate / 1e6:.2f} M scored tokens/s; 62 M tokens would take {62e6 / rate:.1f}s on {world} GPU(s)", flush=True)
    if a.ttt_chunks > 0:
        n_tok = a.ttt_chunks * spec.eval.chunk_tokens
        t0 = tick()
        par = None
        if world > 1:          # packed gradient all-reduce on the peer-memory kernels instead of NCCL
            from parameter_golf_b200.parallel.peer_allreduce import PeerAllReduce
            par = PeerAllReduce(gpt.count_params(m) + 64)
        loss, bpb = eval_score_first_ttt(runner, val[: n_tok + 1], m, spec.eval, luts, rank, world, "full_sgd", dev, (print if rank == 0 else (lambda *x: None)),
                                         all_reduce=(par.mean_ if par is not None else None))
        t1 = tick()
        per = (t1 - t0) / a.ttt_chunks
        out.update({"ttt_chunks": a.ttt_chunks, "ttt_s_per_chunk": round(per, 3), "ttt_1893_chunks_projection_s": round(per * 1893, 1), "ttt_val_loss": loss})
        if rank == 0:
            print(f"[ttt] {a.ttt_chunks} chunks of {spec.eval.chunk_tokens} tokens: {per:.2f}s per chunk; 1,893 chunks would take {per * 1893:.0f}s on {world} GPU(s)", flush=True)
    native.check_status()
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
