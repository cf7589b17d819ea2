#!/usr/bin/env python
"""Headline benchmark: training throughput (tokens/s, ms/step) of the 11-layer record-style GPT.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched once per rank by torch.distributed.run)
    python bench.py --impl reference --gpus N --steps K --warmup W

Config: 11 layers, d_model 512, 8 query / 4 KV heads, MLP 3x LeakyReLU(0.5)^2, XSA on the last 4 layers, partial RoPE
16/64, layer-wise LN scale, BigramHash 3072x128, SmearGate, tied vocab-1024 embeddings, seq_len 2048, 786,432 tokens per
optimizer step, Parallel Muon (lr 0.025, wd 0.04) + AdamW, EMA 0.997, bf16 compute. Each rank runs 8/N micro-batches of
48 x 2048 tokens per step (the reference's rule), so the global batch is the same at every N: strong scaling.
Data: synthetic seeded Zipf(1.1) order-1 Markov uint16 shards; weights: random init.

The native arm prints two numbers: `value` is timed on the device with CUDA events over K steps whose token spans are
already resident on the GPU; `e2e` runs the same K steps through the public `EngineBackend.train_step_spans` call with
every micro-batch copied from pinned host memory and the step loss read back to the host.
The reference arm runs the unmodified 2026-03-23 record script installed under baseline/_ref through its own main().
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

VOCAB = 1024
# name -> (spec family, tokens per step, seq_len, published tokens/s on 8xH100, description)
CONFIGS = {
    "record_11l": ("record_11l", 786_432, 2048, 786_432 / 0.0834,
                   "record_11l (11L d512 8H/4KV MLP3x LeakyReLU^2 XSA4 RoPE16 BigramHash3072x128 SmearGate tied-1024)"),
    "baseline_9l": ("baseline_9l", 524_288, 1024, 524_288 / 0.04354,
                    "baseline_9l (9L d512 8H/4KV MLP2x relu^2 full RoPE tied-1024 softcap 30)"),
}
PUBLISHED_TOKENS_PER_S = CONFIGS["record_11l"][3]
GLOBAL_BATCH, SEQ_LEN = 786_432, 2048


def select_config(name: str):
    global GLOBAL_BATCH, SEQ_LEN, PUBLISHED_TOKENS_PER_S
    _, GLOBAL_BATCH, SEQ_LEN, PUBLISHED_TOKENS_PER_S, _ = CONFIGS[name]


class ClockSampler:
    """Samples SM clocks and clock-event (throttle) reasons of one GPU while the timed region runs: an NVML reader thread
    every 20 ms (a timed region of a few steps on 8 GPUs lasts a fraction of a second), or, when the NVML binding is
    missing, an ``nvidia-smi -lms 200`` child process. Read-only queries; no setting of the GPU is touched."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None
        self.thread = None
        self.samples = []          # (sm MHz, reason bitmask)
        self.sm_max = None
        self._stop = False

    def _nvml_loop(self, nv, handle):
        while not self._stop:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)
                try:
                    bits = nv.nvmlDeviceGetCurrentClocksEventReasons(handle)
                except Exception:
                    bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.samples.append((float(mhz), int(bits)))
            except Exception:
                pass
            time.sleep(0.02)

    def start(self):
        try:
            import threading
            import pynvml as nv
            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = int(visible.split(",")[self.gpu]) if visible and all(x.strip().isdigit() for x in visible.split(",")) else self.gpu
            handle = nv.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu)],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread is not None:
            self._stop = True
            self.thread.join(timeout=2)
            if self.samples:
                bits = 0
                for _, b in self.samples:
                    bits |= b
                out.update(sm_mhz=statistics.median(m for m, _ in self.samples), sm_max_mhz=self.sm_max,
                           reasons=sorted(k for k, v in self.REASON_BITS.items() if bits & v), samples=len(self.samples), source="nvml")
            return out
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm), source="nvidia-smi")
        return out


def ensure_data(root: str):
    from parameter_golf_b200.data.shards import write_synthetic_dataset
    return write_synthetic_dataset(root, VOCAB, train_tokens=1 << 24, val_tokens=64 * SEQ_LEN + 1, train_shards=1, seed=1337)


def run_native(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from parameter_golf_b200.data.native_loader import NativeTokenLoader
    from parameter_golf_b200.models import gpt
    from parameter_golf_b200.models.engine import EngineBackend
    from parameter_golf_b200.ops import native
    from parameter_golf_b200.optim.muon import muon_momentum_at
    from parameter_golf_b200.spec import family_preset

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    spec = family_preset(CONFIGS[args.config][0])
    spec.mode = "record_shaped_proxy"
    spec.train.rank, spec.train.world_size = rank, world
    spec.train.backend = "cuda_distributed" if world > 1 else "cuda_single"
    spec.train.cuda_graph = bool(args.cuda_graph)
    spec.validate()
    data_root = os.path.join(tempfile.gettempdir(), "pgb200_bench_data")
    if rank == 0:
        ensure_data(data_root)
    if world > 1:
        dist.barrier()
    accum = 8 // world
    params = gpt.init_params(spec.model, seed=1337)
    backend = EngineBackend(spec, params)
    T = backend.engine.T
    assert T * accum * world == GLOBAL_BATCH and backend.accum == accum
    # C++ loader: a worker thread reads the mmap'd shards ahead into a ring of page-locked buffers; one optimizer step's
    # spans stay valid until the next step asks for its first one
    loader = NativeTokenLoader(os.path.join(data_root, "fineweb_train_*.bin"), rank, world)
    loader.start_prefetch(GLOBAL_BATCH, accum)
    assert loader.pinned

    def next_spans():
        return [loader.next_prefetched() for _ in range(accum)]

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    step = 0
    for _ in range(args.warmup):
        backend.train_step_spans(next_spans(), 1.0, muon_momentum_at(step, 0.92, 0.99, 1500))
        step += 1
    # ---- device-timed region: spans already resident on the GPU ----------------------------------------------------
    staged = []
    for _ in range(args.steps):
        staged.append([s.to("cuda") for s in next_spans()])
    sync_all()
    sampler = ClockSampler(local_rank)
    sampler.start()
    l0 = native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for k in range(args.steps):
        backend.train_step_spans(staged[k], 1.0, muon_momentum_at(step + k, 0.92, 0.99, 1500), read_loss=False, staged=True)
    e1.record()
    sync_all()
    dev_ms = e0.elapsed_time(e1) / args.steps
    launches = native.launch_count() - l0
    step += args.steps
    # ---- end-to-end region: pinned host -> device every micro-batch, loss read back every step --------------------------
    sync_all()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    last_loss = None
    for k in range(args.steps):
        last_loss = backend.train_step_spans(next_spans(), 1.0, muon_momentum_at(step + k, 0.92, 0.99, 1500), read_loss=True)
    e3.record()
    sync_all()
    e2e_ms = e2.elapsed_time(e3) / args.steps
    clocks = sampler.stop()
    native.check_status()
    loader.stop_prefetch()
    t = torch.tensor([dev_ms, e2e_ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = t.tolist()
    if rank == 0:
        value = GLOBAL_BATCH / (dev_ms / 1000.0)
        print(json.dumps({
            "metric": "train_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": value / PUBLISHED_TOKENS_PER_S,
            "dtype": "bf16", "data": "synthetic seeded Zipf(1.1) order-1 Markov uint16 shards; random-init weights",
            "impl": "native",
            "config": {"model": CONFIGS[args.config][4],
                       "global_batch": GLOBAL_BATCH, "seq_len": SEQ_LEN,
                       "parallelism": f"dp{world}" + ((" sharded Parallel Muon" if backend.dist is not None and backend.dist.sharded else " peer-memory gradient all-reduce") if world > 1 else ""),
                       "grad_accum": accum, "micro_batch_tokens": T,
                       "optimizer": f"Muon {spec.train.muon_ns_profile} NS{spec.train.muon_ns_steps} + AdamW" + (f" + EMA {spec.train.ema_decay}" if spec.train.ema_decay > 0 else ""),
                       "l2": "inputs_larger_than_L2 (gigabytes of saved activations per micro-batch; no flush needed)"},
            "clocks": clocks,
            "e2e": {"value": GLOBAL_BATCH / (e2e_ms / 1000.0), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": accum * (T + 1) * 2 + 32, "d2h_bytes_per_step": 20, "last_loss": last_loss},
            "gpu_launches": launches,
        }))
    if world > 1:
        dist.destroy_process_group()


class _BenchDone(Exception):
    pass


def run_reference(args):
    """The unmodified record script, driven through its own environment-variable interface and main()."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    record = args.config == "record_11l"
    script = os.path.join(ref_root, "parameter_golf_reference", "train_gpt_record_2026_03_23.py" if record else "train_gpt_root.py")
    rank = int(os.environ.get("RANK", "0"))

    def unavailable(why):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    if not os.path.exists(script):
        return unavailable("baseline/_ref does not hold the reference install (pip install --target baseline/_ref was not run)")
    try:
        import sentencepiece as spm
        import torch
    except Exception as e:           # pragma: no cover
        return unavailable(f"missing dependency: {e}")
    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    data_root = os.path.join(tempfile.gettempdir(), "pgb200_bench_data")
    tok = os.path.join(data_root, "synthetic_1024_bpe.model")
    done_flag = os.path.join(data_root, ".ref_ready")
    if rank == 0:
        ensure_data(data_root)
        if not os.path.exists(tok):
            import random
            rng = random.Random(0)
            syll = ["".join(rng.choice("abcdefghijklmnopqrstuvwxyz") for _ in range(rng.randint(1, 4))) for _ in range(6000)]
            corpus = os.path.join(data_root, "corpus.txt")
            with open(corpus, "w") as f:
                for _ in range(20000):
                    f.write(" ".join(rng.choice(syll) + rng.choice(syll) for _ in range(12)) + "\n")
            spm.SentencePieceTrainer.train(input=corpus, model_prefix=tok[:-6], vocab_size=VOCAB, model_type="bpe", character_coverage=1.0,
                                           minloglevel=2)
        open(done_flag, "w").write("ok")
    else:
        t0 = time.time()
        while not os.path.exists(done_flag) and time.time() - t0 < 600:
            time.sleep(0.5)
    run_id = f"bench_ref_{args.config}_n{world}"
    workdir = os.path.join(tempfile.gettempdir(), f"pgb200_ref_run_{args.config}_{world}")
    os.makedirs(workdir, exist_ok=True)
    os.chdir(workdir)
    env = {"DATA_PATH": data_root, "TOKENIZER_PATH": tok, "RUN_ID": run_id, "ITERATIONS": str(args.steps), "WARMUP_STEPS": str(args.warmup),
           "WARMDOWN_ITERS": "0", "MAX_WALLCLOCK_SECONDS": "0", "VAL_LOSS_EVERY": "0", "TRAIN_LOG_EVERY": str(max(args.steps, 1)),
           "TRAIN_BATCH_TOKENS": str(GLOBAL_BATCH), "TRAIN_SEQ_LEN": str(SEQ_LEN), "EVAL_SEQ_LEN": str(SEQ_LEN), "VOCAB_SIZE": str(VOCAB),
           "NUM_LAYERS": "11", "MODEL_DIM": "512", "NUM_HEADS": "8", "NUM_KV_HEADS": "4", "MLP_MULT": "3.0", "BIGRAM_VOCAB_SIZE": "3072",
           "BIGRAM_DIM": "128", "XSA_LAST_N": "4", "ROPE_DIMS": "16", "LN_SCALE": "1", "VE_ENABLED": "0", "MATRIX_LR": "0.025", "MUON_WD": "0.04",
           "ADAM_WD": "0.04", "SWA_ENABLED": "0", "QAT_ENABLED": "0", "LATE_QAT_THRESHOLD": "0", "TTT_ENABLED": "0", "SEED": "1337"}
    if not record:       # the root trainer: 9 layers, MLP 2x relu^2, its own defaults for everything it does not know
        env = {k: v for k, v in env.items() if k in ("DATA_PATH", "TOKENIZER_PATH", "RUN_ID", "ITERATIONS", "WARMUP_STEPS", "WARMDOWN_ITERS",
                                                     "MAX_WALLCLOCK_SECONDS", "VAL_LOSS_EVERY", "TRAIN_LOG_EVERY", "TRAIN_BATCH_TOKENS", "TRAIN_SEQ_LEN",
                                                     "VOCAB_SIZE", "MODEL_DIM", "NUM_HEADS", "NUM_KV_HEADS", "SEED")}
        env.update({"NUM_LAYERS": "9", "MLP_MULT": "2", "VAL_BATCH_SIZE": str(GLOBAL_BATCH)})
    os.environ.update(env)
    sys.path.insert(0, os.path.join(ROOT, "baseline", "fa3_shim"))      # flash_attn_interface -> torch SDPA (FA3 is Hopper-only)
    sys.path.insert(0, ref_root)
    orig_mem = torch.cuda.max_memory_allocated

    def stop_after_training(*a, **k):
        # the script's first own call of this function is the "peak memory" log line right after its training loop;
        # calls from inside torch (compiler, allocator statistics) pass through
        if os.path.abspath(sys._getframe(1).f_code.co_filename) == os.path.abspath(script):
            raise _BenchDone()
        return orig_mem(*a, **k)

    sampler = ClockSampler(local_rank)
    sampler.start()
    import runpy
    torch.cuda.max_memory_allocated = stop_after_training        # first call after the training loop, on every rank
    t_wall = time.time()
    try:
        runpy.run_path(script, run_name="__main__")
    except _BenchDone:
        pass
    except Exception as e:
        torch.cuda.max_memory_allocated = orig_mem
        sampler.stop()
        return unavailable(f"reference run failed: {type(e).__name__}: {str(e)[:200]}")
    finally:
        torch.cuda.max_memory_allocated = orig_mem
    clocks = sampler.stop()
    import torch.distributed as dist
    if dist.is_initialized():
        dist.barrier()
    if rank == 0:
        ms = None
        for line in open(os.path.join(workdir, "logs", f"{run_id}.txt")):
            if line.startswith(f"step:{args.steps}/{args.steps} val_loss"):
                ms = float(line.split("train_time:")[1].split("ms")[0]) / args.steps
        if ms is None:
            print(json.dumps({"impl": "reference", "unavailable": "reference log has no final step line"}))
        else:
            value = GLOBAL_BATCH / (ms / 1000.0)
            accum = 8 // world
            print(json.dumps({
                "metric": "train_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": value / PUBLISHED_TOKENS_PER_S, "dtype": "bf16",
                "data": "synthetic seeded Zipf(1.1) order-1 Markov uint16 shards; random-init weights", "impl": "reference",
                "config": {"model": ("records/track_10min_16mb/2026-03-23_LeakyReLU_LegalTTT_ParallelMuon/train_gpt.py (unmodified), VE off, BigramHash 3072"
                                     if record else "train_gpt.py (unmodified root trainer, 9L baseline)"),
                           "global_batch": GLOBAL_BATCH, "seq_len": SEQ_LEN,
                           "parallelism": f"dp{world} Parallel Muon (NCCL)" if record else f"dp{world} DDP + Muon (NCCL)", "grad_accum": accum,
                           "attention": "flash_attn_interface shim -> torch SDPA flash backend" if record else "torch SDPA",
                           "timing": "the script's own synchronized train_time"},
                "clocks": clocks,
                "e2e": {"value": value, "unit": "tokens/s", "note": "the script's loop already copies each batch host->device and logs from the host",
                        "h2d_bytes_per_step": 2 * 8 * (GLOBAL_BATCH // world), "d2h_bytes_per_step": 4},
                "gpu_launches": None, "wall_s": time.time() - t_wall,
            }))
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--config", default="record_11l", choices=sorted(CONFIGS), help="record_11l is the headline; baseline_9l is the 9-layer DDP baseline")
    ap.add_argument("--cuda-graph", action="store_true", help="replay each micro-batch forward+backward from a captured CUDA graph (native arm)")
    args = ap.parse_args()
    select_config(args.config)
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        sys.exit(run_reference(args))
    run_native(args)


if __name__ == "__main__":
    main()
