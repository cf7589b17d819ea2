"""Where one training step of the record configuration spends its device time, without a profiler.

    python bench/step_profile.py [--steps 2] [--warmup 2]

Every call into the kernel library is bracketed by CUDA events (`native.enable_timing`); the table gives, per kernel
(GEMMs split by epilogue and shape), calls per step, milliseconds per step and the share of the summed kernel time,
next to the wall time of the step measured by one pair of events around it. Kernel times include the gap to the
previous launch only when the stream was idle, so "sum of kernels" vs "step" shows how launch-bound the step is.
Single GPU (8 micro-batches of 48 x 2048 tokens per step), synthetic data.
"""
import argparse
import json
import os
import sys
import tempfile

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("overrides", nargs="*", help="spec overrides, key=value")
    args = ap.parse_args()
    from parameter_golf_b200.data.native_loader import NativeTokenLoader
    from parameter_golf_b200.data.shards import write_synthetic_dataset
    from parameter_golf_b200.models import gpt
    from parameter_golf_b200.models.engine import EngineBackend
    from parameter_golf_b200.ops import native
    from parameter_golf_b200.spec import family_preset

    spec = family_preset("record_11l")
    spec.mode = "record_shaped_proxy"
    spec.train.backend = "cuda_single"
    spec.apply_overrides(args.overrides)          # e.g. train.save_layer_acts=none
    spec.validate()
    root = write_synthetic_dataset(os.path.join(tempfile.gettempdir(), "pgb200_bench_data"), 1024, train_tokens=1 << 24,
                                   val_tokens=64 * 2048 + 1, train_shards=1, seed=1337)
    backend = EngineBackend(spec, gpt.init_params(spec.model, seed=1337))
    accum, tokens = backend.accum, 786432
    loader = NativeTokenLoader(os.path.join(root, "fineweb_train_*.bin"), 0, 1)
    loader.start_prefetch(tokens, accum)

    def step():
        return backend.train_step_spans([loader.next_prefetched() for _ in range(accum)], 1.0, 0.95, read_loss=True)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    native.enable_timing(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    wall = e0.elapsed_time(e1) / args.steps
    rep = native.timing_report()
    native.enable_timing(False)
    loader.stop_prefetch()
    native.check_status()
    total = sum(t for _, t in rep.values()) / args.steps
    print(f"step {wall:.2f} ms; sum of kernel brackets {total:.2f} ms ({100 * total / wall:.1f} % of the step)")
    rows = []
    for key, (calls, ms) in sorted(rep.items(), key=lambda kv: -kv[1][1]):
        rows.append({"op": key, "calls_per_step": calls / args.steps, "ms_per_step": round(ms / args.steps, 3), "share": round(ms / args.steps / total, 4)})
        print(f"{ms / args.steps:9.3f} ms {100 * ms / args.steps / total:5.1f} %  x{calls / args.steps:7.1f}  {1000 * ms / calls:8.1f} us  {key}")
    print(json.dumps({"bench": "step_profile", "step_ms": wall, "kernel_sum_ms": total, "rows": rows}))


if __name__ == "__main__":
    main()
