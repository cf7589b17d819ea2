"""Per-phase device times of the sharded optimizer tail (CUDA events, max over ranks), overlapped schedule against the
serial one, on the record 11-layer configuration.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench/dist_tail_profile.py [--steps 5] [--warmup 3]

Each phase is reported as milliseconds after the last backward kernel of the step (the event recorded on the main stream
when the backward pass has been queued). ``main stream resumes`` is the exposed part: what the next step's forward waits
for. The serial schedule runs the same kernels on one stream, starting the gradient reduction after the whole backward
pass (the shape of the step before the reduction moved under the backward). Counterpart of the reference's overlap
observer timing (``parameter-golf-rs/crates/pg-train/src/lib.rs:3155-3243``).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from parameter_golf_b200.models import gpt  # noqa: E402
from parameter_golf_b200.models.engine import EngineBackend  # noqa: E402
from parameter_golf_b200.ops import native as N  # noqa: E402
from parameter_golf_b200.spec import family_preset  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    rows = {}
    for overlap in (False, True):
        spec = family_preset("record_11l")           # the 11-layer record configuration, 786,432 tokens per step
        spec.mode = "record_shaped_proxy"
        t = spec.train
        t.rank, t.world_size, t.backend = rank, world, "cuda_distributed"
        t.distributed_optimizer_backend = "sharded_parallel_muon"
        spec.validate()
        params = gpt.init_params(spec.model, t.seed)
        be = EngineBackend(spec, params, overlap_optimizer=overlap)
        T = be.engine.T
        g = torch.Generator().manual_seed(1 + rank)
        spans = [torch.randint(0, spec.model.vocab_size, (T + 1,), generator=g).to(torch.int16).cuda() for _ in range(be.accum)]
        acc = {}
        for s in range(a.warmup + a.steps):
            if s >= a.warmup:
                be.dist.enable_timing(True)
            be.train_step_spans(spans, 1.0, 0.95, staged=True)
            if s >= a.warmup:
                for name, ms in be.dist.phase_times():
                    acc.setdefault(name, []).append(ms)
                be.dist.enable_timing(False)
        torch.cuda.synchronize()
        N.check_status()
        names = list(acc)
        v = torch.tensor([sum(acc[k]) / len(acc[k]) for k in names], device="cuda", dtype=torch.float64)
        lo = v.clone()
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        # max over ranks: what the fastest rank sees (it also waits for the slowest rank's backward to end);
        # min over ranks: the rank whose backward ends last, i.e. the communication and optimizer work itself
        rows["overlapped" if overlap else "serial"] = {k: [round(a_, 4), round(b_, 4)] for k, a_, b_ in zip(names, v.tolist(), lo.tolist())}
        dist.barrier()
        be.dist.close()
        del be
        torch.cuda.empty_cache()
    if rank == 0:
        print(json.dumps({"bench": "sharded_optimizer_tail", "gpus": world, "unit": "ms after the end of the rank's own backward pass: [max over ranks, min over ranks]", "rows": rows}))
        for mode, r in rows.items():
            print(mode)
            for k, x in r.items():
                print(f"  {k:28s} max over ranks {x[0]:8.3f} ms   min over ranks {x[1]:8.3f} ms")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
