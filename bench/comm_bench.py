"""Muon collective sweep: the framework's peer-memory paths against NCCL (+cuBLAS) on the record parameter set.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench/comm_bench.py \
        [--widths 1,2,4,8,16] [--iters 10] [--tokens 98304]

Counterpart of the reference's ``nccl-bench`` (all-reduce / reduce-scatter / all-gather bus-bandwidth sweep,
``parameter-golf-rs/crates/pg-bench/src/bin/nccl_bench.rs:7-17``), restated on the tensors the optimizer really moves:
the four weight banks of the 11-layer model (QKV 512x1024, O 512x512, MLP 512x1536 and 1536x512 per layer), scaled
``width`` times in both dimensions.

Two pipelines are timed per width, each as (ours) vs (NCCL + torch/cuBLAS), and the collective step of each alone
(``rs``: peer-load reduce vs ``reduce_scatter_tensor``; ``ag``: store fan-out + ready counters vs ``all_gather_into_tensor``):

* ``rs_ns``  gradient reduce-scatter fused with the Newton-Schulz input: every rank reduces its own slots of the fp32
  gradient banks straight out of its peers' memory (plain NVLink loads, no staging copy), then one kernel applies
  momentum and Nesterov and writes the bf16 Newton-Schulz input with its sum of squares (the normalisation itself rides
  on the first Newton-Schulz products).  Baseline: ``reduce_scatter_tensor`` per bank (fp32, padded to equal shards as
  the reference's Parallel Muon does) followed by the momentum kernel and a normalisation kernel, the reference's sequence.
* ``ag_qkv`` updated-weight all-gather fused with the next forward's first QKV GEMM: owners cast their fp32 slots to
  bf16 and store them into every rank's weight buffer, bump per-layer ready counters, and the GEMM's producer warp
  polls layer 0's counter before its first weight tile.  Baseline: ``all_gather_into_tensor`` per bank (bf16) followed
  by a cuBLAS matmul.

Device-timed with CUDA events, max over ranks, 3 warm-ups.  Every timed repetition starts with a barrier so that no
rank's clock starts while a peer still works on the previous one.  Reports, per pipeline: milliseconds, the bytes that
have to cross NVLink per rank, bus GB/s (bytes / time) and the fraction of the roofline
``max(bytes / link bandwidth, GEMM FLOPs / measured bf16 peak)`` for both link figures: the 770 GB/s peer copy measured on
this pool and the 900 GB/s nominal.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from parameter_golf_b200.ops import native as N  # noqa: E402
from parameter_golf_b200.parallel.dist_engine import shard_range  # noqa: E402
from parameter_golf_b200.parallel.symm import SymmetricBuffer  # noqa: E402

LINK_GBS = 770.0        # measured peer copy bandwidth per direction per GPU on this pool
LINK_NOMINAL_GBS = 900.0   # NVLink 5 nominal per direction per GPU
LAYERS = 11


def bank_shapes(w):
    d, kv, mlp = 512 * w, 256 * w, 1536 * w
    return {"qo": (2 * LAYERS, d, d), "kv": (2 * LAYERS, kv, d), "up": (LAYERS, mlp, d), "down": (LAYERS, d, mlp)}


def timed(fn, iters, pre):
    ms = []
    for i in range(3 + iters):
        pre()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        if i >= 3:
            ms.append(a.elapsed_time(b))
    t = torch.tensor([sum(ms) / len(ms)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--widths", default="1,2,4,8,16")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--tokens", type=int, default=98304)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    C = N.load()
    peak_tf = 1590.0
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if os.path.exists(os.path.join(root, "MEASURED_PEAKS.json")):
        peak_tf = json.load(open(os.path.join(root, "MEASURED_PEAKS.json"))).get("bf16_tflops", peak_tf)
    sig = SymmetricBuffer(1024 * 4)
    sig.view(0, (1024,), torch.int32).zero_()
    flags = sig.view(0, (1024,), torch.int32)
    hp = torch.tensor([1.0, 0.95, 1, 1, 1.0, 0, 0, 0], device="cuda")
    epoch = [0]
    rows = []

    def barrier():
        epoch[0] += 1
        C.comm_barrier(sig.table, rank, world, 0, epoch[0], N.status_word())

    for w in [int(x) for x in args.widths.split(",")]:
        shapes = bank_shapes(w)
        d = 512 * w
        # ---- gradient side ---------------------------------------------------------------------------------------------
        off, g_off = 0, {}
        for k, s in shapes.items():
            g_off[k] = off
            off += s[0] * s[1] * s[2]
        gbuf = SymmetricBuffer(off * 4)
        gall = gbuf.view(0, (off,), torch.float32)
        gall.normal_()
        own = {k: shard_range(s[0], rank, world) for k, s in shapes.items()}
        red = {k: torch.empty((own[k][1] - own[k][0],) + s[1:], device="cuda") for k, s in shapes.items()}
        mom = {k: torch.zeros_like(v) for k, v in red.items()}
        U = {k: torch.empty_like(v, dtype=torch.bfloat16) for k, v in red.items()}
        X0 = {k: torch.empty_like(v, dtype=torch.bfloat16) for k, v in red.items()}
        sq = {k: torch.zeros(max(v.shape[0], 1), device="cuda") for k, v in red.items()}
        stats = torch.zeros(8, device="cuda")

        def ns_input(k, g):
            if g.shape[0]:
                sq[k].zero_()
                C.muon_momentum(g, mom[k], U[k], sq[k], hp, True)

        def ours_rs():
            barrier()                                  # every rank's gradients are final before anyone reads them
            for k, s in shapes.items():
                s0, s1 = own[k]
                if s1 > s0:
                    per = s[1] * s[2]
                    C.comm_reduce_peers(gbuf.table, world, g_off[k] + s0 * per, (s1 - s0) * per, red[k], 1.0 / world, stats, 1.0, None, 0, None)
                    ns_input(k, red[k])

        # NCCL baseline: equal padded shards, as the reference's Parallel Muon lays its banks out
        pad = {k: -(-s[0] // world) for k, s in shapes.items()}
        gpad = {k: torch.randn((pad[k] * world,) + s[1:], device="cuda") for k, s in shapes.items()}
        shard = {k: torch.empty((pad[k],) + s[1:], device="cuda") for k, s in shapes.items()}
        mom_b = {k: torch.zeros_like(v) for k, v in shard.items()}
        U_b = {k: torch.empty_like(v, dtype=torch.bfloat16) for k, v in shard.items()}
        X_b = {k: torch.empty_like(v, dtype=torch.bfloat16) for k, v in shard.items()}
        sq_b = {k: torch.zeros(pad[k], device="cuda") for k in shapes}

        def nccl_rs():
            for k in shapes:
                dist.reduce_scatter_tensor(shard[k], gpad[k], op=dist.ReduceOp.AVG)
                sq_b[k].zero_()
                C.muon_momentum(shard[k], mom_b[k], U_b[k], sq_b[k], hp, True)
                C.muon_normalize(U_b[k], X_b[k], sq_b[k], 1e-7)

        def pre():
            torch.cuda.synchronize()
            dist.barrier()

        def ours_rs_only():
            barrier()
            for k, s in shapes.items():
                s0, s1 = own[k]
                if s1 > s0:
                    per = s[1] * s[2]
                    C.comm_reduce_peers(gbuf.table, world, g_off[k] + s0 * per, (s1 - s0) * per, red[k], 1.0 / world, stats, 1.0, None, 0, None)

        def nccl_rs_only():
            for k in shapes:
                dist.reduce_scatter_tensor(shard[k], gpad[k], op=dist.ReduceOp.AVG)

        total = off
        rs_bytes = total * 4 * (world - 1) / world
        roof = rs_bytes / (LINK_GBS * 1e9) * 1e3
        t_ours = timed(ours_rs_only, args.iters, pre)
        t_nccl = timed(nccl_rs_only, args.iters, pre)
        rows.append({"pipeline": "rs", "width": w, "gpus": world, "ours_ms": round(t_ours, 4), "nccl_ms": round(t_nccl, 4),
                     "nvlink_bytes_per_rank": int(rs_bytes), "ours_bus_gbs": round(rs_bytes / t_ours / 1e6, 1),
                     "nccl_bus_gbs": round(rs_bytes / t_nccl / 1e6, 1), "roofline_ms": round(roof, 4),
                     "ours_frac_of_roofline": round(roof / t_ours, 3), "nccl_frac_of_roofline": round(roof / t_nccl, 3)})
        t_ours = timed(ours_rs, args.iters, pre)
        t_nccl = timed(nccl_rs, args.iters, pre)
        rows.append({"pipeline": "rs_ns", "width": w, "gpus": world, "ours_ms": round(t_ours, 4), "nccl_ms": round(t_nccl, 4),
                     "nvlink_bytes_per_rank": int(rs_bytes), "ours_bus_gbs": round(rs_bytes / t_ours / 1e6, 1),
                     "nccl_bus_gbs": round(rs_bytes / t_nccl / 1e6, 1), "roofline_ms": round(roof, 4),
                     "ours_frac_of_roofline": round(roof / t_ours, 3), "nccl_frac_of_roofline": round(roof / t_nccl, 3)})
        del gpad, shard, mom_b, U_b, X_b, red, mom, U, X0
        gbuf.close()
        torch.cuda.empty_cache()

        # ---- weight side ---------------------------------------------------------------------------------------------
        kv = 256 * w
        qkvw = d + 2 * kv
        n_w = LAYERS * qkvw * d + LAYERS * d * d + 2 * LAYERS * 3 * d * d
        wbuf = SymmetricBuffer(n_w * 2)
        w_off = {"qkv": 0, "o": LAYERS * qkvw * d, "up": LAYERS * qkvw * d + LAYERS * d * d, "down": LAYERS * qkvw * d + LAYERS * d * d + LAYERS * 3 * d * d}
        master = {k: torch.randn((own[k][1] - own[k][0],) + s[1:], device="cuda") * 0.02 for k, s in shapes.items()}
        Wqkv0 = wbuf.view(0, (qkvw, d), torch.bfloat16)
        T = args.tokens
        X = torch.randn(T, d, device="cuda").bfloat16()
        Y = torch.empty(T, qkvw, device="cuda", dtype=torch.bfloat16)
        step = [0]

        def dst_of(k, s):
            if k == "qo":
                return (s, w_off["qkv"] + s * qkvw * d) if s < LAYERS else (s - LAYERS, w_off["o"] + (s - LAYERS) * d * d)
            if k == "kv":
                layer = s % LAYERS
                return layer, w_off["qkv"] + layer * qkvw * d + (d if s < LAYERS else d + kv) * d
            if k == "up":
                return s, w_off["up"] + s * 3 * d * d
            return s, w_off["down"] + s * 3 * d * d

        desc = {}
        for k, s in shapes.items():
            s0, s1 = own[k]
            rows_d = []
            for slot in range(s0, s1):
                layer, dst = dst_of(k, slot)
                rows_d.append([dst, -1, 0, 128 + layer])
            desc[k] = torch.tensor(rows_d, dtype=torch.int64, device="cuda").reshape(-1, 4)

        def ours_push():
            for k, s in shapes.items():
                if own[k][1] > own[k][0]:
                    C.comm_push_cast_slots(master[k], wbuf.table, world, desc[k], s[2], False)     # one launch per bank shard
                    C.comm_flag_add_slots(sig.table, world, desc[k], 1)

        def ours_ag():
            step[0] += 1
            ours_push()
            # layer 0 is complete once its Q, K, V, O, up and down slots have all arrived: 6 increments per step
            N.gemm(X, Wqkv0, Y, wait_flag=flags[128:129], wait_value=6 * step[0])

        def ours_ag_only():
            step[0] += 1
            ours_push()
            C.comm_wait_flag(flags[128:129], 6 * step[0], N.status_word())

        shard_w = {k: torch.randn((pad[k],) + s[1:], device="cuda").bfloat16() for k, s in shapes.items()}
        full_w = {k: torch.empty((pad[k] * world,) + s[1:], device="cuda", dtype=torch.bfloat16) for k, s in shapes.items()}
        Wq_lib = torch.randn(qkvw, d, device="cuda").bfloat16()

        def nccl_ag_only():
            for k in shapes:
                dist.all_gather_into_tensor(full_w[k], shard_w[k])

        def nccl_ag():
            nccl_ag_only()
            torch.matmul(X, Wq_lib.t(), out=Y)

        params = sum(s[0] * s[1] * s[2] for s in shapes.values())
        ag_bytes = params * 2 * (world - 1) / world
        flops = 2.0 * T * qkvw * d
        roof = ag_bytes / (LINK_GBS * 1e9) * 1e3
        t_ours = timed(ours_ag_only, args.iters, pre)
        t_nccl = timed(nccl_ag_only, args.iters, pre)
        rows.append({"pipeline": "ag", "width": w, "gpus": world, "ours_ms": round(t_ours, 4), "nccl_ms": round(t_nccl, 4),
                     "nvlink_bytes_per_rank": int(ag_bytes), "ours_bus_gbs": round(ag_bytes / t_ours / 1e6, 1),
                     "nccl_bus_gbs": round(ag_bytes / t_nccl / 1e6, 1), "roofline_ms": round(roof, 4),
                     "ours_frac_of_roofline": round(roof / t_ours, 3), "nccl_frac_of_roofline": round(roof / t_nccl, 3)})
        t_ours = timed(ours_ag, args.iters, pre)
        t_nccl = timed(nccl_ag, args.iters, pre)
        roof = max(ag_bytes / (LINK_GBS * 1e9), flops / (peak_tf * 1e12)) * 1e3
        rows.append({"pipeline": "ag_qkv", "width": w, "gpus": world, "ours_ms": round(t_ours, 4), "nccl_ms": round(t_nccl, 4),
                     "nvlink_bytes_per_rank": int(ag_bytes), "gemm_gflop": round(flops / 1e9, 1), "ours_bus_gbs": round(ag_bytes / t_ours / 1e6, 1),
                     "nccl_bus_gbs": round(ag_bytes / t_nccl / 1e6, 1), "roofline_ms": round(roof, 4),
                     "ours_frac_of_roofline": round(roof / t_ours, 3), "nccl_frac_of_roofline": round(roof / t_nccl, 3)})
        torch.cuda.synchronize()
        N.check_status()
        del shard_w, full_w, master, X, Y
        wbuf.close()
        torch.cuda.empty_cache()
        for r in rows[-4:]:
            nominal = r["nvlink_bytes_per_rank"] / (LINK_NOMINAL_GBS * 1e9) * 1e3
            if "gemm_gflop" in r:
                nominal = max(nominal, r["gemm_gflop"] * 1e9 / (peak_tf * 1e12) * 1e3)
            r["ours_frac_of_nominal_roofline"] = round(nominal / r["ours_ms"], 3)
            r["nccl_frac_of_nominal_roofline"] = round(nominal / r["nccl_ms"], 3)
        if rank == 0:
            for r in rows[-4:]:
                print(f"[w={w} N={world}] {r['pipeline']:7s} ours {r['ours_ms']:9.3f} ms ({r['ours_bus_gbs']:7.1f} GB/s, {r['ours_frac_of_roofline']:.2f} of the 770 GB/s roofline, "
                      f"{r['ours_frac_of_nominal_roofline']:.2f} of the 900 GB/s one)   NCCL {r['nccl_ms']:9.3f} ms ({r['nccl_bus_gbs']:7.1f} GB/s, {r['nccl_frac_of_roofline']:.2f}, "
                      f"{r['nccl_frac_of_nominal_roofline']:.2f})", flush=True)
    if rank == 0:
        print(json.dumps({"bench": "muon_collectives", "gpus": world, "link_gbs": LINK_GBS, "bf16_peak_tflops": peak_tf, "rows": rows}))
    sig.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
