"""Times the fused soft-capped cross-entropy kernels and the embedding-gradient scatter with CUDA events.

    python bench/ce_bench.py                    # 98,304 rows: V = 1024 (one warp per row) and V = 8192 (one CTA per row)
    python bench/ce_bench.py --rows 16384       # small case for profiler captures

Loss + gradient in place over the bf16 logits, as the engine calls it; with and without per-row loss weights. The inputs
(201 MB at V = 1024, 1.6 GB at V = 8192) are larger than L2, so no flush is needed between launches. Bytes moved: the
narrow kernel reads the logits once and writes the gradient once; the wide one reads them twice. Fractions are of the
measured copy bandwidth when ``MEASURED_PEAKS.json`` sits at the repository root.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from parameter_golf_b200.ops import native  # noqa: E402


def timed(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=98304)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    C = native.load()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    peak = None
    if os.path.exists(os.path.join(root, "MEASURED_PEAKS.json")):
        peak = json.load(open(os.path.join(root, "MEASURED_PEAKS.json"))).get("hbm_gbs")
    T = a.rows
    out = []
    for V in (1024, 8192):
        z = (torch.randn(T, V, device="cuda") * 4).bfloat16()
        tgt = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
        prev = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
        nll = torch.empty(T, device="cuda")
        acc = torch.zeros(1, device="cuda")
        table = torch.rand(V, V, device="cuda")
        tw, wt = torch.empty(T, device="cuda"), torch.zeros(1, device="cuda")
        passes = 2 if V <= 2048 else 3
        gb = passes * T * V * 2 / 1e9
        for name, fn in (("loss+grad", lambda: C.softcap_ce(z, tgt, nll, z, acc, 30.0, 1.0 / T)),
                         ("loss+grad weighted", lambda: (C.pair_weights(prev, tgt, table, tw, wt), C.softcap_ce(z, tgt, nll, z, acc, 30.0, 1.0 / T, tw, wt))),
                         ("loss only", lambda: C.softcap_ce(z, tgt, nll, None, None, 30.0, 0.0))):
            ms = timed(fn, a.iters)
            moved = gb if name != "loss only" else T * V * 2 / 1e9
            row = {"op": f"softcap_ce V={V} {name}", "ms": round(ms, 4), "gb": round(moved, 3), "tb_per_s": round(moved / ms, 3),
                   "frac_of_measured_copy": None if peak is None else round(moved / ms * 1000 / peak, 3)}
            out.append(row)
            print(f"{row['op']:42s} {ms:8.3f} ms  {moved / ms:6.2f} TB/s")
        g = torch.randn(T, 512, device="cuda").bfloat16()
        dt = torch.zeros(V, 512, device="cuda")
        ms = timed(lambda: C.embed_scatter_add(tgt, g, dt, 0, 2048), a.iters)
        out.append({"op": f"embed_scatter_add table {V}x512", "ms": round(ms, 4)})
        print(f"{'embed_scatter_add table %dx512' % V:42s} {ms:8.3f} ms")
        del z, table
    torch.cuda.synchronize()
    native.check_status()
    print(json.dumps({"bench": "ce", "rows": T, "l2": "inputs larger than L2", "results": out}))


if __name__ == "__main__":
    main()
