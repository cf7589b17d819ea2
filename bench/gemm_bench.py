"""Times the tcgen05 GEMM on the model's matmul sites against cuBLAS (torch.matmul) with CUDA events.

    python bench/gemm_bench.py                 # record-profile shapes: 98,304 tokens per micro-step
    python bench/gemm_bench.py --tokens 16384  # small case for profiler captures

Every site of the training step appears with its three products (forward, input gradient, weight gradient) and the
fused epilogues the engine uses there. Between timed launches a 256 MB buffer is written so that no operand survives
in L2. Prints one line per product and a closing JSON line; fractions are of the measured cuBLAS bf16 peak when a
``MEASURED_PEAKS.json`` sits at the repository root.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from parameter_golf_b200.ops import native as n  # noqa: E402


def timed(fn, flush, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.fill_(1.0)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=98304)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", default="", help="comma-separated product names to run (e.g. qkv.fwd,mlp_up.dW)")
    ap.add_argument("--no-cublas", action="store_true")
    args = ap.parse_args()
    T = args.tokens
    peak = None
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if os.path.exists(os.path.join(root, "MEASURED_PEAKS.json")):
        peak = json.load(open(os.path.join(root, "MEASURED_PEAKS.json"))).get("bf16_tflops")
    flush = torch.empty(64 * 1024 * 1024, device="cuda")
    sites = [("qkv", 1024, 512), ("attn_out", 512, 512), ("mlp_up", 1536, 512), ("mlp_down", 512, 1536), ("lm_head", 1024, 512)]
    only = set(filter(None, args.only.split(",")))
    rows = []
    for name, N, K in sites:
        X = torch.randn(T, K, device="cuda").bfloat16()
        W = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
        Y = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        Y2 = torch.empty_like(Y)
        dY = torch.randn(T, N, device="cuda").bfloat16()
        dX = torch.empty(T, K, device="cuda", dtype=torch.bfloat16)
        dW = torch.zeros(N, K, device="cuda")
        resid = torch.randn(T, N, device="cuda").bfloat16()
        col = torch.ones(N, device="cuda")
        Hpre = torch.randn(T, K, device="cuda").bfloat16()
        flops = 2.0 * T * N * K
        products = {
            "fwd": (lambda: n.gemm(X, W, Y), lambda: torch.matmul(X, W.t(), out=Y)),
            "dX": (lambda: n.gemm(dY, W, dX, True, False), lambda: torch.matmul(dY, W, out=dX)),
            "dW": (lambda: n.gemm(dY, X, dW, False, False, n.EPI_F32_ATOMIC), lambda: torch.matmul(dY.t(), X)),
        }
        if name in ("attn_out", "mlp_down"):
            products["fwd+resid"] = (lambda: n.gemm(X, W, Y, epi=n.EPI_RESID_BF16, aux=resid, colscale=col), None)
        if name in ("attn_out", "mlp_down"):      # what the engine runs: residual add with the output scale folded into W
            products["fwd+axpby"] = (lambda: n.gemm(X, W, Y, epi=n.EPI_AXPBY_BF16, alpha=1.0, beta=1.0, aux=resid), None)
        if name == "mlp_up":
            products["fwd+act"] = (lambda: n.gemm(X, W, Y, epi=n.EPI_ACT_SQ, slope=0.5, D2=Y2), None)
        if name == "mlp_down":
            products["dX+actgrad"] = (lambda: n.gemm(dY, W, dX, True, False, epi=n.EPI_MUL_ACTGRAD, slope=0.5, aux=Hpre), None)
        for pname, (mine, lib) in products.items():
            key = f"{name}.{pname}"
            if only and key not in only:
                continue
            ms = timed(mine, flush, args.iters)
            ms_lib = timed(lib, flush, args.iters) if (lib is not None and not args.no_cublas) else None
            tf = flops / ms / 1e9
            row = {"product": key, "M": T, "N": N, "K": K, "ms": round(ms, 4), "tflops": round(tf, 1),
                   "cublas_ms": None if ms_lib is None else round(ms_lib, 4),
                   "frac_of_measured_peak": None if peak is None else round(tf / peak, 3)}
            rows.append(row)
            lib_txt = "" if ms_lib is None else f"  cuBLAS {ms_lib:.3f} ms ({flops / ms_lib / 1e9:.0f} TF)"
            print(f"{key:22s} M={T} N={N:5d} K={K:5d}  {ms:.3f} ms  {tf:6.0f} TF{lib_txt}")
    torch.cuda.synchronize()
    n.check_status()
    print(json.dumps({"bench": "gemm", "tokens": T, "l2": "flushed between launches (256 MB write)", "rows": rows}))


if __name__ == "__main__":
    main()
