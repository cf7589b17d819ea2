"""Attention micro-benchmark (counterpart of the reference's ``attention-bench`` binary,
``parameter-golf-rs/crates/pg-bench/src/bin/attention_bench.rs:19-32``): causal GQA attention forward and backward at the
record shape (B=48, S=2048, H=8, Hkv=4, hd=64) or a smaller one, timed with CUDA events, against PyTorch SDPA.

    python bench/attention_bench.py [--batch 48] [--seq 2048] [--iters 10] [--no-sdpa]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from parameter_golf_b200.ops import native as n  # noqa: E402


def timeit(fn, iters, warmup=3):
    for _ in range(warmup):
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
    ap.add_argument("--batch", type=int, default=48)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-sdpa", action="store_true")
    a = ap.parse_args()
    B, S, H, Hkv, hd = a.batch, a.seq, a.heads, a.kv_heads, 64
    qkv = torch.randn(B * S, (H + 2 * Hkv) * hd, device="cuda").bfloat16()
    q, k, v = qkv[:, :H * hd], qkv[:, H * hd:(H + Hkv) * hd], qkv[:, (H + Hkv) * hd:]
    y = torch.empty(B * S, H * hd, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn_like(y)
    dqkv = torch.empty_like(qkv)
    dq, dk, dv = dqkv[:, :H * hd], dqkv[:, H * hd:(H + Hkv) * hd], dqkv[:, (H + Hkv) * hd:]
    lse = torch.empty(B, H, S, device="cuda")
    ds = torch.empty(B, H, S, device="cuda")
    fl = 4.0 * B * H * S * S * hd / 2
    f = timeit(lambda: n.attn_fwd(q, k, v, y, B, S, H, Hkv, hd, lse), a.iters, a.warmup)
    b = timeit(lambda: n.attn_bwd(q, k, v, y, dy, lse, dq, dk, dv, B, S, H, Hkv, hd, dsum=ds), a.iters, a.warmup)
    b2 = timeit(lambda: n.attn_bwd(q, k, v, y, dy, lse, dq, dk, dv, B, S, H, Hkv, hd, dsum=ds, reproducible=True), a.iters, a.warmup)
    n.check_status()
    print(f"native  fwd {f:.3f} ms ({fl / f / 1e9:.0f} TFLOP/s)  bwd {b:.3f} ms ({2.5 * fl / b / 1e9:.0f} TFLOP/s at 2.5x forward FLOPs)"
          f"  two-kernel reproducible bwd {b2:.3f} ms")
    if not a.no_sdpa:
        import torch.nn.functional as F
        from torch.nn.attention import SDPBackend, sdpa_kernel
        q4 = q.reshape(B, S, H, hd).transpose(1, 2).detach().requires_grad_(True)
        k4 = k.reshape(B, S, Hkv, hd).transpose(1, 2).detach().requires_grad_(True)
        v4 = v.reshape(B, S, Hkv, hd).transpose(1, 2).detach().requires_grad_(True)
        for name, be in (("sdpa-flash", SDPBackend.FLASH_ATTENTION), ("sdpa-cudnn", SDPBackend.CUDNN_ATTENTION)):
            try:
                with sdpa_kernel(be):
                    ff = timeit(lambda: F.scaled_dot_product_attention(q4, k4, v4, is_causal=True, enable_gqa=True), a.iters, a.warmup)
                    o4 = F.scaled_dot_product_attention(q4, k4, v4, is_causal=True, enable_gqa=True)
                    g4 = torch.randn_like(o4)
                    bb = timeit(lambda: torch.autograd.grad(o4, (q4, k4, v4), g4, retain_graph=True), a.iters, a.warmup)
                print(f"{name} fwd {ff:.3f} ms ({fl / ff / 1e9:.0f} TFLOP/s)  bwd {bb:.3f} ms ({2.5 * fl / bb / 1e9:.0f} TFLOP/s)")
            except Exception as e:
                print(f"{name} unavailable: {type(e).__name__}")


if __name__ == "__main__":
    main()
