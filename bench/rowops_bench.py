"""Row, loss, embedding and optimizer kernels one at a time at the record width (counterpart of the reference's per-kernel
timing in ``parameter-golf-rs/crates/pg-bench/src/bin/parity_kernels.rs``): CUDA-event time with L2 flushed between
launches, the bytes each call has to move (inputs read once + outputs written once), GB/s and the fraction of the measured
copy bandwidth (``MEASURED_PEAKS.json``, 6.65 TB/s if absent).

    python bench/rowops_bench.py [--tokens 32768] [--iters 10] [--only mix_norm_bwd]

``--only`` runs one kernel family once per iteration and nothing else after set-up, ``--once`` every family exactly once:
the forms the profiler captures use (`ncu -k regex:<kernels> -c <n>`). Shapes: d = 512, 8 query / 4 KV heads of 64, MLP 1536, vocabulary 1024, bigram 3072 x 128.
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from parameter_golf_b200.ops import native as N  # noqa: E402
from parameter_golf_b200.ops import reference as R  # noqa: E402

BF = torch.bfloat16


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", default=None)
    ap.add_argument("--once", action="store_true", help="launch every kernel exactly once, untimed (one profiler capture covers all families)")
    a = ap.parse_args()
    T, S, d, H, Hkv, hd, mlp, V, bk, bd = a.tokens, a.seq, 512, 8, 4, 64, 1536, 1024, 3072, 128
    kv, qkvw = Hkv * hd, H * hd + 2 * Hkv * hd
    C = N.load()
    peak = 6650.0
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = json.load(open(pk)).get("hbm_gbs", peak)
    g = torch.Generator(device="cuda").manual_seed(0)

    def bf(*shape):
        return torch.randn(*shape, device="cuda", generator=g).to(BF)

    def f32(*shape):
        return torch.randn(*shape, device="cuda", generator=g)

    x, x0, skip, x_in, h, d_h, d_res, d_x, d_x0, d_skip = (bf(T, d) for _ in range(10))
    mix, sw, d_mix, d_sw = f32(2, d), f32(d), torch.zeros(2, d, device="cuda"), torch.zeros(d, device="cuda")
    pre, post, d_post, d_pre = bf(T, qkvw), bf(T, qkvw), bf(T, qkvw), bf(T, qkvw)
    cos, sin = R.rope_tables(S, 16, 10000.0, train_seq_len=1024, device="cuda")
    gain, d_gain = f32(H), torch.zeros(H, device="cuda")
    y, z, dz, dy = bf(T, d), bf(T, d), bf(T, d), bf(T, d)
    vview, dv = pre[:, d + kv:], d_pre[:, d + kv:]
    gate, d_gate = f32(d), torch.zeros(d, device="cuda")
    ids = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
    tgt = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
    logits, nll, loss_sum = bf(T, V), torch.empty(T, device="cuda"), torch.zeros(1, device="cuda")
    E, BE = bf(V, d), bf(bk, bd)
    e_out, b_out = bf(T, d), bf(T, bd)
    dE, dBE = torch.zeros(V, d, device="cuda"), torch.zeros(bk, bd, device="cuda")
    nmat = 11
    pm = nmat * d * mlp                                   # one MLP bank: 8.65 M parameters
    p32, g32, m32, v32, ema = (f32(pm).abs() * 0.01 for _ in range(5))
    U = torch.empty(pm, device="cuda", dtype=BF)
    sq = torch.zeros(nmat, device="cuda")
    hp = torch.tensor([1.0, 0.95, 0.1, 0.05, 1.0, 0, 0, 0], device="cuda")
    Wb = torch.empty(nmat * mlp, d, device="cuda", dtype=BF)
    b2, b4 = 2, 4
    kernels = {
        # name: (call, bytes moved)
        "mix_norm_fwd": (lambda: C.mix_norm_fwd(x, x0, None, None, mix, x_in, h, 0.7, 1e-6), 4 * T * d * b2),
        "mix_norm_fwd_skip": (lambda: C.mix_norm_fwd(x, x0, skip, sw, mix, x_in, h, 0.7, 1e-6), 5 * T * d * b2),
        "norm_fwd": (lambda: C.mix_norm_fwd(x, None, None, None, None, None, h, 0.7, 1e-6), 2 * T * d * b2),
        "norm_bwd": (lambda: C.mix_norm_bwd(d_h, d_res, x_in, None, None, None, None, None, None, d_x, None, None, None, None, False, 0.7, 1e-6),
                     4 * T * d * b2),
        "mix_norm_bwd": (lambda: C.mix_norm_bwd(d_h, d_res, x_in, x, x0, None, None, mix, None, d_x, d_x0, None, d_mix, None, False, 0.7, 1e-6),
                         8 * T * d * b2),       # d_h, d_res, x_in, x, x0 read; d_x written; d_x0 read and written
        "mix_norm_bwd_skip": (lambda: C.mix_norm_bwd(d_h, d_res, x_in, x, x0, skip, sw, mix, None, d_x, d_x0, d_skip, d_mix, d_sw, False, 0.7, 1e-6),
                              10 * T * d * b2),
        "qk_norm_rope_fwd": (lambda: C.qk_norm_rope_fwd(pre, post, cos, sin, gain, H, Hkv, hd, 16, S, 1e-6), 2 * T * (d + kv) * b2),
        "qk_norm_rope_bwd": (lambda: C.qk_norm_rope_bwd(d_post, pre, d_pre, cos, sin, gain, d_gain, H, Hkv, hd, 16, S, 1e-6), 3 * T * (d + kv) * b2),
        "xsa_fwd": (lambda: C.xsa_fwd(y, vview, z, Hkv, H // Hkv, hd, 1e-8), T * (2 * d + kv) * b2),
        "xsa_bwd": (lambda: C.xsa_bwd(dz, y, vview, dy, dv, False, Hkv, H // Hkv, hd, 1e-8), T * (3 * d + 2 * kv) * b2),
        "norm_smear_fwd": (lambda: C.norm_smear_fwd(x, gate, None, h, S, -1, 1e-6), 2 * T * d * b2),
        "norm_smear_bwd": (lambda: C.norm_smear_bwd(d_h, x, gate, None, d_x, d_gate, S, -1, 1e-6), 3 * T * d * b2),
        "softcap_ce": (lambda: C.softcap_ce(logits, tgt, nll, logits, loss_sum, 30.0, 1.0 / T), 2 * T * V * b2),
        "embed_gather": (lambda: C.embed_gather(ids, E, e_out, 0, S), T * d * b2 + T * 4),
        "embed_gather_bigram": (lambda: C.embed_gather(ids, BE, b_out, bk, S), T * bd * b2 + T * 4),
        "embed_scatter_add": (lambda: C.embed_scatter_add(ids, d_x, dE, 0, S), T * d * b2 + T * 4),
        "embed_scatter_add_bigram": (lambda: C.embed_scatter_add(ids, b_out, dBE, bk, S), T * bd * b2 + T * 4),
        "adamw": (lambda: C.adamw(p32, g32, m32, v32, ema, hp, 0.01, 0.9, 0.95, 1e-8, 0.04, 0.997), 9 * pm * b4),
        "muon_momentum": (lambda: C.muon_momentum(g32.view(nmat, -1), m32.view(nmat, -1), U.view(nmat, -1), sq, hp, True), pm * (3 * b4 + b2)),
        "muon_apply": (lambda: C.muon_apply(p32, U, ema, hp, 0.025, 0.04, 1.0, 0.997), pm * (4 * b4 + b2)),
        "cast_rows": (lambda: C.cast_rows(p32.view(nmat * mlp, d), Wb, None, 0, 1, False), pm * (b4 + b2)),
        "cast_rows_fake_quant": (lambda: C.cast_rows(p32.view(nmat * mlp, d), Wb, None, 0, 1, True), pm * (2 * b4 + b2)),
        "sumsq": (lambda: C.sumsq(g32, 1.0, sq), pm * b4),
    }
    if a.once:
        for fn, _ in kernels.values():
            fn()
        torch.cuda.synchronize()
        N.check_status()
        return
    if a.only:
        fn, _ = kernels[a.only]
        for _ in range(a.iters):
            fn()
        torch.cuda.synchronize()
        N.check_status()
        return
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rows = []
    for name, (fn, nbytes) in kernels.items():
        for _ in range(3):
            fn()
        ms = []
        for _ in range(a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ms.append(e0.elapsed_time(e1))
        t = sorted(ms)[len(ms) // 2]
        gbs = nbytes / t / 1e6
        rows.append({"kernel": name, "ms": round(t, 4), "mbytes": round(nbytes / 1e6, 1), "gbs": round(gbs, 1), "frac_of_measured_copy": round(gbs / peak, 3)})
        print(f"{name:26s} {t * 1e3:9.1f} us  {nbytes / 1e6:8.1f} MB  {gbs:8.1f} GB/s  {gbs / peak:5.2f} of the measured {peak:.0f} GB/s copy")
    N.check_status()
    print(json.dumps({"bench": "rowops", "tokens": T, "l2": "flushed between launches (256 MB write)", "hbm_gbs_measured": peak, "rows": rows}))


if __name__ == "__main__":
    main()
