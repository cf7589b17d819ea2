"""CPU-only preliminary sweeps: quantisation schemes, prune/quantise ordering, architecture budget.

    python bench/preliminary.py                 # all three experiments, a few seconds
    python bench/preliminary.py --only arch     # one of: quant, prune, arch

Counterpart of ``parameter-golf-rs/crates/pg-bench/src/bin/preliminary.rs:25-290``:

1. every (attention bits, MLP bits, embedding bits) combination of interest on synthetic heavy-tailed weights of the
   record shape: packed bytes, zstd-22 bytes and reconstruction MSE;
2. prune-then-quantise against quantise-then-prune at several keep ratios, and the 2:4 mask;
3. parameter counts, estimated artifact bytes at int6 / mixed int5-int6 and the CUDA engine's memory estimate for every
   built-in family, against the 16,000,000-byte budget.

Prints tables and one closing JSON line.
"""
import argparse
import json
import os
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from parameter_golf_b200.models import gpt  # noqa: E402
from parameter_golf_b200.plan import estimate_engine_memory  # noqa: E402
from parameter_golf_b200.quant import container as C  # noqa: E402
from parameter_golf_b200.quant import quantize as Q  # noqa: E402
from parameter_golf_b200.spec import FAMILIES, family_preset  # noqa: E402

BUDGET = 16_000_000


def realistic_weights(rows: int, cols: int, seed: int) -> torch.Tensor:
    """Gaussian bulk with a 1 % heavy tail, the shape trained projection matrices tend to have."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, cols, generator=g) * 0.02
    tail = torch.rand(rows, cols, generator=g) < 0.01
    return torch.where(tail, w * 6.0, w)


def packed_and_compressed(q: torch.Tensor, bits: int):
    raw = C.pack_bits(q.numpy().astype(np.int8), bits)
    return len(raw), len(C.zstd_compress(raw, 22))


def quant_sweep():
    print("== 1. quantisation sweep (synthetic record-shaped weights: attention 512x512, MLP 1536x512, embedding 1024x512)")
    mats = {"attn": realistic_weights(512, 512, 1), "mlp": realistic_weights(1536, 512, 2), "embed": realistic_weights(1024, 512, 3)}
    counts = {"attn": 11 * 2 + 11, "mlp": 11 * 2, "embed": 1}          # q,o (512x512) + k,v (2 x 256x512 = one 512x512); up, down
    rows = []
    print(f"{'attn':>5} {'mlp':>4} {'emb':>4} {'packed MB':>10} {'zstd-22 MB':>11} {'attn mse':>10} {'mlp mse':>10} {'fits 16 MB':>10}")
    cache = {}
    for a, m_, e in [(8, 8, 8), (7, 7, 8), (6, 6, 8), (6, 5, 8), (6, 4, 8), (5, 5, 8), (5, 4, 8), (7, 4, 8), (8, 4, 8), (4, 4, 8), (6, 6, 6), (5, 5, 6)]:
        tot_p = tot_z = 0
        mse = {}
        for name, bits in (("attn", a), ("mlp", m_), ("embed", e)):
            if (name, bits) not in cache:
                q, s = Q.quantize_rows(mats[name], bits)
                p, z = packed_and_compressed(q, bits)
                err = float((mats[name] - Q.dequantize_rows(q, s.half())).pow(2).mean())
                cache[(name, bits)] = (p, z, err)
            p, z, err = cache[(name, bits)]
            tot_p += p * counts[name]
            tot_z += z * counts[name]
            mse[name] = err
        rows.append({"attn_bits": a, "mlp_bits": m_, "embed_bits": e, "packed_bytes": tot_p, "zstd_bytes": tot_z, "attn_mse": mse["attn"],
                     "mlp_mse": mse["mlp"], "fits": tot_z <= BUDGET})
        print(f"{a:>5} {m_:>4} {e:>4} {tot_p / 1e6:>10.2f} {tot_z / 1e6:>11.2f} {mse['attn']:>10.3e} {mse['mlp']:>10.3e} {str(tot_z <= BUDGET):>10}")
    # the group-scaled low-bit schemes of the 2026-03-24 submissions on the same matrices: codes + one fp16 scale per 128 columns, xz
    import lzma
    from parameter_golf_b200.quant import binary as B1
    from parameter_golf_b200.quant import ternary as T3
    for label, quant, deq, pack in (("ternary", T3.quantize_ternary, T3.dequantize_ternary, T3.pack_trits),
                                    ("binary", B1.quantize_binary, B1.dequantize_binary, B1.pack_signs)):
        tot_p = tot_z = 0
        mse = {}
        for name in ("attn", "mlp"):
            q, sc = quant(mats[name], 128)
            raw = pack(q.numpy()) + sc.half().numpy().tobytes()
            tot_p += len(raw) * counts[name]
            tot_z += len(lzma.compress(raw, preset=9)) * counts[name]
            mse[name] = float((mats[name] - deq(q, sc.half().float(), 128)).pow(2).mean())
        emb = cache[("embed", 8)]
        tot_p, tot_z = tot_p + emb[0], tot_z + emb[1]
        rows.append({"scheme": label, "packed_bytes": tot_p, "xz_bytes": tot_z, "attn_mse": mse["attn"], "mlp_mse": mse["mlp"], "fits": tot_z <= BUDGET})
        print(f"{label:>14} {tot_p / 1e6:>10.2f} {tot_z / 1e6:>11.2f} {mse['attn']:>10.3e} {mse['mlp']:>10.3e} {str(tot_z <= BUDGET):>10}   (xz instead of zstd)")
    return rows


def prune_sweep():
    print("== 2. prune-then-quantise (A) against quantise-then-prune (B), int6, and the 2:4 mask")
    rows = []
    for name, (r, c) in (("attention 512x512", (512, 512)), ("MLP up 1536x512", (1536, 512))):
        w = realistic_weights(r, c, 7)
        print(f"  {name}")
        for keep in (0.9, 0.75, 0.5):
            ab = Q.ordering_ab_test(w, keep, 6)
            rows.append({"matrix": name, "keep": keep, **ab})
            print(f"    keep {keep:.2f}: A {ab['prune_then_quantize_mse']:.3e}  B {ab['quantize_then_prune_mse']:.3e}  "
                  f"{'A' if ab['prune_then_quantize_mse'] <= ab['quantize_then_prune_mse'] else 'B'} wins")
        mask = Q.prune_2_of_4(w)
        q, s = Q.quantize_rows(w * mask, 6)
        err = float((w - Q.dequantize_rows(q, s.half())).pow(2).mean())
        rows.append({"matrix": name, "keep": "2:4", "prune_then_quantize_mse": err})
        print(f"    2:4 mask ({float(mask.float().mean()):.2f} kept) then int6: mse {err:.3e}")
    return rows


def arch_sweep():
    print("== 3. architecture families: parameters, estimated artifact bytes, engine memory for one record micro-batch")
    print(f"{'family':>28} {'params':>12} {'int6 MB':>9} {'int5/6 MB':>10} {'fits':>5} {'engine GiB @98,304 tok':>23}   (ternary / binary families: their own scheme before xz in both columns; xz takes a few percent off the scales and codes)")
    rows = []
    from parameter_golf_b200.spec import ARCH_VARIANTS, arch_label, arch_variant
    # the families, then the reference's ten sweep architectures (pg-bench/src/bin/preliminary.rs:247-290, pg-model/src/arch.rs:137-168)
    for fam in list(FAMILIES) + [f"arch:{k}" for k in ARCH_VARIANTS]:
        s = arch_variant(fam[5:]) if fam.startswith("arch:") else family_preset(fam)
        if fam.startswith("arch:"):
            fam = arch_label(fam[5:])
        m = s.model
        shapes = gpt.param_shapes(m)
        n_params = gpt.count_params(m)
        bank = {k: int(np.prod(shapes[k])) for k in gpt.BANKS}
        emb = int(np.prod(shapes["tok_emb"]))
        other = n_params - sum(bank.values()) - emb
        ratio = 0.78                                         # zstd-22 on packed int6 of trained-like weights (measured in part 1)
        int6 = (sum(bank.values()) * 6 / 8 + emb) * ratio + other * 2
        attn = bank["qo_bank"] + bank["kv_bank"]
        mlp = bank["mlp_up_bank"] + bank["mlp_down_bank"]
        mixed = ((attn * 6 + mlp * 5) / 8 + emb) * ratio + other * 2
        if s.quant.scheme == "ternary_b158":                # five codes per byte plus one fp16 scale per group; xz gains little on top
            tern = sum(bank.values()) * (1 / 5 + 2 / s.quant.ternary_group) + emb + other * (1 if s.quant.float_storage == "fp8" else 2)
            int6 = mixed = tern
        if s.quant.scheme == "binary_b1":                   # eight codes per byte plus one fp16 scale per group
            int6 = mixed = sum(bank.values()) * (1 / 8 + 2 / s.quant.ternary_group) + emb + other * (1 if s.quant.float_storage == "fp8" else 2)
        try:
            mem = estimate_engine_memory(s, 98304).total / 2 ** 30
        except Exception:
            mem = float("nan")
        rows.append({"family": fam, "params": n_params, "int6_bytes": int(int6), "mixed_bytes": int(mixed), "fits": mixed <= BUDGET,
                     "engine_gib": mem})
        print(f"{fam:>28} {n_params:>12,} {int6 / 1e6:>9.2f} {mixed / 1e6:>10.2f} {str(mixed <= BUDGET):>5} {mem:>23.1f}")
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="", help="quant, prune or arch")
    a = ap.parse_args()
    t0 = time.perf_counter()
    out = {"bench": "preliminary"}
    if a.only in ("", "quant"):
        out["quant"] = quant_sweep()
    if a.only in ("", "prune"):
        out["prune"] = prune_sweep()
    if a.only in ("", "arch"):
        out["arch"] = arch_sweep()
    out["seconds"] = round(time.perf_counter() - t0, 2)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
