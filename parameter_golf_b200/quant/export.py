"""Export a trained parameter dict to the quantised artifact and load it back.

Tensor order and names follow ``parameter-golf-rs/crates/pg-quant/src/export.rs:48-183``: for each group in
``qo_bank.q, qo_bank.o, kv_bank.k, kv_bank.v, mlp_up_bank, mlp_down_bank, tok_emb``: optional four LQER tensors
``<g>.lqer.{a,b}.{weight,scale}``, then ``<g>.weight`` (dtype code I8, shape [rows, cols], payload bit-packed to
``ceil(rows*cols*bits/8)`` bytes) and ``<g>.scale`` (F16 [rows]); then ``bigram_embed``, ``bigram_proj`` (F16),
``bigram_scale`` (F32 [1]); ``smear_gate``, ``skip_weights`` (F16); per block
``blocks.{i}.{attn_scale,mlp_scale,resid_mix,q_gain}`` (F16) plus gate tensors; ``ve_embed``, ``ve_proj`` (F16),
``ve_scale`` (F32), ``ve_layer_scales`` (F16). Per-group bit widths are recorded in the metadata ``"groups"`` map
and read back from there at load (``export.rs:987-1000``). Legacy ``pgrs_int6`` artifacts with un-split
``qo_bank.weight`` / ``kv_bank.weight`` names are accepted (``export.rs:769-807``).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from ..models.gpt import bank_views, param_shapes, up_rows
from ..spec import RunSpec
from . import container as C
from .quantize import GROUPS, LqerFactors, dequantize_rows, lqer_factors, lqer_reconstruct, prune_rows, quantize_rows, scheme_bits

CODE_BUDGET_ENV = "PG_SUBMISSION_CODE_BYTES"
DEPTH_LORA = ("q_down", "q_up", "v_down", "v_up")


def _f16(name, t) -> C.TensorRecord:
    a = t.detach().cpu().float().numpy().astype("<f2")
    return C.TensorRecord(name, tuple(a.shape), "f16", a.tobytes())


def _flt(name, t, storage: str) -> C.TensorRecord:
    """A 2-D float tensor in the artifact's float storage: f16, or FP8 e4m3 at one byte per element (the ternary record's
    choice for everything it does not code, train_gpt_cuda_ternary.py:218-221)."""
    if storage != "fp8" or t.ndim != 2:
        return _f16(name, t)
    a = t.detach().cpu().float().clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    return C.TensorRecord(name, tuple(a.shape), "f8e4m3", a.tobytes())


def _f32(name, t) -> C.TensorRecord:
    a = t.detach().cpu().float().numpy().astype("<f4")
    return C.TensorRecord(name, tuple(a.shape), "f32", a.tobytes())


def metadata_json(spec: RunSpec, bits: Dict[str, int]) -> str:
    m, q = spec.model, spec.quant
    md = {
        "format": "pgrs_quant", "version": 2, "variant_fingerprint": f"{spec.fingerprint():016x}",
        "scheme": q.scheme, "compression": q.compression, "matrix_bits": q.matrix_bits, "embed_bits": q.embed_bits,
        "attn_gate_bits": q.attn_gate_bits, "mlp_clip_sigmas": q.mlp_clip_sigmas, "attn_clip_sigmas": q.attn_clip_sigmas,
        "embed_clip_sigmas": q.embed_clip_sigmas, "gptq_calibration_batches": q.gptq_calibration_batches,
        "prune_keep_ratio": q.prune_keep_ratio, "lqer_enabled": int(q.lqer.enabled), "lqer_rank": q.lqer.rank,
        "lqer_top_k": q.lqer.top_k, "lqer_a_bits": q.lqer.a_bits, "lqer_b_bits": q.lqer.b_bits,
        "lqer_group_size": q.lqer.group_size, "lqer_asymmetric": int(q.lqer.asymmetric),
        "vocab_size": m.vocab_size, "num_layers": m.num_layers, "model_dim": m.model_dim, "num_heads": m.num_heads,
        "num_kv_heads": m.num_kv_heads, "head_dim": m.head_dim, "mlp_dim": m.mlp_dim,
        "attn_out_gate_enabled": int(m.attn_out_gate.enabled), "attn_out_gate_width": m.attn_out_gate.width,
        "sparse_attn_gate_enabled": int(m.sparse_attn_gate.enabled), "sparse_attn_gate_width": m.sparse_attn_gate.width,
        "groups": {g: bits[g] for g in GROUPS}, "code_storage": q.code_storage, "scheme": q.scheme, "ternary_group": q.ternary_group,
    }
    return json.dumps(md, separators=(",", ":"))


def quantize_groups(spec: RunSpec, params: Dict[str, torch.Tensor], precomputed: Optional[Dict[str, Tuple[torch.Tensor, torch.Tensor]]] = None):
    """(q int8, scale f32) per group. ``precomputed`` lets GPTQ supply its own integers."""
    bits = scheme_bits(spec.quant.scheme, spec.quant.matrix_bits, spec.quant.embed_bits)
    views = bank_views(spec.model, params)
    out = {}
    for g in GROUPS:
        if precomputed is not None and g in precomputed:
            out[g] = precomputed[g]
            continue
        w = views[g].detach().cpu().float()
        if spec.quant.prune_keep_ratio is not None and g != "tok_emb":
            w = prune_rows(w, spec.quant.prune_keep_ratio)
        if spec.quant.scheme == "ternary_b158" and g != "tok_emb":
            from .ternary import quantize_ternary
            out[g] = quantize_ternary(w, spec.quant.ternary_group)          # codes in {-1, 0, 1}, scales [rows, groups]
        elif spec.quant.scheme == "binary_b1" and g != "tok_emb":
            from .binary import quantize_binary
            out[g] = quantize_binary(w, spec.quant.ternary_group)           # codes in {-1, 1}, scales [rows, groups]
        elif g == "tok_emb" and bits[g] == 16:
            out[g] = (w.half(), torch.ones(w.shape[0]))                     # kept as fp16: no codes, the scale is a placeholder
        else:
            out[g] = quantize_rows(w, bits[g])
            if spec.quant.coarse_layers and spec.quant.coarse_step > 1 and g != "tok_emb":
                out[g] = (_coarsen_rows(out[g][0], spec, bits[g]), out[g][1])
    return out, bits


def _coarsen_rows(q: torch.Tensor, spec: RunSpec, bits: int) -> torch.Tensor:
    """Codes of the blocks in ``quant.coarse_layers`` rounded to multiples of ``quant.coarse_step`` (a group's rows are the
    blocks' matrices stacked in order), kept inside the code range; see `int8_baseline.coarsen_bank_codes`."""
    n, step = spec.model.num_layers, spec.quant.coarse_step
    per = q.shape[0] // n
    lo, hi = -(1 << (bits - 1)), (1 << (bits - 1)) - 1
    q = q.clone()
    for l in set(int(x) for x in spec.quant.coarse_layers):
        blk = q[l * per:(l + 1) * per]
        q[l * per:(l + 1) * per] = (torch.round(blk.float() / step) * step).clamp(lo, hi).to(q.dtype)
    return q


def _store_codes(q: torch.Tensor, bits: int, storage: str) -> bytes:
    if storage == "bytes":
        return q.cpu().numpy().astype(np.int8).tobytes()
    return C.pack_bits(q.cpu().numpy(), bits)


def build_artifact(spec: RunSpec, params: Dict[str, torch.Tensor], precomputed=None, quantized=None) -> bytes:
    """Serialise to the (uncompressed) PGRS byte string. ``quantized`` = (codes and scales per group, bits) skips quantisation."""
    m = spec.model
    qs, bits = quantized if quantized is not None else quantize_groups(spec, params, precomputed)
    views = bank_views(m, params)
    recs = []
    for g in GROUPS:
        q, s = qs[g]
        s16 = s.half()
        if spec.quant.lqer.enabled and g != "tok_emb":
            resid = views[g].detach().cpu().float() - dequantize_rows(q, s16)
            f = lqer_factors(resid, spec.quant.lqer.rank, spec.quant.lqer.a_bits, spec.quant.lqer.b_bits)
            recs.append(C.TensorRecord(f"{g}.lqer.a.weight", tuple(f.a_q.shape), "i8", C.pack_bits(f.a_q.numpy(), spec.quant.lqer.a_bits)))
            recs.append(_f16(f"{g}.lqer.a.scale", f.a_s))
            recs.append(C.TensorRecord(f"{g}.lqer.b.weight", tuple(f.b_q.shape), "i8", C.pack_bits(f.b_q.numpy(), spec.quant.lqer.b_bits)))
            recs.append(_f16(f"{g}.lqer.b.scale", f.b_s))
        if spec.quant.scheme == "ternary_b158" and g != "tok_emb":
            from .ternary import pack_trits
            data = q.cpu().numpy().astype(np.int8).tobytes() if spec.quant.code_storage == "bytes" else pack_trits(q.cpu().numpy())
            recs.append(C.TensorRecord(f"{g}.weight", tuple(q.shape), "i8", data))        # five codes per byte, base 3
        elif spec.quant.scheme == "binary_b1" and g != "tok_emb":
            from .binary import pack_signs
            data = q.cpu().numpy().astype(np.int8).tobytes() if spec.quant.code_storage == "bytes" else pack_signs(q.cpu().numpy())
            recs.append(C.TensorRecord(f"{g}.weight", tuple(q.shape), "i8", data))        # eight codes per byte
        elif g == "tok_emb" and bits[g] == 16:
            recs.append(_f16(f"{g}.weight", q))
        else:
            recs.append(C.TensorRecord(f"{g}.weight", tuple(q.shape), "i8", _store_codes(q, bits[g], spec.quant.code_storage)))
        recs.append(_f16(f"{g}.scale", s16))
    if m.bigram.enabled:
        fs = spec.quant.float_storage
        if fs == "fp8":
            recs.append(_flt("bigram_embed", params["bigram_embed"], fs))
        else:
            recs.append(_f16("bigram_embed", params["bigram_embed"].reshape(-1)))
        if "bigram_proj" in params:
            recs.append(_flt("bigram_proj", params["bigram_proj"], fs) if fs == "fp8" else _f16("bigram_proj", params["bigram_proj"].reshape(-1)))
        recs.append(_f32("bigram_scale", params["bigram_scale"].reshape(1)))
    if "smear_gate" in params:
        recs.append(_f16("smear_gate", params["smear_gate"]))
    if "skip_weights" in params:
        recs.append(_f16("skip_weights", params["skip_weights"]))
    for i in range(m.num_layers):
        for k in ("attn_scale", "mlp_scale", "resid_mix", "q_gain"):
            recs.append(_f16(f"blocks.{i}.{k}", params[k][i]))
        if m.attn_out_gate.enabled:
            recs.append(_f16(f"blocks.{i}.attn_gate_weight", params["attn_gate_weight"][i]))
            recs.append(_f16(f"blocks.{i}.attn_gate_bias", params["attn_gate_bias"][i]))
        if m.sparse_attn_gate.enabled:
            recs.append(_f16(f"blocks.{i}.sparse_attn_gate_weight", params["sparse_attn_gate_weight"][i]))
        if m.value_residual:
            recs.append(_f16(f"blocks.{i}.vr_lambda", params["vr_lambda"][i]))
        if m.dtg:
            recs.append(_f16(f"blocks.{i}.dtg_gate_weight", params["dtg_gate_weight"][i]))
            recs.append(_f16(f"blocks.{i}.dtg_gate_bias", params["dtg_gate_bias"][i].reshape(1)))
        if m.block_smear:
            recs.append(_f16(f"blocks.{i}.block_smear_gate", params["block_smear_gate"][i]))
        if m.gated_attention:
            recs.append(_f16(f"blocks.{i}.gated_attn_weight", params["gated_attn_weight"][i]))
            recs.append(_f16(f"blocks.{i}.gated_attn_bias", params["gated_attn_bias"][i]))
    # the multi-token-prediction heads are training-only and are left out (records/.../2026-03-23_.../train_gpt.py:1778)
    if m.value_embedding.enabled:
        recs.append(_flt("ve_embed", params["ve_embed"], spec.quant.float_storage))
        recs.append(_flt("ve_proj", params["ve_proj"], spec.quant.float_storage))
        recs.append(_f32("ve_scale", params["ve_scale"].reshape(1)))
        recs.append(_f16("ve_layer_scales", params["ve_layer_scales"]))
    if not m.tie_embeddings:
        recs.append(_flt("lm_head", params["lm_head"], spec.quant.float_storage))
    if m.vocab_bias:
        recs.append(_f16("vocab_bias", params["vocab_bias"]))
    if "depth_lora_q_up" in params:
        for v in range(m.depth):
            for k in DEPTH_LORA:
                recs.append(_f16(f"depth.{v}.{k}", params[f"depth_lora_{k}"][v]))
    if m.embed_dim > 0:
        recs.append(_flt("embed_proj_in", params["embed_proj_in"], spec.quant.float_storage))
        recs.append(_flt("embed_proj_out", params["embed_proj_out"], spec.quant.float_storage))
    return C.write_pgrs(recs, metadata_json(spec, bits))


def export_model(spec: RunSpec, params: Dict[str, torch.Tensor], path: Optional[str] = None, precomputed=None) -> bytes:
    if spec.quant.scheme == "int8_zlib":         # the baseline trainer's own artifact, outside the PGRS family
        from .int8_baseline import export_int8_zlib
        q = spec.quant
        blob, _ = export_int8_zlib({k: v.detach().float().cpu() for k, v in params.items()}, keep_fp16=("tok_emb",) if q.embed_bits == 16 else (),
                                   coarse_layers=q.coarse_layers, coarse_step=q.coarse_step, num_layers=spec.model.num_layers)
    else:
        qs, bits = quantize_groups(spec, params, precomputed)
        blob = C.compress_payload(build_artifact(spec, params, quantized=(qs, bits)), spec.quant.compression)
        limit = spec.quant.target_artifact_bytes - code_bytes()
        if spec.quant.prune_to_target and spec.quant.scheme not in ("none", "ternary_b158", "binary_b1") and len(blob) > limit > 0:
            # +-1 pruning to the byte budget (the 2026-03-25 record's selective prune, train_gpt.py:1997-2040): the codes whose
            # removal costs least squared error go to zero until the compressed artifact fits beside the code
            from .quantize import selective_prune_to_target
            codes = {g: qs[g][0] for g in GROUPS if g != "tok_emb"}
            scales = {g: qs[g][1] for g in GROUPS if g != "tok_emb"}

            # The search runs on a fast proxy (zstd level 3 when the real mode is level 22, scaled by the ratio of the two on
            # the unpruned artifact, with a margin); level 22 on 27 MB takes ~10 s per try. The result is checked with the
            # real compressor and tightened if the proxy was optimistic.
            fast = spec.quant.compression == "zstd22"

            def real_size(cand):
                merged = dict(qs)
                merged.update({g: (cand[g], qs[g][1]) for g in cand})
                return len(C.compress_payload(build_artifact(spec, params, quantized=(merged, bits)), spec.quant.compression))

            ratio = len(blob) / max(len(C.zstd_compress(build_artifact(spec, params, quantized=(qs, bits)), 3)), 1) if fast else 1.0

            def size_of(cand):
                if not fast:
                    return real_size(cand)
                merged = dict(qs)
                merged.update({g: (cand[g], qs[g][1]) for g in cand})
                return int(len(C.zstd_compress(build_artifact(spec, params, quantized=(merged, bits)), 3)) * ratio)

            goal = limit
            for attempt in range(4):
                pruned, count = selective_prune_to_target(codes, scales, size_of, goal, max_iters=10, max_magnitude=spec.quant.prune_max_magnitude)
                merged = dict(qs)
                merged.update({g: (pruned[g], qs[g][1]) for g in pruned})
                blob = C.compress_payload(build_artifact(spec, params, quantized=(merged, bits)), spec.quant.compression)
                if len(blob) <= limit or not fast:
                    break
                goal = int(goal - 1.5 * (len(blob) - limit))           # the proxy under-estimated: aim lower by the miss and a half
            export_model.last_pruned = count
    if path:
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "wb") as f:
            f.write(blob)
    return blob


def _np(rec: C.TensorRecord) -> np.ndarray:
    dt = {"f16": "<f2", "f32": "<f4", "i32": "<i4", "u16": "<u2", "u32": "<u4", "i8": "i1"}.get(rec.dtype)
    if rec.dtype == "f8e4m3":
        raw = torch.frombuffer(bytearray(rec.data), dtype=torch.uint8).view(torch.float8_e4m3fn)
        return raw.float().numpy().reshape(rec.dims)
    if rec.dtype == "bf16":
        u = np.frombuffer(rec.data, dtype="<u2").astype(np.uint32) << 16
        return u.view(np.float32).reshape(rec.dims)
    return np.frombuffer(rec.data, dtype=dt).reshape(rec.dims)


def load_artifact(blob: bytes, spec: RunSpec, device="cpu", dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """De-quantise an artifact into a parameter dict laid out as `param_shapes`."""
    if blob[:1] == b"\x78":                      # zlib stream: the baseline's int8 export
        import zlib
        from .int8_baseline import MAGIC, dequantize_state_dict_int8, deserialize
        raw = zlib.decompress(blob)
        if raw[:4] != MAGIC:
            raise C.ArtifactError("zlib stream does not hold an int8 baseline container")
        out = dequantize_state_dict_int8(deserialize(raw))
        return {k: v.to(device=device, dtype=dtype if v.is_floating_point() else v.dtype) for k, v in out.items()}
    recs, metadata = C.read_pgrs(C.decompress_payload(blob))
    md = json.loads(metadata)
    m = spec.model
    if md.get("format") not in ("pgrs_quant", "pgrs_int6"):
        raise C.ArtifactError(f"unknown artifact format {md.get('format')!r}")
    for key, exp in (("vocab_size", m.vocab_size), ("num_layers", m.num_layers), ("model_dim", m.model_dim),
                     ("num_heads", m.num_heads), ("num_kv_heads", m.num_kv_heads), ("head_dim", m.head_dim),
                     ("mlp_dim", m.mlp_dim), ("attn_out_gate_enabled", int(m.attn_out_gate.enabled)),
                     ("sparse_attn_gate_enabled", int(m.sparse_attn_gate.enabled))):
        if key in md and int(md[key]) != int(exp):
            raise C.ArtifactError(f"artifact metadata mismatch for {key}: expected {exp}, got {md[key]}")
    by = {r.name: r for r in recs}
    n, d, kv, mlp = m.num_layers, m.model_dim, m.kv_dim, m.mlp_dim
    legacy = md.get("format") == "pgrs_int6"

    def group(g: str) -> torch.Tensor:
        bits = 6 if legacy else int(md["groups"][g])
        wrec, srec = by[f"{g}.weight"], by[f"{g}.scale"]
        rows, cols = wrec.dims
        if wrec.dtype == "f16":                  # an embedding table kept as fp16 (quant.embed_bits = 16)
            return torch.from_numpy(_np(wrec).astype(np.float32))
        if md.get("scheme") == "ternary_b158" and g != "tok_emb":
            from .ternary import dequantize_ternary, unpack_trits
            if len(wrec.data) == rows * cols:
                q = torch.from_numpy(np.frombuffer(wrec.data, dtype=np.int8).copy().reshape(rows, cols))
            else:
                q = torch.from_numpy(unpack_trits(wrec.data, rows * cols).copy().reshape(rows, cols))
            return dequantize_ternary(q, torch.from_numpy(_np(srec).astype(np.float32)), int(md.get("ternary_group", 128)))
        if md.get("scheme") == "binary_b1" and g != "tok_emb":
            from .binary import dequantize_binary, unpack_signs
            if len(wrec.data) == rows * cols:
                q = torch.from_numpy(np.frombuffer(wrec.data, dtype=np.int8).copy().reshape(rows, cols))
            else:
                q = torch.from_numpy(unpack_signs(wrec.data, rows * cols).copy().reshape(rows, cols))
            return dequantize_binary(q, torch.from_numpy(_np(srec).astype(np.float32)), int(md.get("ternary_group", 128)))
        if (legacy or md.get("code_storage") == "bytes") and len(wrec.data) == rows * cols:
            q = torch.from_numpy(np.frombuffer(wrec.data, dtype=np.int8).astype(np.int32).reshape(rows, cols))
        else:
            q = torch.from_numpy(C.unpack_bits(wrec.data, rows * cols, bits).reshape(rows, cols))
        w = dequantize_rows(q, torch.from_numpy(_np(srec).astype(np.float32)))
        if f"{g}.lqer.a.weight" in by:
            ar, br = by[f"{g}.lqer.a.weight"], by[f"{g}.lqer.b.weight"]
            f = LqerFactors(
                torch.from_numpy(C.unpack_bits(ar.data, ar.dims[0] * ar.dims[1], int(md["lqer_a_bits"])).reshape(ar.dims)),
                torch.from_numpy(_np(by[f"{g}.lqer.a.scale"]).astype(np.float32)),
                torch.from_numpy(C.unpack_bits(br.data, br.dims[0] * br.dims[1], int(md["lqer_b_bits"])).reshape(br.dims)),
                torch.from_numpy(_np(by[f"{g}.lqer.b.scale"]).astype(np.float32)))
            w = w + lqer_reconstruct(f)
        return w

    p: Dict[str, torch.Tensor] = {}
    if "qo_bank.weight" in by and "qo_bank.q.weight" not in by:      # legacy un-split names
        p["qo_bank"] = group("qo_bank").reshape(2 * n, d, d)
        p["kv_bank"] = group("kv_bank").reshape(2 * n, kv, d)
    else:
        p["qo_bank"] = torch.cat([group("qo_bank.q"), group("qo_bank.o")]).reshape(2 * n, d, d)
        p["kv_bank"] = torch.cat([group("kv_bank.k"), group("kv_bank.v")]).reshape(2 * n, kv, d)
    p["mlp_up_bank"] = group("mlp_up_bank").reshape(n, up_rows(m), d)
    p["mlp_down_bank"] = group("mlp_down_bank").reshape(n, d, mlp)
    p["tok_emb"] = group("tok_emb")
    shapes = param_shapes(m)
    for name in ("bigram_embed", "bigram_proj", "bigram_scale", "smear_gate", "skip_weights", "ve_embed", "ve_proj",
                 "ve_scale", "ve_layer_scales", "lm_head", "embed_proj_in", "embed_proj_out", "vocab_bias"):
        if name in shapes:
            if name not in by:
                raise C.ArtifactError(f"artifact is missing tensor {name}")
            p[name] = torch.from_numpy(_np(by[name]).astype(np.float32)).reshape(shapes[name])
    for k in ("attn_scale", "mlp_scale", "resid_mix", "q_gain", "attn_gate_weight", "attn_gate_bias", "sparse_attn_gate_weight", "vr_lambda", "dtg_gate_weight",
              "dtg_gate_bias", "block_smear_gate", "gated_attn_weight", "gated_attn_bias"):
        if k in shapes:
            p[k] = torch.stack([torch.from_numpy(_np(by[f"blocks.{i}.{k}"]).astype(np.float32)) for i in range(n)]).reshape(shapes[k])
    for k in DEPTH_LORA:
        if f"depth_lora_{k}" in shapes:
            p[f"depth_lora_{k}"] = torch.stack([torch.from_numpy(_np(by[f"depth.{v}.{k}"]).astype(np.float32)) for v in range(m.depth)])
    return {k: v.to(device=device, dtype=dtype) for k, v in p.items()}


def code_bytes(root: Optional[str] = None) -> int:
    """Submission code size: ``PG_SUBMISSION_CODE_BYTES`` if set, else the Python/C++/CUDA sources
    under ``root`` (``parameter-golf-rs/crates/pg-train/src/lib.rs:6017-6051``)."""
    if os.environ.get(CODE_BUDGET_ENV):
        return int(os.environ[CODE_BUDGET_ENV])
    root = root or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    total = 0
    for dp, _, fns in os.walk(root):
        for fn in fns:
            if fn.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                total += os.path.getsize(os.path.join(dp, fn))
    return total


def check_budget(model_bytes: int, code: int, limit: int = 16_000_000) -> bool:
    """``code_bytes + model_bytes < limit`` (strict; ``pg-model/src/plan.rs:69-89``)."""
    return code + model_bytes < limit
