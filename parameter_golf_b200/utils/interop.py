"""PyTorch interop without third-party packages: safetensors reader/writer, state-dict name mapping, step parity.

* safetensors (F32/BF16/F16): 8-byte little-endian header length, JSON header ``{name: {dtype, shape, data_offsets}}``,
  then the raw little-endian payload (``parameter-golf-rs/crates/pg-compat/src/safetensors.rs:43-130``, ``writer.rs``).
* Name map between the Python records' ``state_dict`` (per-block ``blocks.{i}.attn_scale`` …, ``bigram.embed.weight`` …) and
  this framework's stacked parameter dict (``pg-compat/src/loader.rs:69-188``).
* Parity report of two step dumps with the reference tolerances ``loss_atol = 1e-3``, ``grad_max_rel = 0.02``
  (``pg-compat/src/parity.rs:30-34,85-198``).
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass, field
from typing import Dict, List

import numpy as np
import torch

from ..models.gpt import param_shapes
from ..spec import ModelSpec

_ST_DTYPES = {"F32": (np.dtype("<f4"), torch.float32), "F16": (np.dtype("<f2"), torch.float16), "BF16": (np.dtype("<u2"), torch.bfloat16)}
LOSS_ATOL = 1e-3
GRAD_MAX_REL = 0.02


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype == torch.float32:
            code, raw = "F32", t.numpy().astype("<f4").tobytes()
        elif t.dtype == torch.float16:
            code, raw = "F16", t.numpy().astype("<f2").tobytes()
        elif t.dtype == torch.bfloat16:
            code, raw = "BF16", t.view(torch.int16).numpy().astype("<i2").tobytes()
        else:
            raise TypeError(f"{name}: dtype {t.dtype} is not supported (F32/F16/BF16)")
        header[name] = {"dtype": code, "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    with open(path, "rb") as f:
        buf = f.read()
    if len(buf) < 8:
        raise ValueError("not a safetensors file")
    (hl,) = struct.unpack_from("<Q", buf, 0)
    if 8 + hl > len(buf):
        raise ValueError("safetensors header length exceeds the file")
    header = json.loads(buf[8:8 + hl])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        if info["dtype"] not in _ST_DTYPES:
            raise TypeError(f"{name}: dtype {info['dtype']} is not supported")
        npdt, tdt = _ST_DTYPES[info["dtype"]]
        a, b = info["data_offsets"]
        raw = np.frombuffer(buf, dtype=npdt, count=(b - a) // npdt.itemsize, offset=8 + hl + a).copy()
        t = torch.from_numpy(raw.view(np.int16) if info["dtype"] == "BF16" else raw)
        if info["dtype"] == "BF16":
            t = t.view(torch.bfloat16)
        out[name] = t.reshape(info["shape"])
    return out


def from_python_state_dict(m: ModelSpec, sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Map a record-style ``GPT.state_dict()`` onto this framework's parameter dict."""
    n = m.num_layers
    p: Dict[str, torch.Tensor] = {}
    direct = {"tok_emb.weight": "tok_emb", "qo_bank": "qo_bank", "kv_bank": "kv_bank", "mlp_up_bank": "mlp_up_bank", "mlp_down_bank": "mlp_down_bank",
              "skip_weights": "skip_weights", "smear.gate": "smear_gate", "bigram.embed.weight": "bigram_embed", "bigram.proj.weight": "bigram_proj",
              "ve_shared.embed.weight": "ve_embed", "ve_shared.proj.weight": "ve_proj", "lm_head.weight": "lm_head", "vocab_bias": "vocab_bias"}
    for src, dst in direct.items():
        if src in sd:
            p[dst] = sd[src].float()
    for src, dst in (("bigram.scale", "bigram_scale"), ("ve_shared.scale", "ve_scale")):
        if src in sd:
            p[dst] = sd[src].float().reshape(1)
    for k in ("attn_scale", "mlp_scale", "resid_mix"):
        if f"blocks.0.{k}" in sd:
            p[k] = torch.stack([sd[f"blocks.{i}.{k}"].float() for i in range(n)])
    if "blocks.0.attn.q_gain" in sd:
        p["q_gain"] = torch.stack([sd[f"blocks.{i}.attn.q_gain"].float() for i in range(n)])
    if "blocks.0.attn.vr_lambda" in sd:
        p["vr_lambda"] = torch.stack([sd[f"blocks.{i}.attn.vr_lambda"].float() for i in range(n)])
    if "blocks.0.dtg_gate.weight" in sd:
        p["dtg_gate_weight"] = torch.stack([sd[f"blocks.{i}.dtg_gate.weight"].float().reshape(-1) for i in range(n)])
        p["dtg_gate_bias"] = torch.stack([sd[f"blocks.{i}.dtg_gate.bias"].float().reshape(()) for i in range(n)])
    if "blocks.0.attn.attn_gate.weight" in sd:
        p["gated_attn_weight"] = torch.stack([sd[f"blocks.{i}.attn.attn_gate.weight"].float() for i in range(n)])
        p["gated_attn_bias"] = torch.stack([sd[f"blocks.{i}.attn.attn_gate.bias"].float() for i in range(n)])
    if "blocks.0.smear.gate" in sd:
        p["block_smear_gate"] = torch.stack([sd[f"blocks.{i}.smear.gate"].float() for i in range(n)])
    heads = [sd[k].float() for k in sorted((k for k in sd if k.startswith("mtp_heads.") and k.endswith(".weight")), key=lambda k: int(k.split(".")[1]))]
    if heads:
        p["mtp_heads"] = torch.stack(heads)
    ls = [sd[k].float().reshape(()) for k in sorted(sd) if k.startswith("ve_layer_scales.")]
    if ls:
        p["ve_layer_scales"] = torch.stack(ls)
    want = param_shapes(m)
    missing = [k for k in want if k not in p]
    if missing:
        raise KeyError(f"state dict lacks {missing}")
    for k in want:
        if tuple(p[k].shape) != tuple(want[k]):
            raise ValueError(f"{k}: shape {tuple(p[k].shape)} != expected {want[k]}")
    return p


def to_python_state_dict(m: ModelSpec, p: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    n = m.num_layers
    sd = {"tok_emb.weight": p["tok_emb"]}
    for k in ("qo_bank", "kv_bank", "mlp_up_bank", "mlp_down_bank", "skip_weights"):
        if k in p:
            sd[k] = p[k]
    if "smear_gate" in p:
        sd["smear.gate"] = p["smear_gate"]
    if "bigram_embed" in p:
        sd["bigram.embed.weight"] = p["bigram_embed"]
        sd["bigram.scale"] = p["bigram_scale"].reshape(())
        if "bigram_proj" in p:
            sd["bigram.proj.weight"] = p["bigram_proj"]
    if "ve_embed" in p:
        sd["ve_shared.embed.weight"], sd["ve_shared.proj.weight"] = p["ve_embed"], p["ve_proj"]
        sd["ve_shared.scale"] = p["ve_scale"].reshape(())
        for i in range(p["ve_layer_scales"].numel()):
            sd[f"ve_layer_scales.{i}"] = p["ve_layer_scales"][i].reshape(1)
    for i in range(n):
        for k in ("attn_scale", "mlp_scale", "resid_mix"):
            sd[f"blocks.{i}.{k}"] = p[k][i]
        sd[f"blocks.{i}.attn.q_gain"] = p["q_gain"][i]
        if "vr_lambda" in p:
            sd[f"blocks.{i}.attn.vr_lambda"] = p["vr_lambda"][i]
        if "dtg_gate_weight" in p:
            sd[f"blocks.{i}.dtg_gate.weight"] = p["dtg_gate_weight"][i].reshape(1, -1)
            sd[f"blocks.{i}.dtg_gate.bias"] = p["dtg_gate_bias"][i].reshape(1)
        if "block_smear_gate" in p:
            sd[f"blocks.{i}.smear.gate"] = p["block_smear_gate"][i]
        if "gated_attn_weight" in p:
            sd[f"blocks.{i}.attn.attn_gate.weight"], sd[f"blocks.{i}.attn.attn_gate.bias"] = p["gated_attn_weight"][i], p["gated_attn_bias"][i]
    if "mtp_heads" in p:
        for k in range(p["mtp_heads"].shape[0]):
            sd[f"mtp_heads.{k}.weight"] = p["mtp_heads"][k]
    if "lm_head" in p:
        sd["lm_head.weight"] = p["lm_head"]
    if "vocab_bias" in p:
        sd["vocab_bias"] = p["vocab_bias"]
    return sd


@dataclass
class ParityReport:
    loss_diff: float = 0.0
    worst_grad_rel: float = 0.0
    worst_grad_name: str = ""
    per_tensor: Dict[str, float] = field(default_factory=dict)
    missing: List[str] = field(default_factory=list)

    @property
    def ok(self) -> bool:
        return self.loss_diff <= LOSS_ATOL and self.worst_grad_rel <= GRAD_MAX_REL and not self.missing


def compare_step_dumps(a: Dict[str, torch.Tensor], b: Dict[str, torch.Tensor]) -> ParityReport:
    """``a``/``b``: {"loss": scalar, "grad.<name>": tensor, …}. Relative error is max|a-b| / max|b| per tensor."""
    rep = ParityReport()
    rep.loss_diff = float((a["loss"].double() - b["loss"].double()).abs())
    for k, vb in b.items():
        if not k.startswith("grad."):
            continue
        if k not in a:
            rep.missing.append(k)
            continue
        rel = float((a[k].double() - vb.double()).abs().max() / (vb.double().abs().max() + 1e-12))
        rep.per_tensor[k] = rel
        if rel > rep.worst_grad_rel:
            rep.worst_grad_rel, rep.worst_grad_name = rel, k
    return rep


# ---- command line: the parity workflow between a PyTorch script and this framework ------------------------------------------------
def dump_step(spec, params: Dict[str, torch.Tensor], ids: torch.Tensor, targets: torch.Tensor, python_names: bool = False) -> Dict[str, torch.Tensor]:
    """``{"loss", "grad.<name>"...}`` of one forward+backward of the autograd model in fp32 (the step dump the parity report
    compares, pg-compat/src/loader.rs:230-360). With ``python_names`` the gradients are keyed as the Python records name their
    parameters, so the dump lines up with one written from ``model.named_parameters()``."""
    from ..models.runner import OracleRunner
    loss, grads = OracleRunner(spec.model, {k: v.float() for k, v in params.items()}).loss_and_grads(ids, targets)
    if python_names:
        grads = to_python_state_dict(spec.model, grads)
    out = {"loss": loss.reshape(1).float()}
    out.update({f"grad.{k}": v.float().contiguous() for k, v in grads.items()})
    return out


def main(argv=None) -> int:
    """``python -m parameter_golf_b200.utils.interop <command>``:

    * ``import --family F --state model.safetensors --artifact out.pgrs``: a Python-record ``state_dict`` to a quantised artifact;
    * ``export --family F --artifact a.pgrs --state out.safetensors``: an artifact's (de-quantised) weights under the Python names;
    * ``dump-step --family F --state model.safetensors --tokens t.bin --out step.safetensors [--python-names]``: loss and gradients
      of one step on the first ``batch x (seq + 1)`` tokens of a shard;
    * ``compare a.safetensors b.safetensors``: the parity report (loss |a - b| <= 1e-3, worst gradient relative error <= 0.02);
      exit code 1 when it fails."""
    import argparse
    import sys
    ap = argparse.ArgumentParser(prog="parameter_golf_b200.utils.interop")
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("import", "export", "dump-step"):
        p = sub.add_parser(name)
        p.add_argument("--family", default="record_11l")
        p.add_argument("--spec")
        p.add_argument("--state", required=True)
        p.add_argument("overrides", nargs="*")
        if name != "dump-step":
            p.add_argument("--artifact", required=True)
        else:
            p.add_argument("--tokens", required=True)
            p.add_argument("--out", required=True)
            p.add_argument("--batch", type=int, default=2)
            p.add_argument("--seq-len", type=int, default=0)
            p.add_argument("--python-names", action="store_true")
    p = sub.add_parser("compare")
    p.add_argument("a")
    p.add_argument("b")
    a = ap.parse_args(argv)
    if a.cmd == "compare":
        rep = compare_step_dumps(read_safetensors(a.a), read_safetensors(a.b))
        print(f"loss_diff={rep.loss_diff:.3e}\nworst_grad_rel={rep.worst_grad_rel:.3e}\nworst_grad_name={rep.worst_grad_name}\n"
              f"missing={','.join(rep.missing)}\nloss_atol={LOSS_ATOL}\ngrad_max_rel={GRAD_MAX_REL}\nparity_ok={str(rep.ok).lower()}")
        for k, v in sorted(rep.per_tensor.items(), key=lambda kv: -kv[1])[:10]:
            print(f"rel.{k}={v:.3e}")
        return 0 if rep.ok else 1
    from ..spec import RunSpec, family_preset
    spec = RunSpec.load(a.spec) if a.spec else family_preset(a.family)
    spec.apply_overrides(a.overrides)
    spec.validate()
    if a.cmd == "import":
        from ..quant.export import export_model
        params = from_python_state_dict(spec.model, read_safetensors(a.state))
        blob = export_model(spec, params, a.artifact)
        print(f"artifact_bytes={len(blob)}\nvariant_fingerprint={spec.fingerprint():016x}")
    elif a.cmd == "export":
        from ..quant.export import load_artifact
        with open(a.artifact, "rb") as fh:
            params = load_artifact(fh.read(), spec)
        sd = to_python_state_dict(spec.model, params)
        write_safetensors(a.state, {k: v.float().contiguous() for k, v in sd.items()}, {"variant_fingerprint": f"{spec.fingerprint():016x}"})
        print(f"tensors={len(sd)}")
    else:
        from ..data.shards import open_shard
        params = from_python_state_dict(spec.model, read_safetensors(a.state))
        S = a.seq_len or spec.model.train_seq_len
        toks = torch.from_numpy(np.asarray(open_shard(a.tokens)[: a.batch * S + 1]).astype(np.int64))
        if toks.numel() < a.batch * S + 1:
            print(f"the shard holds {toks.numel()} tokens, {a.batch * S + 1} are needed", file=sys.stderr)
            return 2
        ids, tgt = toks[:-1].reshape(a.batch, S), toks[1:].reshape(a.batch, S)
        dump = dump_step(spec, params, ids, tgt, a.python_names)
        write_safetensors(a.out, dump, {"tokens": str(a.batch * S)})
        print(f"loss={float(dump['loss']):.6f}\ntensors={len(dump)}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
