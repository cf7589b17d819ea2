"""Execution plan: everything a run derives from its validated spec before touching a device.

Counterpart of ``parameter-golf-rs/crates/pg-model/src/plan.rs:91-176`` (`ExecutionPlan::from_run_spec`), `:487-529`
(fingerprint) and ``config.rs:1736-1760`` (`checkpoint_layers`, `estimate_memory`): bank layout, one feature mask per
executed block (a layer that runs twice appears twice), which blocks keep their activations, a byte estimate of the
CUDA engine's device memory for one micro-batch, the quantisation layout and the evaluation plan.

The memory estimate follows the buffers `models.engine.CudaEngine` really allocates (same shapes, same dtypes), so
``estimate.total`` tracks ``torch.cuda.memory_allocated()`` after engine construction to within the allocator's
rounding; a GPU test checks that.
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional, Tuple

from .models import gpt
from .spec import RunSpec

HBM_BYTES_B200 = 180 * 10 ** 9


@dataclass
class BankLayout:
    qo_bank: Tuple[int, int, int]
    kv_bank: Tuple[int, int, int]
    mlp_up_bank: Tuple[int, int, int]
    mlp_down_bank: Tuple[int, int, int]

    def elems(self) -> Dict[str, int]:
        return {k: math.prod(v) for k, v in asdict(self).items()}


@dataclass
class LayerFeatureMask:
    layer: int
    pass_index: int
    xsa: bool
    value_embedding: bool
    recurrent: bool
    parallel_residual: bool
    attn_out_gate: bool
    sparse_attn_gate: bool
    saved: bool              # activations kept for the backward (False: the block is recomputed there)
    unet_role: str           # "encoder" | "decoder" | "none"


@dataclass
class MemoryEstimate:
    params_fp32: int = 0
    grads_fp32: int = 0
    optimizer_state: int = 0
    ema: int = 0
    weights_bf16: int = 0
    activations: int = 0
    backward_scratch: int = 0
    logits: int = 0

    @property
    def total(self) -> int:
        return sum(asdict(self).values())


@dataclass
class ExecutionPlan:
    name: str
    fingerprint: str
    micro_batch_tokens: int
    grad_accum_steps: int
    bank_layout: BankLayout
    layer_schedule: List[LayerFeatureMask]
    saved_mode: str
    memory: MemoryEstimate
    quant_layout: Dict[str, object] = field(default_factory=dict)
    eval_plan: Dict[str, object] = field(default_factory=dict)

    @staticmethod
    def from_run_spec(spec: RunSpec, micro_batch_tokens: Optional[int] = None) -> "ExecutionPlan":
        spec.validate()
        m, t = spec.model, spec.train
        n, d, kv, mlp = m.num_layers, m.model_dim, m.kv_dim, m.mlp_dim
        world = max(t.world_size, 1)
        accum = t.grad_accum_steps if t.grad_accum_steps > 0 else (max(8 // world, 1) if t.backend != "cpu" else 1)
        if micro_batch_tokens is None:
            micro_batch_tokens = max(t.batch_tokens // (world * accum), t.seq_len)
        sched = gpt.layer_schedule(m)
        saved = saved_slots(sched, t.save_layer_acts)
        enc = m.depth // 2
        unet = m.skip_topology == "unet"
        passes: Dict[int, int] = {}
        for l, _ in sched:
            passes[l] = passes.get(l, 0) + 1
        masks = [LayerFeatureMask(layer=l, pass_index=rep, xsa=l in m.xsa_layers(),
                                  value_embedding=m.value_embedding.enabled and l in m.value_embedding.layers,
                                  recurrent=passes[l] > 1, parallel_residual=m.parallel,
                                  attn_out_gate=m.attn_out_gate.enabled, sparse_attn_gate=m.sparse_attn_gate.enabled,
                                  saved=saved[j], unet_role=("encoder" if (j if m.cycled else l) < enc else "decoder") if unet else "none")
                 for j, (l, rep) in enumerate(sched)]
        q, e = spec.quant, spec.eval
        return ExecutionPlan(
            name=spec.name, fingerprint=f"{spec.fingerprint():016x}", micro_batch_tokens=micro_batch_tokens, grad_accum_steps=accum,
            bank_layout=BankLayout((2 * n, d, d), (2 * n, kv, d), (n, gpt.up_rows(m), d), (n, d, mlp)),
            layer_schedule=masks, saved_mode=t.save_layer_acts, memory=estimate_engine_memory(spec, micro_batch_tokens),
            quant_layout={"scheme": q.scheme, "compression": q.compression, "matrix_bits": q.matrix_bits, "embed_bits": q.embed_bits,
                          "gptq_calibration_batches": q.gptq_calibration_batches, "target_artifact_bytes": q.target_artifact_bytes},
            eval_plan={"stride": e.stride, "legal_score_first": e.legal_score_first, "qttt": e.qttt,
                       "adaptation_backend": e.adaptation_backend, "lora_rank": e.lora_rank, "lora_alpha": e.lora_alpha,
                       "chunk_tokens": e.chunk_tokens})

    def summary_lines(self) -> List[str]:
        """``key=value`` lines for the CLI (`python -m parameter_golf_b200.train plan ...`)."""
        mem = self.memory
        out = [f"plan.name={self.name}", f"plan.fingerprint={self.fingerprint}", f"plan.micro_batch_tokens={self.micro_batch_tokens}",
               f"plan.grad_accum_steps={self.grad_accum_steps}", f"plan.blocks={len(self.layer_schedule)}",
               f"plan.saved_mode={self.saved_mode}", f"plan.saved_blocks={sum(x.saved for x in self.layer_schedule)}"]
        out += [f"plan.bank.{k}={'x'.join(map(str, v))}" for k, v in asdict(self.bank_layout).items()]
        out += [f"plan.memory.{k}={v}" for k, v in asdict(mem).items()]
        out += [f"plan.memory.total={mem.total}", f"plan.memory.total_gib={mem.total / 2 ** 30:.2f}",
                f"plan.memory.fraction_of_180GB={mem.total / HBM_BYTES_B200:.4f}"]
        for x in self.layer_schedule:
            flags = [k for k in ("xsa", "value_embedding", "recurrent", "parallel_residual", "attn_out_gate", "sparse_attn_gate", "saved")
                     if getattr(x, k)]
            out.append(f"plan.block.{x.layer}.{x.pass_index}={x.unet_role}:{'+'.join(flags) or '-'}")
        out += [f"plan.quant.{k}={v}" for k, v in self.quant_layout.items()]
        out += [f"plan.eval.{k}={v}" for k, v in self.eval_plan.items()]
        return out


def saved_slots(sched, mode: str) -> List[bool]:
    """The CUDA engine's activation-keeping rule (`CudaEngine._saved_slots`) as a free function of the block schedule."""
    passes: Dict[int, int] = {}
    for l, _ in sched:
        passes[l] = passes.get(l, 0) + 1
    inner = lambda l: 3 <= l <= 8
    mode = str(mode).lower()
    if mode == "all":
        return [True] * len(sched)
    if mode == "none":
        return [False] * len(sched)
    if mode == "edges":
        return [(not inner(l)) and passes[l] == 1 for l, _ in sched]
    if mode == "inner":
        return [inner(l) for l, _ in sched]
    if mode == "recurrent":
        return [passes[l] > 1 for l, _ in sched]
    raise ValueError(f"unknown save_layer_acts mode {mode!r}")



def logit_chunk_rows(T: int, V: int, override: int = 0) -> int:
    """Rows of the output projection the CUDA engine materialises at a time. The full ``[T, V]`` logits are kept when they are
    small (vocabulary 1024: 201 MB per micro-batch); above 2^27 elements (vocabulary 8192 at 98,304 tokens: 1.6 GB) the
    projection, the cross-entropy and the two products that consume its gradient run per chunk of rows, so only
    ``[rows, V]`` ever exists (the reference reaches the same end with a vocabulary-tiled online log-sum-exp,
    ``parameter-golf-rs/crates/pg-kernels/src/gpu_kernels.rs:4241-4386``). ``override`` > 0 forces a chunk size."""
    if override > 0:
        return min(T, max(128, override // 128 * 128))
    if T * V <= (1 << 27):
        return T
    return min(T, max(128, ((1 << 26) // V) // 128 * 128))


def estimate_engine_memory(spec: RunSpec, micro_batch_tokens: int, train: bool = True) -> MemoryEstimate:
    """Bytes of the buffers `CudaEngine` allocates for one micro-batch of ``micro_batch_tokens`` tokens."""
    m, t = spec.model, spec.train
    T = int(micro_batch_tokens)
    n, d, kv, mlp, V, H = m.num_layers, m.model_dim, m.kv_dim, m.mlp_dim, m.vocab_size, m.num_heads
    qkvw = d + 2 * kv
    shapes = gpt.param_shapes(m)
    nparam = sum(math.prod(s) for s in shapes.values())
    bank_elems = sum(math.prod(shapes[k]) for k in gpt.BANKS)
    est = MemoryEstimate()
    est.params_fp32 = 4 * nparam
    # bf16 compute copies: packed QKV, Wo, Wup, Wd, un-scaled Wo / Wd for the scale gradients, tables
    tables = V * d + (0 if m.tie_embeddings else V * d)
    if m.bigram.enabled:
        tables += m.bigram.vocab_size * m.bigram.dim + d * m.bigram.dim
    if m.value_embedding.enabled:
        tables += V * m.value_embedding.dim + len(m.value_embedding.layers) * kv * m.value_embedding.dim
    est.weights_bf16 = 2 * (n * qkvw * d + 2 * n * d * d + n * mlp * d + 2 * n * d * mlp + tables)
    sched = gpt.layer_schedule(m)
    nslots = len(sched)
    if not train:
        nact = 1
    else:
        saved = saved_slots(sched, t.save_layer_acts)
        nact = sum(saved) + (0 if all(saved) else 1)
    gates = int(m.attn_out_gate.enabled) + int(m.sparse_attn_gate.enabled)
    # per activation set: x_in, h, y, x_mid (+ mm unless parallel residual), qkv_pre, qk_post, hu, a, lse, gate outputs
    per_set = 2 * T * d * (4 + (0 if m.parallel else 1)) + 2 * 2 * T * qkvw + 2 * 2 * T * mlp + 4 * T * H
    per_set += gates * (2 * T * d + 4 * T * H)
    act = nact * per_set
    if train:
        xsa_sets = {(j if saved[j] else -1) for j, (l, _) in enumerate(sched) if l in m.xsa_layers()}
        act += len(xsa_sets) * 2 * T * d
    elif m.xsa_last_n > 0:
        act += 2 * T * d
    act += nslots * 2 * T * d                                    # block outputs, always kept
    act += 2 * T * d * (3 + int(m.bigram.enabled))               # e, x0, hf (+ xe)
    if m.bigram.enabled:
        act += 2 * T * m.bigram.dim
    if m.value_embedding.enabled:
        act += 2 * T * m.value_embedding.dim
    act += 8 * T                                                  # ids, targets
    est.activations = act
    est.logits = 2 * logit_chunk_rows(T, V, t.logit_chunk_rows) * V + 4 * T
    if train:
        est.grads_fp32 = 4 * nparam
        est.optimizer_state = 4 * bank_elems + 2 * 4 * (nparam - bank_elems)          # Muon momentum; AdamW m and v
        # Newton-Schulz workspaces (bf16 X, Gram, polynomial, product per bank) and fp32 staging of the scaled-weight gradients
        est.optimizer_state += 2 * 4 * bank_elems // 2 + 4 * (d * mlp + d * d)
        est.ema = 4 * nparam if t.ema_decay > 0 else 0
        enc = n // 2
        scratch = 2 * T * d * 7 + 2 * T * mlp + 2 * 2 * T * qkvw + 4 * T * H           # dx, dx_mid, d_m, d_z, d_y, d_h, d_x0, d_hu, d_qk_post, d_qkv_pre, dsum
        scratch += 2 * T * d * (max(enc - 1, 0) if m.skip_topology == "unet" else 0)    # U-Net skip gradients
        scratch += 2 * T * d                                                            # d_xe
        if not t.reproducible_backward:
            scratch += 4 * T * d                                                        # fp32 dQ accumulator of the single-pass attention backward
        if m.bigram.enabled:
            scratch += 2 * T * m.bigram.dim
        if gates and not m.parallel:
            scratch += 2 * T * d
        est.backward_scratch = scratch
    return est
