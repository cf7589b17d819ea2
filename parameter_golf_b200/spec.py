"""Run specification: TOML ``RunSpec`` + CLI overrides + ``train_gpt.py`` environment names.

Three configuration surfaces are accepted and merged into one validated, fingerprinted object:

* a TOML file with the same section/key names as the reference's ``RunSpec``
  (``parameter-golf-rs/crates/pg-model/src/spec.rs:137-718``): ``name``, ``mode``,
  ``[model]``, ``[train]``, ``[quant]``, ``[eval]``; every key is optional;
* ``key=value`` overrides (``train.matrix_lr=0.02``) from the command line
  (``parameter-golf-rs/crates/pg-train/src/main.rs:132-208``);
* the environment variables of the Python entrypoint (``train_gpt.py:39-87`` and the record
  scripts' extensions), e.g. ``NUM_LAYERS``, ``TRAIN_BATCH_TOKENS``, ``XSA_LAST_N``.

``RunSpec.validate`` holds the fail-closed rules (``pg-model/src/plan.rs:369-485``) and
``RunSpec.fingerprint`` the 64-bit variant fingerprint stamped into artifacts
(``pg-model/src/plan.rs:487-529``).
"""
from __future__ import annotations

import dataclasses
import json
import os
import tomllib
from dataclasses import dataclass, field, fields, is_dataclass
from typing import Any, Optional

RUN_MODES = ("smoke", "proxy", "record_shaped_proxy", "record")
TRAIN_BACKENDS = ("cpu", "cuda_single", "cuda_single_parity", "cuda_distributed")
DIST_OPT_BACKENDS = ("all_reduce_replicated_muon", "sharded_parallel_muon")
QUANT_SCHEMES = ("none", "gptq_lite_int6", "mixed_int5_int6", "aggressive", "tight_int7_int4", "full_gptq_int6",
                 "int8_zlib", "ternary_b158", "binary_b1")       # int8_zlib: the baseline trainer's per-row int8 + zlib-9 export (train_gpt.py:342-422)
COMPRESSION_MODES = ("none", "zstd22", "lzma9", "pergroup")
CALIBRATION_MODES = ("disabled", "self_generated")
ADAPTATION_BACKENDS = ("none", "cpu_q_only", "gpu_lora_phased", "full_sgd", "lact", "slot", "doc_lora")
NS_PROFILES = ("simple", "quintic", "polar_express")
FAMILIES = (
    "baseline_sp8192", "xsa_all_sp8192", "recurrence_mid_sp8192", "parallel_resid_sp8192",
    "hybrid_competitive_sp8192", "frontier_1855_like",
    # families of this framework, named after the benchmark configurations
    "tiny_cpu", "baseline_9l", "record_11l",
    "ternary_10l",       # the 2026-03-24 ternary record's shape: autograd path only (head_dim 96, ternary QAT)
    "binary_15l",        # the 2026-03-24 binary non-record submission's shape: 15 x 768, 1-bit weights, per-block smear; autograd path only
)


@dataclass
class BigramSpec:
    enabled: bool = False
    vocab_size: int = 2048
    dim: int = 128
    trigram: bool = False        # also add the row hashed from (t-2, t-1, t) of the same table (TRIGRAM of the 2026-03-25 record; autograd path)


@dataclass
class RopeSpec:
    mode: str = "partial"          # none | partial | yarn
    dims: int = 16                 # 0 or head_dim => full rotary
    base: float = 10000.0
    yarn_max_len: int = 2048       # mode = yarn: the context the frequencies are stretched to (YARN_MAX_LEN) ...
    yarn_train_len: int = 1024     # ... from this training length; low frequencies slow down by up to yarn_max_len / yarn_train_len


@dataclass
class ValueEmbeddingSpec:
    enabled: bool = False
    dim: int = 128
    layers: list = field(default_factory=lambda: [9, 10])


@dataclass
class RecurrenceSpec:
    enabled: bool = False
    start_layer: int = 0
    repeat_layers: int = 0
    # Cycled form (autograd path only; records/track_non_record_16mb/2026-03-21_DepthRecurrence_MixedPrecisionQuant/train_gpt.py:831-863):
    # with effective_depth > num_layers the num_layers unique blocks run in the order 0, 1, ..., n-1, 0, 1, ... for
    # effective_depth virtual layers; the U-Net split, its skip weights and xsa_last_n then count virtual layers.
    effective_depth: int = 0
    repeats: int = 2                  # passes of each recurrent block in a row; other values than 2 run on the autograd path only
                                      # (TRAINING_DEPTH_RECURRENCE of the ternary record repeats every block)
    depth_lora_rank: int = 0          # > 0: a low-rank correction of the query and value projections per virtual layer (its DepthLoRA)


@dataclass
class ParallelResidualSpec:
    enabled: bool = False
    split_attention_mlp: bool = True      # the MLP reads the block input beside the attention only when both are set
                                          # (pg-model/src/spec.rs:421-422); the reference's own default is false and its presets set true


@dataclass
class CaseOpsSpec:
    """Case-operator tokenisation of the late SP8192 stack: the validation bytes cannot be read off the token surfaces, so
    bits-per-byte needs the per-position byte sidecar (``eval.caseops_byte_sidecar_pattern``)."""
    enabled: bool = False
    byte_sidecar: bool = False


@dataclass
class AttnOutGateSpec:
    enabled: bool = False
    width: int = 12


@dataclass
class SparseAttnGateSpec:
    enabled: bool = False
    width: int = 12
    scale: float = 1.0


@dataclass
class ModelSpec:
    family: str = "record_11l"
    vocab_size: int = 1024
    num_layers: int = 11
    model_dim: int = 512
    num_heads: int = 8
    num_kv_heads: int = 4
    mlp_mult: float = 3.0
    activation: str = "leaky_relu_sq"     # relu_sq | leaky_relu_sq | swiglu (autograd path only: mlp_up_bank holds gate rows then up rows)
    leaky_slope: float = 0.5
    train_seq_len: int = 2048
    eval_seq_len: int = 2048
    bigram: BigramSpec = field(default_factory=BigramSpec)
    xsa_last_n: int = 0
    value_embedding: ValueEmbeddingSpec = field(default_factory=ValueEmbeddingSpec)
    skip_topology: str = "unet"           # none | unet
    recurrence: RecurrenceSpec = field(default_factory=RecurrenceSpec)
    parallel_residual: ParallelResidualSpec = field(default_factory=ParallelResidualSpec)
    attn_out_gate: AttnOutGateSpec = field(default_factory=AttnOutGateSpec)
    caseops: CaseOpsSpec = field(default_factory=CaseOpsSpec)
    sparse_attn_gate: SparseAttnGateSpec = field(default_factory=SparseAttnGateSpec)
    rope: RopeSpec = field(default_factory=RopeSpec)
    smear_gate: bool = False
    smear_gate_boundary_token_id: Optional[int] = None
    logit_softcap: float = 30.0
    qk_gain_init: float = 1.5
    ln_scale: bool = False
    tie_embeddings: bool = True
    tied_embed_init_std: float = 0.005
    embed_init: str = "normal"            # normal | overtone: the tied table's singular values reshaped to s_1 / sqrt(k)
    resid_mix_init: str = "identity"      # identity (x, no x0) | phase: sigmoid(3 (l / (n-1) - 1/2)) on x and the rest on x0, per layer
    compute_precision: str = "bf16_tensor_core"  # f32 / f32_tf32 (CPU oracle) | bf16_tensor_core
    attention_backend: str = "native"     # recorded, never dispatched on: there is one attention implementation per backend. The reference's
                                          # names (naive_f32 | flash_f32 | cudnn_sdpa_bf16) are accepted so that its spec files load
    # Optional ideas of the Python records that their own runs leave off (train_gpt.py:70-92 of the 2026-03-23 record). They run on
    # the autograd path (train.backend = cpu); the CUDA engine rejects them at validation.
    value_residual: bool = False          # v <- lambda_0 * v(first layer) + lambda_1 * v in every later layer, lambda learned per layer
    mtp_num_heads: int = 0                # extra output heads that predict the tokens 2, 3, ... ahead, training only, not exported
    mtp_loss_weight: float = 0.2
    dtg: bool = False                     # per-block scalar gate on the block's update, sigmoid(w . x_in + b) read from the detached input (DTG_ENABLED)
    softcap_kind: str = "tanh"            # tanh | poly5 (the ternary record's degree-5 polynomial cap)
    z_loss_weight: float = 0.0            # training only: this weight times the mean squared log-partition is added to the loss
    embed_dim: int = 0                    # > 0: factored tied embedding, tok_emb [V, embed_dim] with learned projections to and from
                                          # model_dim (the ternary record's 254-wide bottleneck); 0 = tok_emb [V, model_dim]
    qat_kind: str = "int6"                # what QAT simulates in the bank matrices: int6 rows, or ternary / binary codes with one scale per group
    qat_noise_qmax: int = 127             # qat_kind = noise: uniform noise of one quantisation step (row max / qmax) on the blocks that run more
                                          # than once (all blocks when none does), with gradients flowing through it
    qat_ternary_group: int = 128          # qat_kind = ternary | binary: input columns per scale (keep equal to quant.ternary_group)
    normed_out_proj: bool = False         # RMSNorm on the inputs of the attention output and MLP down projections (the ternary and
                                          # binary submissions' "normed" linear layers, which see un-normalised activations)
    gated_attention: bool = False         # per-head sigmoid(W_h . x + b_h) on the attention output, full-width input, W from zero and b = 4
                                          # (GATED_ATTENTION of the 2026-03-23 record; autograd path)
    vocab_bias: bool = False              # a learned bias per vocabulary entry added to the logits before the soft-cap (zero at the start)
    block_smear: bool = False             # every block ends with x + tanh(g) * (causal running mean of x - x), g[d] learned per block from zero
    fp8_qat: bool = False                 # while QAT is on, the small 2-D float tensors (bigram / value-embedding tables and
                                          # projections, an untied head) go through an FP8 e4m3 round trip (FP_STORAGE=FP8)

    @property
    def head_dim(self) -> int:
        return self.model_dim // self.num_heads

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def mlp_dim(self) -> int:
        return int(self.mlp_mult * self.model_dim + 1e-6)        # MLP_HIDDEN / model_dim * model_dim must give MLP_HIDDEN back

    @property
    def rope_dims(self) -> int:
        if self.rope.mode == "none":
            return 0
        d = self.rope.dims
        return self.head_dim if d <= 0 or d >= self.head_dim else d

    @property
    def cycled(self) -> bool:
        return self.recurrence.enabled and self.recurrence.effective_depth > 0

    @property
    def depth(self) -> int:
        """Virtual layers: block executions whose position counts for the U-Net split and the per-depth adapters."""
        return self.recurrence.effective_depth if self.cycled else self.num_layers

    @property
    def parallel(self) -> bool:
        """Attention and MLP of a block both read the block input (split parallel residual)."""
        return self.parallel_residual.enabled and self.parallel_residual.split_attention_mlp

    def for_evaluation(self, depth_recurrence: int = 0) -> "ModelSpec":
        """The model as the evaluator runs it: a copy whose blocks all repeat ``depth_recurrence`` times when that is > 1."""
        if depth_recurrence <= 1 or self.cycled:
            return self
        import copy
        m = copy.deepcopy(self)
        m.recurrence.enabled, m.recurrence.start_layer, m.recurrence.repeat_layers, m.recurrence.repeats = True, 0, self.num_layers, depth_recurrence
        return m

    def xsa_layers(self) -> list:
        """Blocks with the exclusive-self-attention step: the last xsa_last_n layers; in the cycled form every block that runs as
        one of the last xsa_last_n virtual layers (the flag sits on the block, so it holds in all of that block's passes)."""
        if self.cycled:
            return sorted({v % self.num_layers for v in range(max(0, self.depth - self.xsa_last_n), self.depth)})
        return list(range(max(0, self.num_layers - self.xsa_last_n), self.num_layers))


@dataclass
class TrainSpec:
    backend: str = "cpu"
    distributed_optimizer_backend: str = "all_reduce_replicated_muon"
    batch_tokens: int = 524_288
    seq_len: int = 2048
    grad_accum_steps: int = 0           # 0 = automatic: 8 // world_size on CUDA backends, 1 on cpu
    # Curriculum of the ternary record (train_gpt_cuda_ternary.py:1210-1289; cpu backend only, the CUDA engine's buffers have one
    # shape): start with shorter sequences and / or a smaller global batch and switch to seq_len / batch_tokens once the given
    # fraction of the wall-clock budget (of the step count without a cap) has passed. 0 = off.
    seq_len_start: int = 0
    seq_schedule_fraction: float = 0.33
    batch_tokens_start: int = 0
    batch_schedule_fraction: float = 0.33
    train_data_pattern: Optional[str] = None
    validation_data_pattern: Optional[str] = None
    rank: int = 0
    world_size: int = 1
    artifact_path: str = "artifact.pgrs"
    prime_steps: int = 0                # cpu backend (ignored with a log line on the CUDA backends): run this many steps first, then put weights, optimizer state, data position and
                                        # random state back (the Python trainers' WARMUP_STEPS, which primes compiled kernels without
                                        # training, train_gpt.py:937-961; the CUDA engine compiles nothing at run time)
    fast_bank_updates: bool = False     # accepted for the reference's spec files; bank updates are always the fused kernels here
    warmup_steps: int = 0
    total_iterations: int = 9000
    warmdown_iters: int = 3500
    warmdown_frac: float = 0.0
    min_lr_scale: float = 0.0
    wallclock_warmdown: bool = True
    max_wallclock_seconds: float = 600.0
    record_max_ms_per_step: float = 130.0   # record mode fails closed when the measured step time is above this; 0 disables (PG_RECORD_MAX_MS_PER_STEP)
    timing_skip_steps: int = 0              # steps left out of the measured step time (start-up, PG_RECORD_TIMING_SKIP_STEPS)
    matrix_lr: float = 0.025
    matrix_optimizer: str = "muon"      # muon | adamw (cpu backend: the banks go to AdamW at adam_matrix_lr; MATRIX_OPTIMIZER / ADAM_LR of the ternary script)
    adam_matrix_lr: float = 0.05
    scalar_lr: float = 0.025
    embed_lr: float = 0.6
    tied_embed_lr: float = 0.035
    head_lr: float = 0.008
    muon_momentum: float = 0.99
    muon_momentum_warmup_start: float = 0.92
    muon_momentum_warmup_steps: int = 1500
    muon_wd: float = 0.04
    muon_ns_profile: str = "quintic"
    muon_ns_steps: int = 5
    adam_wd: float = 0.04
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    adam_eps: float = 1e-8
    grad_clip_norm: float = 0.3
    ema_decay: float = 0.997
    ema_start_fraction: float = 0.0     # cpu backend: the average starts (from the weights of that moment) once this fraction of the
                                        # wall-clock budget, or of the steps without a cap, has passed (EMA_START_FRACTION of the ternary record)
    swa_enabled: bool = True
    swa_every: int = 50
    swa_threshold: float = 0.2
    lawa_enabled: bool = False     # latest-weight averaging: the last lawa_k snapshots, one every lawa_freq steps, replace the EMA weights
    lawa_k: int = 10
    lawa_freq: int = 100
    late_qat_threshold: float = 0.15
    qat_fraction: float = 0.0           # > 0: QAT switches on for the last fraction of the wall-clock budget (of the steps without a cap),
                                        # whatever the learning-rate scale (QAT_FRACTION of the depth-recurrence submission)
    qat_enabled: bool = False
    seed: int = 1337
    val_loss_every: int = 0
    train_log_every: int = 200
    churn_log_every: int = 0            # cpu backend, ternary / binary QAT: every N steps log the fraction of bank codes that changed since
                                        # the last such line (CHURN_LOG_EVERY of the 2026-03-24 scripts: how settled the discrete weights are)
    val_batch_size: int = 524_288
    grad_wire_dtype: str = "bf16"       # wire dtype of bank-gradient reduce-scatter
    cuda_graph: bool = False            # replay the micro-batch forward+backward from a captured CUDA graph
    reproducible_backward: bool = False # CUDA engine: bit-reproducible gradient kernels (two-kernel attention backward) instead of the faster fp32 red.add forms
    save_layer_acts: str = "all"        # CUDA engine activation checkpointing: all | edges | inner | recurrent | none
    logit_chunk_rows: int = 0           # CUDA engine: rows of logits materialised at a time (0 = automatic: everything unless [T, V] exceeds 2^27 elements)
    checkpoint_every: int = 0
    checkpoint_path: Optional[str] = None
    resume_from: Optional[str] = None
    # complementary training: loss weight per (previous token, target) pair from bigram statistics; 0 disables
    complementary_alpha: float = 0.0
    complementary_shape: str = "floored"        # "linear" | "power" | "floored"
    complementary_power: float = 2.0
    complementary_floor: float = 0.2
    complementary_min_w: float = 0.25
    complementary_stats_tokens: int = 4_194_304  # training tokens counted into the bigram table at start-up
    complementary_stats_path: Optional[str] = None   # load the table from this file if it exists, else build and save it


@dataclass
class LqerSpec:
    enabled: bool = False
    rank: int = 4
    top_k: int = 0
    a_bits: int = 8
    b_bits: int = 8
    group_size: int = 0
    asymmetric: bool = False


@dataclass
class QuantSpec:
    scheme: str = "gptq_lite_int6"
    calibration: str = "disabled"
    prune_keep_ratio: Optional[float] = None
    lqer: LqerSpec = field(default_factory=LqerSpec)
    compression: str = "zstd22"
    code_storage: str = "bit_packed"    # bit_packed: codes packed LSB-first at their bit width (the Rust engine's artifact);
                                        # bytes: one int8 per code (the Python records' container: the entropy coder then sees the code distribution)
    prune_to_target: bool = True        # zero the cheapest +-1 codes until artifact + code fit target_artifact_bytes
    prune_max_magnitude: int = 1        # widen the candidates to |code| <= this when the +-1 codes are not enough
    ternary_group: int = 128            # scheme ternary_b158 (and model.qat_kind = ternary): input columns per scale
    float_storage: str = "f16"          # f16 | fp8: how the 2-D float tensors that are not quantised to integer codes are stored
                                        # (fp8 = e4m3, one byte per element; 1-D control tensors stay f16)
    matrix_bits: int = 6
    embed_bits: int = 8                 # 16 = keep the (tied) embedding table as fp16 instead of integer codes
    coarse_layers: list = field(default_factory=list)   # blocks whose integer codes are rounded to multiples of coarse_step
    coarse_step: int = 1                # (INT4_LAYERS / INT4_STEP of the 10-layer mixed-precision record: 4 turns int8 codes into 64 levels)
    attn_gate_bits: int = 8
    mlp_clip_sigmas: float = 0.0
    attn_clip_sigmas: float = 0.0
    embed_clip_sigmas: float = 0.0
    gptq_calibration_batches: int = 64
    gptq_block_size: int = 128
    gptq_damping: float = 0.01
    gptq_temperature: float = 0.8
    target_artifact_bytes: int = 16_000_000


@dataclass
class EvalSpec:
    stride: int = 64
    legal_score_first: bool = False
    qttt: bool = False
    adaptation_backend: str = "none"
    lora_rank: int = 16
    lora_alpha: float = 16.0
    phased_ttt_prefix_docs: int = 0
    phased_ttt_phases: int = 1
    phased_ttt_weight_decay: float = 0.0
    ttt_beta2: float = 0.99            # carried for the reference's spec files and audit line; the adapter update is SGD with weight decay
    chunk_tokens: int = 32768
    tokenizer_vocab_path: Optional[str] = None
    caseops_byte_sidecar_pattern: Optional[str] = None
    max_tokens: Optional[int] = None
    batch_windows: int = 32
    ttt_lr: float = 0.002
    ttt_epochs: int = 1
    ttt_momentum: float = 0.9
    ttt_batch_seqs: int = 32
    ttt_grad_clip: float = 1.0
    ttt_freeze_blocks: int = 0
    max_eval_seconds: float = 600.0
    temperature: float = 1.0           # capped logits are divided by this when scoring (autograd runner); `find_temperature` picks it
    temperature_grid: list = field(default_factory=lambda: [0.90, 0.95, 1.00, 1.05, 1.10])
    depth_recurrence: int = 0          # > 1: the autograd evaluator runs every block this many times in a row, whatever the training
                                       # schedule was (EVAL_DEPTH_RECURRENCE of the ternary script)
    auto_temperature: bool = False     # trainer, cpu backend: pick the temperature from the grid on training tokens before the final evaluation (TEMP_SCALING)
    temperature_calibration_tokens: int = 65536       # training tokens the grid is scored on
    byte_table_seed: int = 20240520
    # adaptation_backend = doc_lora: documents (cut at doc_boundary_token_id) scored in isolation, chunk by chunk, with adapters
    # per document trained by one Adam step after each scored chunk (TTT_LORA_RANK / TTT_LORA_LR / TTT_CHUNK_SIZE / TTT_BATCH_SIZE)
    doc_lora_rank: int = 8             # 0 = no adapters: plain document-isolated, strided scoring
    doc_lora_lr: float = 0.01
    doc_chunk_size: int = 256
    doc_batch_size: int = 64
    doc_boundary_token_id: int = 1


@dataclass
class RunSpec:
    name: str = "run"
    model: ModelSpec = field(default_factory=ModelSpec)
    train: TrainSpec = field(default_factory=TrainSpec)
    quant: QuantSpec = field(default_factory=QuantSpec)
    eval: EvalSpec = field(default_factory=EvalSpec)
    mode: str = "smoke"
    allow_unsupported_variants: bool = False

    # ---- construction -------------------------------------------------------------------
    @staticmethod
    def from_dict(d: dict) -> "RunSpec":
        """A spec from a (possibly partial) nested dictionary. Keys that are absent keep the values of the family the dictionary
        names in ``model.family``, or of ``baseline_sp8192`` when it names none: the reference fills missing keys from
        ``RunSpec::for_family(BaselineSp8192)`` (pg-model/src/spec.rs:693-697 with ``#[serde(default)]``), and its shipped spec
        files rely on that."""
        family = (d.get("model") or {}).get("family", "baseline_sp8192")
        if family not in FAMILIES:
            raise ValueError(f"unknown model.family {family!r}; known: {FAMILIES}")
        return _overlay(family_preset(family), d)

    @staticmethod
    def load(path: str) -> "RunSpec":
        with open(path, "rb") as f:
            return RunSpec.from_dict(tomllib.load(f))

    @staticmethod
    def for_family(family: str) -> "RunSpec":
        return family_preset(family)

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)

    def describe_keys(self) -> list:
        """Every ``section.key`` this spec accepts, with its type name and current value, in declaration order: the list a
        ``section.key=value`` override or a TOML file may use."""
        out = []

        def walk(obj, prefix):
            for f in dataclasses.fields(obj):
                v = getattr(obj, f.name)
                if dataclasses.is_dataclass(v):
                    walk(v, prefix + f.name + ".")
                else:
                    tname = f.type if isinstance(f.type, str) else getattr(f.type, "__name__", str(f.type))
                    out.append((prefix + f.name, tname, v))
        walk(self, "")
        return out

    @staticmethod
    def env_names() -> dict:
        """``train_gpt.py`` environment variable name -> the spec key(s) `apply_env` sets from it, read off `apply_env` itself
        so that the list cannot drift from the code."""
        import inspect
        import re
        alias = {"m": "model", "t": "train", "q": "quant", "e": "eval"}
        names: dict = {}
        current = None
        for line in inspect.getsource(RunSpec.apply_env).splitlines():
            hit = re.search(r'has\("([A-Z0-9_]+)"\)', line)
            if hit:
                current = hit.group(1)
                names.setdefault(current, [])
            if current:
                for var, key in re.findall(r"\b([mtqe])\.([a-z_][a-z0-9_.]*)\s*=(?!=)", line):
                    k = f"{alias[var]}.{key}"
                    if k not in names[current]:
                        names[current].append(k)
                if re.search(r"\bself\.name\s*=", line) and "name" not in names[current]:
                    names[current].append("name")
            if hit and ":" in line.split("has(")[1] and not line.rstrip().endswith(":"):
                current = None              # one-line form: the assignment was on the same line
        return names

    def to_toml(self) -> str:
        return _to_toml(self.to_dict())

    def apply_overrides(self, overrides: list) -> "RunSpec":
        """Apply ``section.key=value`` strings (dots descend into sub-tables)."""
        for ov in overrides:
            if "=" not in ov:
                raise ValueError(f"override must be key=value: {ov!r}")
            key, val = ov.split("=", 1)
            obj: Any = self
            parts = key.strip().split(".")
            for p in parts[:-1]:
                if not hasattr(obj, p):
                    raise KeyError(f"unknown spec section {p!r} in {key!r}")
                obj = getattr(obj, p)
            leaf = parts[-1]
            if not hasattr(obj, leaf):
                raise KeyError(f"unknown spec key {key!r}")
            setattr(obj, leaf, _coerce(val.strip(), getattr(obj, leaf), _field_type(obj, leaf)))
        return self

    def apply_env(self, env: Optional[dict] = None) -> "RunSpec":
        """Overlay the ``train_gpt.py`` environment names (only the ones that are set)."""
        env = os.environ if env is None else env
        m, t, q, e = self.model, self.train, self.quant, self.eval

        def has(k):
            return k in env and env[k] != ""

        def I(k):
            return int(env[k])

        def F(k):
            return float(env[k])

        def B(k):
            return bool(int(env[k]))

        if has("RUN_ID"): self.name = env["RUN_ID"]
        if has("DATA_PATH"):
            t.train_data_pattern = os.path.join(env["DATA_PATH"], "fineweb_train_*.bin")
            t.validation_data_pattern = os.path.join(env["DATA_PATH"], "fineweb_val_*.bin")
        if has("TOKENIZER_PATH"): e.tokenizer_vocab_path = env["TOKENIZER_PATH"]
        if has("SEED"): t.seed = I("SEED")
        if has("VAL_BATCH_SIZE"): t.val_batch_size = I("VAL_BATCH_SIZE")
        if has("VAL_LOSS_EVERY"): t.val_loss_every = I("VAL_LOSS_EVERY")
        if has("TRAIN_LOG_EVERY"): t.train_log_every = I("TRAIN_LOG_EVERY")
        if has("CHURN_LOG_EVERY"): t.churn_log_every = I("CHURN_LOG_EVERY")
        if has("ITERATIONS"): t.total_iterations = I("ITERATIONS")
        if has("WARMDOWN_ITERS"): t.warmdown_iters = I("WARMDOWN_ITERS")
        if has("WARMDOWN_FRACTION"): t.warmdown_frac = F("WARMDOWN_FRACTION")
        if has("WARMDOWN_FRAC"): t.warmdown_frac = F("WARMDOWN_FRAC")
        if has("GRAD_ACCUM_STEPS"): t.grad_accum_steps = I("GRAD_ACCUM_STEPS")
        if has("SEQ_LEN_START"): t.seq_len_start = I("SEQ_LEN_START")
        if has("SEQ_SCHEDULE_FRACTION"): t.seq_schedule_fraction = F("SEQ_SCHEDULE_FRACTION")
        if has("BATCH_TOKENS_START"): t.batch_tokens_start = I("BATCH_TOKENS_START")
        if has("BATCH_SCHEDULE_FRACTION"): t.batch_schedule_fraction = F("BATCH_SCHEDULE_FRACTION")
        if has("WARMUP_STEPS"):
            # in the Python trainers these are priming steps whose effect is undone, not a learning-rate warm-up
            # (train.warmup_steps is the reference engine's linear warm-up and is set from TOML / CLI only)
            t.prime_steps = I("WARMUP_STEPS")
        if has("TRAIN_BATCH_TOKENS"): t.batch_tokens = I("TRAIN_BATCH_TOKENS")
        if has("TRAIN_SEQ_LEN"): t.seq_len = m.train_seq_len = I("TRAIN_SEQ_LEN")
        if has("EVAL_SEQ_LEN"): m.eval_seq_len = I("EVAL_SEQ_LEN")
        if has("EVAL_STRIDE"): e.stride = I("EVAL_STRIDE")
        if has("MAX_WALLCLOCK_SECONDS"): t.max_wallclock_seconds = F("MAX_WALLCLOCK_SECONDS")
        if has("QK_GAIN_INIT"): m.qk_gain_init = F("QK_GAIN_INIT")
        if has("VOCAB_SIZE"): m.vocab_size = I("VOCAB_SIZE")
        if has("NUM_LAYERS"): m.num_layers = I("NUM_LAYERS")
        if has("NUM_KV_HEADS"): m.num_kv_heads = I("NUM_KV_HEADS")
        if has("MODEL_DIM"): m.model_dim = I("MODEL_DIM")
        if has("NUM_HEADS"): m.num_heads = I("NUM_HEADS")
        if has("MLP_MULT"): m.mlp_mult = F("MLP_MULT")
        if has("MLP_HIDDEN") and I("MLP_HIDDEN") > 0: m.mlp_mult = I("MLP_HIDDEN") / m.model_dim
        if has("ACTIVATION"):
            m.activation = {"relu2": "relu_sq", "relu_sq": "relu_sq", "leaky_relu_sq": "leaky_relu_sq", "swiglu": "swiglu"}.get(env["ACTIVATION"].lower(), env["ACTIVATION"].lower())
        if has("SMEAR"): m.block_smear = B("SMEAR")
        if has("BITNET_GROUP_SIZE"): m.qat_ternary_group = q.ternary_group = I("BITNET_GROUP_SIZE")
        if has("TIE_EMBEDDINGS"): m.tie_embeddings = B("TIE_EMBEDDINGS")
        if has("ROPE_BASE"): m.rope.base = F("ROPE_BASE")
        if has("ROPE_DIMS"): m.rope.dims = I("ROPE_DIMS")
        if has("ROPE_TYPE"): m.rope.mode = "yarn" if env["ROPE_TYPE"].lower() == "yarn" else m.rope.mode
        if has("YARN_MAX_LEN"): m.rope.yarn_max_len = I("YARN_MAX_LEN")
        if has("LOGIT_SOFTCAP"): m.logit_softcap = F("LOGIT_SOFTCAP")
        if has("EMBED_LR"): t.embed_lr = F("EMBED_LR")
        if has("HEAD_LR"): t.head_lr = F("HEAD_LR")
        if has("TIED_EMBED_LR"): t.tied_embed_lr = F("TIED_EMBED_LR")
        if has("TIED_EMBED_INIT_STD"): m.tied_embed_init_std = F("TIED_EMBED_INIT_STD")
        if has("MATRIX_LR"): t.matrix_lr = F("MATRIX_LR")
        if has("MATRIX_OPTIMIZER"): t.matrix_optimizer = "adamw" if env["MATRIX_OPTIMIZER"].lower().startswith("adam") else "muon"
        if has("ADAM_LR"): t.adam_matrix_lr = F("ADAM_LR")
        if has("SCALAR_LR"): t.scalar_lr = F("SCALAR_LR")
        if has("MUON_MOMENTUM"): t.muon_momentum = F("MUON_MOMENTUM")
        if has("MUON_BACKEND_STEPS"): t.muon_ns_steps = I("MUON_BACKEND_STEPS")
        if has("PG_MUON_NS_PROFILE"): t.muon_ns_profile = _ns_profile_name(env["PG_MUON_NS_PROFILE"])
        if has("PG_GPU_MUON_NS_PROFILE"): t.muon_ns_profile = _ns_profile_name(env["PG_GPU_MUON_NS_PROFILE"])
        if has("MUON_MOMENTUM_WARMUP_START"): t.muon_momentum_warmup_start = F("MUON_MOMENTUM_WARMUP_START")
        if has("MUON_MOMENTUM_WARMUP_STEPS"): t.muon_momentum_warmup_steps = I("MUON_MOMENTUM_WARMUP_STEPS")
        if has("BETA1"): t.adam_beta1 = F("BETA1")
        if has("BETA2"): t.adam_beta2 = F("BETA2")
        if has("ADAM_EPS"): t.adam_eps = F("ADAM_EPS")
        if has("GRAD_CLIP_NORM"): t.grad_clip_norm = F("GRAD_CLIP_NORM")
        if has("MUON_WD"): t.muon_wd = F("MUON_WD")
        if has("ADAM_WD"): t.adam_wd = F("ADAM_WD")
        if has("EMA_DECAY"): t.ema_decay = F("EMA_DECAY")
        if has("EMA") and not B("EMA"): t.ema_decay = 0.0
        if has("EMA_START_FRACTION"): t.ema_start_fraction = F("EMA_START_FRACTION")
        if has("SWA_ENABLED"): t.swa_enabled = B("SWA_ENABLED")
        if has("SWA_EVERY"): t.swa_every = I("SWA_EVERY")
        if has("LAWA_ENABLED"): t.lawa_enabled = B("LAWA_ENABLED")
        if has("LAWA_K"): t.lawa_k = I("LAWA_K")
        if has("LAWA_FREQ"): t.lawa_freq = I("LAWA_FREQ")
        if has("QAT_ENABLED"): t.qat_enabled = B("QAT_ENABLED")
        if has("FP_STORAGE"):
            fp8 = env["FP_STORAGE"].strip().upper() == "FP8"
            q.float_storage = "fp8" if fp8 else "f16"
            m.fp8_qat = fp8
        if has("LATE_QAT_THRESHOLD"): t.late_qat_threshold = F("LATE_QAT_THRESHOLD")
        if has("BIGRAM_VOCAB_SIZE"):
            m.bigram.vocab_size = I("BIGRAM_VOCAB_SIZE")
            m.bigram.enabled = m.bigram.vocab_size > 0
        if has("BIGRAM_DIM"): m.bigram.dim = I("BIGRAM_DIM")
        # spellings other record scripts use for the same settings
        if has("ADAM_WEIGHT_DECAY"): t.adam_wd = F("ADAM_WEIGHT_DECAY")
        if has("BIGRAM_HASH_BUCKETS"):
            m.bigram.vocab_size = I("BIGRAM_HASH_BUCKETS")
            m.bigram.enabled = m.bigram.vocab_size > 0
        if has("BIGRAM_HASH_DIM"): m.bigram.dim = I("BIGRAM_HASH_DIM")
        if has("EMA_ENABLED") and not B("EMA_ENABLED"): t.ema_decay = 0.0
        if has("EVAL_BATCH_SEQS"): e.batch_windows = I("EVAL_BATCH_SEQS")
        if has("SW_EVAL_BATCH"): e.batch_windows = I("SW_EVAL_BATCH")
        if has("FP16_EMBED_EXPORT") and B("FP16_EMBED_EXPORT"): q.embed_bits = 16
        if has("INT6_LAYER_START") and has("INT6_LAYER_END") and I("INT6_LAYER_START") >= 0:
            q.coarse_layers = list(range(I("INT6_LAYER_START"), I("INT6_LAYER_END")))      # int8 codes of these blocks rounded to 64 levels
            q.coarse_step = 4
        if has("QAT_THRESHOLD"): t.late_qat_threshold = F("QAT_THRESHOLD")
        if has("LATE_QAT") and not B("LATE_QAT"): t.late_qat_threshold = 0.0
        if has("SWA_START_FRAC"): t.swa_threshold = F("SWA_START_FRAC")
        if has("USE_SMEARGATE"): m.smear_gate = B("USE_SMEARGATE")
        if has("USE_ZSTD"): q.compression = "zstd22" if B("USE_ZSTD") else q.compression
        if has("LORA_RANK"): e.doc_lora_rank = I("LORA_RANK")
        if has("LORA_LR"): e.doc_lora_lr = F("LORA_LR")
        if has("XSA_LAST_N"): m.xsa_last_n = I("XSA_LAST_N")
        if has("GATED_ATTENTION"): m.gated_attention = B("GATED_ATTENTION")
        if has("TRIGRAM"): m.bigram.trigram = B("TRIGRAM")
        if has("QAT_FRACTION"): t.qat_fraction = F("QAT_FRACTION")
        if has("MUON_WEIGHT_DECAY"): t.muon_wd = F("MUON_WEIGHT_DECAY")
        if has("MTP_HEADS"): m.mtp_num_heads = I("MTP_HEADS")
        if has("TEMP_SCALING"): e.auto_temperature = B("TEMP_SCALING")
        if has("EVAL_DEPTH_RECURRENCE"): e.depth_recurrence = I("EVAL_DEPTH_RECURRENCE")
        if has("SLIDING_EVAL_STRIDE"): e.stride = I("SLIDING_EVAL_STRIDE")
        if has("SLIDING_BATCH_SIZE"): e.batch_windows = I("SLIDING_BATCH_SIZE")
        if has("VAL_MAX_TOKENS") and I("VAL_MAX_TOKENS") > 0: e.max_tokens = I("VAL_MAX_TOKENS")
        if has("TRAINING_DEPTH_RECURRENCE") and I("TRAINING_DEPTH_RECURRENCE") > 1:
            m.recurrence.enabled, m.recurrence.start_layer, m.recurrence.repeat_layers = True, 0, m.num_layers
            m.recurrence.repeats = I("TRAINING_DEPTH_RECURRENCE")
        if has("NUM_UNIQUE_BLOCKS"): m.num_layers = I("NUM_UNIQUE_BLOCKS")
        if has("EFFECTIVE_DEPTH"):
            m.recurrence.effective_depth = I("EFFECTIVE_DEPTH")
            m.recurrence.enabled = m.recurrence.effective_depth > 0
        if has("DEPTH_LORA_RANK"): m.recurrence.depth_lora_rank = I("DEPTH_LORA_RANK")
        if has("BIGRAM_BUCKETS"):
            m.bigram.vocab_size = I("BIGRAM_BUCKETS")
            m.bigram.enabled = m.bigram.vocab_size > 0
        if has("EMBED_DIM"): m.embed_dim = I("EMBED_DIM")
        if has("SOFTCAP_TYPE"): m.softcap_kind = "poly5" if env["SOFTCAP_TYPE"].lower().startswith("poly") else "tanh"
        if has("VALUE_RESIDUAL"): m.value_residual = B("VALUE_RESIDUAL")
        if has("DTG_ENABLED"): m.dtg = B("DTG_ENABLED")
        if has("MTP_NUM_HEADS"): m.mtp_num_heads = I("MTP_NUM_HEADS")
        if has("MTP_LOSS_WEIGHT"): m.mtp_loss_weight = F("MTP_LOSS_WEIGHT")
        if has("LN_SCALE"): m.ln_scale = B("LN_SCALE")
        if has("VE_ENABLED"): m.value_embedding.enabled = B("VE_ENABLED")
        if has("VE_DIM"): m.value_embedding.dim = I("VE_DIM")
        if has("VE_LAYERS"):
            m.value_embedding.layers = [int(x) for x in env["VE_LAYERS"].split(",") if x.strip()]
        if has("TTT_ENABLED") and B("TTT_ENABLED"):
            e.legal_score_first = True
            e.adaptation_backend = "full_sgd"
        if has("TTT_LR"): e.ttt_lr = F("TTT_LR")
        if has("TTT_EPOCHS"): e.ttt_epochs = I("TTT_EPOCHS")
        if has("TTT_CHUNK_TOKENS"): e.chunk_tokens = I("TTT_CHUNK_TOKENS")
        if has("TTT_FREEZE_BLOCKS"): e.ttt_freeze_blocks = I("TTT_FREEZE_BLOCKS")
        if has("TTT_MOMENTUM"): e.ttt_momentum = F("TTT_MOMENTUM")
        if has("TTT_BATCH_SEQS"): e.ttt_batch_seqs = I("TTT_BATCH_SEQS")
        if has("TTT_GRAD_CLIP"): e.ttt_grad_clip = F("TTT_GRAD_CLIP")
        if has("TTT_LORA_RANK"): e.doc_lora_rank = I("TTT_LORA_RANK")
        if has("TTT_LORA_LR"): e.doc_lora_lr = F("TTT_LORA_LR")
        if has("TTT_CHUNK_SIZE"): e.doc_chunk_size = I("TTT_CHUNK_SIZE")
        if has("TTT_BATCH_SIZE"): e.doc_batch_size = I("TTT_BATCH_SIZE")
        if has("TTT_EVAL_SEQ_LEN"): m.eval_seq_len = I("TTT_EVAL_SEQ_LEN")
        if has("GPTQ_CALIB_BATCHES"): q.gptq_calibration_batches = I("GPTQ_CALIB_BATCHES")
        if has("GPTQ_BLOCK_SIZE"): q.gptq_block_size = I("GPTQ_BLOCK_SIZE")
        if has("INT4_LAYERS"): q.coarse_layers = [int(x) for x in env["INT4_LAYERS"].split(",") if x.strip()]
        if has("INT4_STEP"): q.coarse_step = I("INT4_STEP")
        if has("PG_RECORD_MAX_MS_PER_STEP"): t.record_max_ms_per_step = F("PG_RECORD_MAX_MS_PER_STEP")
        if has("PG_RECORD_TIMING_SKIP_STEPS"): t.timing_skip_steps = I("PG_RECORD_TIMING_SKIP_STEPS")
        if has("TARGET_MB"): q.target_artifact_bytes = int(F("TARGET_MB") * 1024 * 1024)
        return self

    # ---- validation / fingerprint ----------------------------------------------------------
    def validate(self) -> "RunSpec":
        m, t, q, e = self.model, self.train, self.quant, self.eval
        errs = []

        def chk(c, msg):
            if not c:
                errs.append(msg)

        chk(self.mode in RUN_MODES, f"mode must be one of {RUN_MODES}")
        chk(t.backend in TRAIN_BACKENDS, f"train.backend must be one of {TRAIN_BACKENDS}")
        chk(t.distributed_optimizer_backend in DIST_OPT_BACKENDS, "unknown distributed_optimizer_backend")
        chk(q.scheme in QUANT_SCHEMES, f"quant.scheme must be one of {QUANT_SCHEMES}")
        chk(q.compression in COMPRESSION_MODES, "unknown quant.compression")
        chk(q.code_storage in ("bit_packed", "bytes"), "quant.code_storage must be bit_packed or bytes")
        chk(q.calibration in CALIBRATION_MODES, "unknown quant.calibration")
        chk(e.adaptation_backend in ADAPTATION_BACKENDS, "unknown eval.adaptation_backend")
        chk(t.save_layer_acts in ("all", "edges", "inner", "recurrent", "none"), "train.save_layer_acts must be all|edges|inner|recurrent|none")
        chk(0.0 <= t.complementary_alpha <= 1.0, "train.complementary_alpha must be in [0, 1]")
        chk(t.complementary_shape in ("linear", "power", "floored"), "unknown train.complementary_shape")
        chk(t.muon_ns_profile in NS_PROFILES, f"train.muon_ns_profile must be one of {NS_PROFILES}")
        chk(m.activation in ("relu_sq", "leaky_relu_sq", "swiglu"), "model.activation must be relu_sq, leaky_relu_sq or swiglu")
        chk(not (m.activation == "swiglu" or m.normed_out_proj or m.block_smear or m.vocab_bias) or t.backend == "cpu",
            "model.activation=swiglu, model.normed_out_proj, model.block_smear and model.vocab_bias run on train.backend=cpu only")
        chk(m.rope.mode in ("none", "partial", "yarn"), "unknown rope.mode")
        chk(m.attention_backend in ("native", "naive_f32", "flash_f32", "cudnn_sdpa_bf16"), "unknown model.attention_backend")
        chk(m.compute_precision in ("f32", "f32_tf32", "bf16_tensor_core"), "unknown model.compute_precision")
        chk(not (m.caseops.enabled and m.caseops.byte_sidecar and self.mode == "record") or bool(e.caseops_byte_sidecar_pattern),
            "model.caseops.byte_sidecar in record mode needs eval.caseops_byte_sidecar_pattern (token surfaces do not give the byte counts)")
        chk(m.rope.mode != "yarn" or (m.rope.yarn_max_len > 0 and m.rope.yarn_train_len > 0), "rope.mode=yarn needs yarn_max_len and yarn_train_len > 0")
        chk(m.skip_topology in ("none", "unet"), "unknown skip_topology")
        chk(m.num_layers >= 1, "num_layers must be >= 1")
        chk(m.model_dim % m.num_heads == 0, "model_dim must be divisible by num_heads")
        chk(m.num_heads % max(m.num_kv_heads, 1) == 0, "num_heads must be divisible by num_kv_heads")
        chk(m.head_dim % 2 == 0, "head_dim must be even for RoPE")
        chk(m.rope_dims % 2 == 0 and m.rope_dims <= m.head_dim, "rope.dims must be even and <= head_dim")
        chk(m.logit_softcap > 0, "logit_softcap must be positive")
        chk(m.xsa_last_n <= m.depth, "xsa_last_n exceeds the number of layers")
        rc = m.recurrence
        chk(rc.effective_depth == 0 or (rc.enabled and rc.effective_depth >= m.num_layers and rc.repeat_layers == 0),
            "recurrence.effective_depth needs recurrence.enabled, effective_depth >= num_layers and repeat_layers = 0")
        chk(rc.depth_lora_rank == 0 or m.cycled, "recurrence.depth_lora_rank needs the cycled form (recurrence.effective_depth)")
        chk(not m.cycled or t.backend == "cpu", "recurrence.effective_depth (cycled blocks) runs on train.backend=cpu only")
        chk(m.qat_noise_qmax >= 1, "model.qat_noise_qmax must be >= 1")
        chk(rc.repeats >= 1 and (rc.repeats == 2 or not rc.enabled or t.backend == "cpu"), "recurrence.repeats other than 2 runs on train.backend=cpu only")
        chk(not (m.gated_attention or (m.bigram.enabled and m.bigram.trigram)) or t.backend == "cpu",
            "model.gated_attention and model.bigram.trigram run on train.backend=cpu only")
        chk(0.0 <= t.qat_fraction <= 1.0, "train.qat_fraction must be in [0, 1]")
        chk(m.mtp_num_heads >= 0 and m.mtp_loss_weight >= 0.0, "mtp_num_heads and mtp_loss_weight must be >= 0")
        chk(not (m.value_residual or m.mtp_num_heads > 0 or m.fp8_qat or m.dtg or m.embed_dim > 0) or t.backend == "cpu",
            "model.value_residual, model.mtp_num_heads, model.dtg, model.embed_dim and model.fp8_qat run on train.backend=cpu only "
            "(the CUDA engine has no path for them)")
        chk(m.softcap_kind in ("tanh", "poly5") and m.z_loss_weight >= 0.0, "model.softcap_kind must be tanh or poly5 and z_loss_weight >= 0")
        chk((m.softcap_kind == "tanh" and m.z_loss_weight == 0.0) or t.backend == "cpu",
            "model.softcap_kind=poly5 and model.z_loss_weight run on train.backend=cpu only (the fused cross-entropy kernel caps with tanh)")
        chk(m.embed_dim == 0 or (m.tie_embeddings and 0 < m.embed_dim <= m.model_dim), "model.embed_dim needs tied embeddings and 0 < embed_dim <= model_dim")
        chk(q.float_storage in ("f16", "fp8"), "quant.float_storage must be f16 or fp8")
        chk(m.embed_init in ("normal", "overtone") and m.resid_mix_init in ("identity", "phase"), "unknown model.embed_init or model.resid_mix_init")
        chk(q.coarse_step >= 1 and all(0 <= int(l) < m.num_layers for l in q.coarse_layers), "quant.coarse_step must be >= 1 and coarse_layers inside the model")
        chk(not q.coarse_layers or q.scheme not in ("ternary_b158", "binary_b1"), "quant.coarse_layers does not apply to the ternary and binary schemes")
        chk(e.doc_lora_rank >= 0 and e.doc_chunk_size >= 1 and e.doc_batch_size >= 1 and e.doc_lora_lr > 0, "eval.doc_* out of range")
        chk(not e.auto_temperature or t.backend == "cpu", "eval.auto_temperature is scored by the autograd runner (train.backend=cpu)")
        chk(e.temperature > 0 and all(x > 0 for x in e.temperature_grid), "eval.temperature and its grid must be positive")
        chk(m.qat_kind in ("int6", "ternary", "binary", "noise"), "model.qat_kind must be int6, ternary, binary or noise")
        chk(m.qat_kind == "int6" or t.backend == "cpu", "model.qat_kind=ternary|binary|noise runs on train.backend=cpu only")
        chk(q.ternary_group >= 8, "quant.ternary_group must be >= 8")
        chk(not ((m.qat_kind == "ternary" and q.scheme == "ternary_b158") or (m.qat_kind == "binary" and q.scheme == "binary_b1"))
            or m.qat_ternary_group == q.ternary_group,
            "model.qat_ternary_group and quant.ternary_group must agree: what is trained is what is stored")
        chk(q.scheme not in ("ternary_b158", "binary_b1") or not q.lqer.enabled, "the ternary and binary schemes have no low-rank residual")
        chk(not t.lawa_enabled or (t.lawa_k >= 1 and t.lawa_freq >= 1), "train.lawa_k and train.lawa_freq must be >= 1")
        chk(m.vocab_size <= 65536, "token ids are uint16: vocab_size must be <= 65536")
        chk(not (m.attn_out_gate.enabled and m.sparse_attn_gate.enabled),
            "attn_out_gate and sparse_attn_gate are mutually exclusive")
        if m.bigram.enabled:
            chk(m.bigram.vocab_size >= 2, "bigram.vocab_size must be >= 2")
            chk(t.backend == "cpu" or (m.bigram.dim % 64 == 0 and m.bigram.dim != m.model_dim),
                "the CUDA engine needs model.bigram.dim to be a multiple of 64 below model_dim (its products tile the output in 64 columns); "
                "the reference families' 112 runs on train.backend=cpu, or set model.bigram.dim=128")
        if m.value_embedding.enabled:
            chk(all(0 <= l < m.num_layers for l in m.value_embedding.layers), "value_embedding.layers out of range")
        if m.recurrence.enabled:
            chk(m.recurrence.start_layer + m.recurrence.repeat_layers <= m.num_layers, "recurrence range out of bounds")
        chk(t.seq_len > 0 and t.batch_tokens % t.seq_len == 0, "batch_tokens must be a multiple of seq_len")
        chk((t.seq_len_start == 0 and t.batch_tokens_start == 0) or t.backend == "cpu",
            "train.seq_len_start and train.batch_tokens_start run on train.backend=cpu only")
        chk(t.prime_steps >= 0, "train.prime_steps must be >= 0")
        chk(t.matrix_optimizer in ("muon", "adamw") and (t.matrix_optimizer == "muon" or t.backend == "cpu"),
            "train.matrix_optimizer must be muon or adamw; adamw on the banks runs on train.backend=cpu only")
        chk(0.0 <= t.ema_start_fraction < 1.0 and (t.ema_start_fraction == 0.0 or t.backend == "cpu"),
            "train.ema_start_fraction must be in [0, 1) and runs on train.backend=cpu only (the CUDA optimizer kernels average from the first step)")
        chk(t.seq_len_start == 0 or (0 < t.seq_len_start <= t.seq_len and t.seq_len % t.seq_len_start == 0), "train.seq_len_start must divide train.seq_len")
        chk(t.seq_len_start >= 0 and t.batch_tokens_start >= 0 and 0.0 <= t.seq_schedule_fraction <= 1.0 and 0.0 <= t.batch_schedule_fraction <= 1.0,
            "train.*_start must be >= 0 and the schedule fractions in [0, 1]")
        chk(t.world_size >= 1 and 0 <= t.rank < t.world_size, "rank must be in [0, world_size)")
        if t.backend in ("cuda_single", "cuda_single_parity"):
            chk(t.world_size == 1, f"backend {t.backend} requires world_size == 1")
        # the cpu backend with world_size > 1 is data parallel over a gloo process group (host-side logic and its tests)
        chk(4 <= q.matrix_bits <= 8 and (4 <= q.embed_bits <= 8 or q.embed_bits == 16), "quant bits must be in [4, 8] (embed_bits may also be 16 = fp16)")
        chk(e.stride >= 1, "eval.stride must be >= 1")
        chk(t.grad_wire_dtype in ("bf16", "f32"), "grad_wire_dtype must be bf16 or f32")
        if self.mode == "record" and not self.allow_unsupported_variants:
            chk(t.backend == "cuda_distributed", "record mode requires the cuda_distributed backend")
            chk(t.train_data_pattern is not None, "record mode requires train.train_data_pattern")
            chk(t.validation_data_pattern is not None, "record mode requires train.validation_data_pattern")
            chk(e.max_tokens is None, "record mode requires the full validation set (eval.max_tokens unset)")
        if errs:
            raise ValueError("invalid run spec: " + "; ".join(errs))
        return self

    def fingerprint(self) -> int:
        """64-bit FNV-1a over the canonical JSON of model/quant/eval and the training knobs that
        change the trained function (optimizer hyper-parameters, batch shape)."""
        t = self.train
        crit = {
            "model": dataclasses.asdict(self.model),
            "quant": dataclasses.asdict(self.quant),
            "eval": {k: v for k, v in dataclasses.asdict(self.eval).items()
                     if k not in ("tokenizer_vocab_path", "caseops_byte_sidecar_pattern", "max_eval_seconds", "temperature_grid",
                                  "temperature_calibration_tokens")},
            "train": {k: getattr(t, k) for k in (
                "batch_tokens", "seq_len", "matrix_lr", "scalar_lr", "embed_lr", "tied_embed_lr", "muon_momentum",
                "muon_wd", "adam_wd", "muon_ns_profile", "muon_ns_steps", "ema_decay", "late_qat_threshold",
                "grad_clip_norm", "distributed_optimizer_backend")},
        }
        h = 0xCBF29CE484222325
        for b in json.dumps(crit, sort_keys=True, separators=(",", ":")).encode():
            h ^= b
            h = (h * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
        return h


# ---- presets ------------------------------------------------------------------------------------

def family_preset(family: str) -> RunSpec:
    """Built-in variants. ``tiny_cpu``, ``baseline_9l`` and ``record_11l`` are the three model shapes of
    the benchmark configurations; the ``*_sp8192`` names mirror the reference's sweep families
    (``pg-model/src/spec.rs:313-399``) at vocabulary 8192."""
    if family not in FAMILIES:
        raise ValueError(f"unknown family {family!r}; known: {FAMILIES}")
    s = RunSpec(name=family)
    m, t = s.model, s.train
    m.family = family
    if family == "tiny_cpu":
        m.vocab_size, m.num_layers, m.model_dim, m.num_heads, m.num_kv_heads = 1024, 2, 128, 4, 2
        m.mlp_mult, m.activation, m.train_seq_len, m.eval_seq_len = 2.0, "relu_sq", 256, 256
        m.rope.dims = 0
        m.compute_precision = "f32"
        t.backend, t.batch_tokens, t.seq_len, t.total_iterations = "cpu", 8 * 256, 256, 20
        t.matrix_lr, t.muon_momentum, t.muon_momentum_warmup_steps = 0.02, 0.95, 0
        t.tied_embed_lr = t.scalar_lr = 0.05
        t.muon_wd = t.adam_wd = 0.0
        t.warmdown_iters, t.grad_clip_norm, t.max_wallclock_seconds = 0, 0.0, 0.0
        t.swa_enabled, t.late_qat_threshold, t.ema_decay = False, 0.0, 0.0
        s.eval.stride = 64
    elif family == "baseline_9l":
        m.num_layers, m.mlp_mult, m.activation = 9, 2.0, "relu_sq"
        m.train_seq_len = m.eval_seq_len = 1024
        m.rope.dims = 0
        t.backend, t.batch_tokens, t.seq_len = "cuda_distributed", 524_288, 1024
        t.total_iterations, t.warmdown_iters = 20000, 1200
        t.matrix_lr, t.scalar_lr, t.tied_embed_lr = 0.04, 0.04, 0.05
        t.muon_momentum, t.muon_momentum_warmup_start, t.muon_momentum_warmup_steps = 0.95, 0.85, 500
        t.muon_wd = t.adam_wd = 0.0
        t.muon_ns_profile = "simple"
        t.grad_clip_norm, t.swa_enabled, t.late_qat_threshold, t.ema_decay = 0.0, False, 0.0, 0.0
    elif family == "record_11l":
        m.num_layers, m.mlp_mult, m.activation = 11, 3.0, "leaky_relu_sq"
        m.xsa_last_n, m.ln_scale, m.smear_gate = 4, True, True
        m.rope.dims = 16
        m.bigram = BigramSpec(True, 3072, 128)
        t.backend, t.distributed_optimizer_backend = "cuda_distributed", "sharded_parallel_muon"
        t.batch_tokens, t.seq_len = 786_432, 2048
        s.quant.scheme = "full_gptq_int6"
        s.quant.calibration = "self_generated"
        s.quant.code_storage, s.quant.prune_max_magnitude = "bytes", 3      # the Python records' container and prune-to-budget step
        s.eval.legal_score_first = True
        s.eval.adaptation_backend = "full_sgd"
    elif family == "ternary_10l":
        # records/track_10min_16mb/2026-03-24_74M_Ternary_UNet_FP8_10L_8192BPE_YaRN_NeoMuon (README "Architecture", run_cuda_ternary.sh):
        # ternary weights trained with a straight-through estimator from the first step, FP8 for the rest, YaRN, three
        # Newton-Schulz steps, the 254-wide factored tied embedding, the degree-5 polynomial soft-cap with a z-loss of 1e-4, sliding evaluation at stride 16.
        m.vocab_size, m.num_layers, m.model_dim, m.num_heads, m.num_kv_heads = 8192, 10, 768, 8, 4
        m.mlp_mult, m.activation = 4.0, "relu_sq"
        m.train_seq_len = m.eval_seq_len = 1024
        m.rope = RopeSpec("yarn", 0, 5000.0, 2048, 1024)
        m.logit_softcap, m.qk_gain_init = 10.0, 2.25
        m.softcap_kind, m.z_loss_weight = "poly5", 1e-4
        m.embed_dim = 254
        m.qat_kind, m.fp8_qat = "ternary", True
        t.backend, t.batch_tokens, t.seq_len = "cpu", 524_288, 1024
        t.qat_enabled, t.late_qat_threshold = True, 0.0
        t.matrix_lr, t.scalar_lr, t.tied_embed_lr, t.head_lr = 0.04, 0.02, 0.02, 0.02
        t.muon_momentum, t.muon_momentum_warmup_start, t.muon_momentum_warmup_steps = 0.95, 0.85, 500
        t.muon_wd, t.adam_wd, t.muon_ns_steps = 0.0, 0.05, 3
        t.total_iterations, t.warmup_steps, t.max_wallclock_seconds = 10000, 5, 599.0
        t.warmdown_frac = 0.2
        t.grad_clip_norm, t.ema_decay, t.swa_enabled = 0.0, 0.0, False      # the script's defaults: no clipping, no weight averaging
        m.normed_out_proj = m.vocab_bias = True
        s.quant.scheme, s.quant.compression, s.quant.float_storage = "ternary_b158", "lzma9", "fp8"
        s.quant.prune_to_target = False
        s.eval.stride, s.eval.auto_temperature = 16, True       # SLIDING_EVAL_STRIDE=16, TEMP_SCALING=1 in the run script
    elif family == "binary_15l":
        # records/track_non_record_16mb/2026-03-24_106M_Binary_Asymmetric_UNet_FP8_15L_8192BPE_YaRN_NeoMuon_Smear (README "Architecture",
        # run_cuda_binary.sh): the ternary recipe with 1-bit weights, 15 blocks (7 before the U-Net's turn, 8 after) and the
        # per-block running-mean smear; 50,000 steps with no wall-clock cap, the last fifth of them warm-down.
        m.vocab_size, m.num_layers, m.model_dim, m.num_heads, m.num_kv_heads = 8192, 15, 768, 8, 4
        m.mlp_mult, m.activation = 4.0, "relu_sq"
        m.train_seq_len = m.eval_seq_len = 1024
        m.rope = RopeSpec("yarn", 0, 5000.0, 2048, 1024)
        m.logit_softcap, m.qk_gain_init = 10.0, 2.25
        m.softcap_kind, m.z_loss_weight = "poly5", 1e-4
        m.embed_dim = 254
        m.qat_kind, m.fp8_qat = "binary", True
        m.normed_out_proj, m.block_smear, m.vocab_bias = True, True, True
        t.backend, t.batch_tokens, t.seq_len = "cpu", 524_288, 1024
        t.qat_enabled, t.late_qat_threshold = True, 0.0
        t.matrix_lr, t.scalar_lr, t.tied_embed_lr, t.head_lr = 0.04, 0.02, 0.02, 0.02
        t.muon_momentum, t.muon_momentum_warmup_start, t.muon_momentum_warmup_steps = 0.95, 0.85, 500
        t.muon_wd, t.adam_wd, t.muon_ns_steps = 0.0, 0.05, 3
        t.total_iterations, t.warmup_steps, t.max_wallclock_seconds = 50000, 5, 0.0
        t.warmdown_frac, t.swa_enabled = 0.2, False
        t.grad_clip_norm, t.ema_decay = 0.0, 0.0
        s.quant.scheme, s.quant.compression, s.quant.float_storage = "binary_b1", "lzma9", "fp8"
        s.quant.prune_to_target = False
        s.eval.stride, s.eval.auto_temperature = 16, True       # SLIDING_EVAL_STRIDE=16, TEMP_SCALING=1 in the run script
    else:
        # The six families of the reference engine, field for field (pg-model/src/spec.rs:313-399 ModelSpec::for_family, with
        # TrainSpec / QuantSpec / EvalSpec defaults of :489-524, :603-664): SP8192 vocabulary, 11 x 512, BigramHash 3072 x 112, value
        # embeddings on the last two blocks, boundary-masked SmearGate, query gain 5.
        m.vocab_size = 8192
        m.num_layers, m.mlp_mult, m.activation = 11, 3.0, "leaky_relu_sq"
        m.train_seq_len = m.eval_seq_len = 2048
        m.bigram = BigramSpec(True, 3072, 112)
        m.xsa_last_n = 4
        m.value_embedding = ValueEmbeddingSpec(True, 128, [9, 10])
        m.rope = RopeSpec("partial", 16, 10000.0)
        m.smear_gate, m.smear_gate_boundary_token_id = True, 1
        m.logit_softcap, m.qk_gain_init, m.ln_scale, m.tie_embeddings = 30.0, 5.0, True, True
        m.attention_backend, m.compute_precision = "flash_f32", "f32_tf32"
        m.attn_out_gate = AttnOutGateSpec(False, 24)                  # its default width (spec.rs:233-240)
        m.parallel_residual = ParallelResidualSpec(False, False)      # the reference's default: `enabled` alone does not split (spec.rs:216-222)
        t.batch_tokens, t.seq_len, t.warmup_steps = 524_288, 2048, 20
        t.muon_ns_profile, t.muon_ns_steps = "polar_express", 5      # its default coefficients (pg-optim/src/muon.rs:19-30), five steps (spec.rs:544)
        t.wallclock_warmdown = False      # the engine's schedule is counted in steps (warm-up from zero, stable, warm-down; pg-optim/src/scheduler.rs:12-66); its wall-clock cap only stops the run
        q, e = s.quant, s.eval
        q.lqer = LqerSpec(False, 4, 3, 2, 4, 64, True)
        q.mlp_clip_sigmas, q.attn_clip_sigmas, q.embed_clip_sigmas, q.gptq_calibration_batches = 12.0, 13.0, 14.0, 0
        e.legal_score_first, e.lora_rank, e.lora_alpha = True, 128, 144.0
        e.phased_ttt_prefix_docs, e.phased_ttt_phases, e.phased_ttt_weight_decay, e.ttt_beta2 = 2000, 3, 1.0, 0.99
        if family == "xsa_all_sp8192":
            m.xsa_last_n = m.num_layers
        elif family == "recurrence_mid_sp8192":
            m.recurrence = RecurrenceSpec(True, 4, 2)
        elif family == "parallel_resid_sp8192":
            m.parallel_residual = ParallelResidualSpec(True, True)
        elif family == "hybrid_competitive_sp8192":
            m.xsa_last_n, m.qk_gain_init = m.num_layers, 5.25
            m.value_embedding = ValueEmbeddingSpec(False, 128, [])
            m.recurrence = RecurrenceSpec(True, 4, 2)
            m.parallel_residual = ParallelResidualSpec(True, True)
            m.caseops = CaseOpsSpec(True, True)
            m.sparse_attn_gate = SparseAttnGateSpec(True, 12, 1.0)
        elif family == "frontier_1855_like":
            m.attention_backend, m.compute_precision = "cudnn_sdpa_bf16", "bf16_tensor_core"
            m.mlp_mult, m.xsa_last_n, m.qk_gain_init = 4.0, m.num_layers, 5.0
            m.value_embedding = ValueEmbeddingSpec(False, 128, [])
            m.recurrence = RecurrenceSpec(True, 4, 2)
            m.parallel_residual = ParallelResidualSpec(True, True)
            m.caseops = CaseOpsSpec(True, True)
            m.sparse_attn_gate = SparseAttnGateSpec(True, 12, 0.5)
            m.bigram.enabled = False
    return s


# The ten architectures of the reference's sweep (pg-model/src/arch.rs:137-168), as
# (model_dim, heads, kv_heads, layers, mlp_mult, rope_dims, first XSA layer, seq_len) over its "sota" base configuration
# (pg-model/src/config.rs:60-110: vocabulary 1024, BigramHash 1536 x 128, value embeddings on blocks 9 and 10, boundary-masked SmearGate).
ARCH_VARIANTS = {
    "baseline": (512, 8, 4, 11, 3, 16, 7, 2048),
    "wide": (576, 8, 4, 11, 3, 16, 7, 2048),                  # head_dim 72
    "wide_narrow_mlp": (576, 8, 4, 11, 2, 16, 7, 2048),
    "deep": (512, 8, 4, 13, 3, 16, 9, 2048),
    "deep_narrow": (384, 6, 3, 16, 3, 12, 12, 2048),
    "full_xsa": (512, 8, 4, 11, 3, 16, 0, 2048),
    "more_rope": (512, 8, 4, 11, 3, 32, 7, 2048),
    "high_gqa": (480, 12, 3, 11, 3, 16, 7, 2048),             # head_dim 40
    "long_ctx": (512, 8, 4, 11, 3, 16, 7, 4096),
    "aggressive_quant": (640, 8, 4, 11, 3, 16, 7, 2048),      # fits 16 MB only at int4
}


def arch_label(name: str) -> str:
    d, h, kv, n, mm, rd, xf, sl = ARCH_VARIANTS[name]
    return f"d{d}_h{h}_kv{kv}_L{n}_m{mm}_r{rd}_x{xf}_s{sl}"


def arch_variant(name: str) -> RunSpec:
    """The run spec of one sweep architecture: the record stack with the eight numbers of `ARCH_VARIANTS` put in. Widths whose
    head_dim is not 64 (wide, high_gqa) run on the autograd path; the CUDA engine's attention kernels are written for 64."""
    if name not in ARCH_VARIANTS:
        raise ValueError(f"unknown architecture {name!r}; known: {tuple(ARCH_VARIANTS)}")
    d, h, kv, n, mm, rd, xf, sl = ARCH_VARIANTS[name]
    s = family_preset("record_11l")
    s.name = f"arch_{name}"
    m = s.model
    m.vocab_size, m.model_dim, m.num_heads, m.num_kv_heads, m.num_layers, m.mlp_mult = 1024, d, h, kv, n, float(mm)
    m.rope = RopeSpec("partial", rd, 10000.0)
    m.xsa_last_n = 0 if xf >= n else n - xf
    m.train_seq_len = m.eval_seq_len = s.train.seq_len = sl
    m.bigram = BigramSpec(True, 1536, 128)
    m.value_embedding = ValueEmbeddingSpec(True, 128, [9, 10])
    m.smear_gate, m.smear_gate_boundary_token_id, m.ln_scale, m.qk_gain_init = True, 1, True, 1.5
    if m.head_dim != 64 or rd % 16:          # shapes the CUDA kernels are not written (or not tested) for
        s.train.backend, s.train.distributed_optimizer_backend = "cpu", "all_reduce_replicated_muon"
    return s


def _ns_profile_name(raw: str) -> str:
    """The reference's spellings of its three coefficient profiles (pg-optim/src/muon.rs:20-30); anything else is polar_express."""
    raw = raw.lower()
    return "simple" if raw in ("simple", "legacy", "ns5") else "quintic" if raw in ("quintic", "modded_nanogpt") else "polar_express"


# ---- helpers --------------------------------------------------------------------------------------

def _field_type(obj, name):
    for f in fields(obj):
        if f.name == name:
            return f.type
    return None


def _coerce(text: str, current, ftype=None):
    if isinstance(current, bool):
        return text.lower() in ("1", "true", "yes", "on")
    if isinstance(current, int):
        return int(text)
    if isinstance(current, float):
        return float(text)
    if isinstance(current, list):
        items = [x.strip() for x in text.strip("[]").split(",") if x.strip()]
        if any(isinstance(c, float) for c in current) or any(("." in x or "e" in x.lower()) for x in items):
            return [float(x) for x in items]          # a list of floats (e.g. eval.temperature_grid)
        return [int(x) for x in items]
    if current is None:
        if text.lower() in ("none", "null", ""):
            return None
        t = str(ftype)
        if "int" in t:
            return int(text)
        if "float" in t:
            return float(text)
        return text
    return text


def _overlay(obj, d: dict):
    """Set the keys of ``d`` on the dataclass ``obj`` (tables recurse into the nested dataclass that is already there)."""
    known = {f.name: f for f in fields(obj)}
    for k, v in d.items():
        if k not in known:
            raise KeyError(f"unknown key {k!r} in [{type(obj).__name__}]")
        cur = getattr(obj, k)
        if is_dataclass(cur):
            if not isinstance(v, dict):
                raise TypeError(f"{k} must be a table")
            _overlay(cur, v)
        else:
            if isinstance(cur, float) and isinstance(v, int) and not isinstance(v, bool):
                v = float(v)
            setattr(obj, k, v)
    return obj


def _to_toml(d: dict, prefix: str = "") -> str:
    scalars, tables = [], []
    for k, v in d.items():
        if isinstance(v, dict):
            tables.append((k, v))
        elif v is None:
            continue
        elif isinstance(v, bool):
            scalars.append(f"{k} = {'true' if v else 'false'}")
        elif isinstance(v, (int, float)):
            scalars.append(f"{k} = {v!r}")
        elif isinstance(v, list):
            scalars.append(f"{k} = [{', '.join(repr(x) for x in v)}]")
        else:
            scalars.append(f"{k} = {json.dumps(v)}")
    out = "\n".join(scalars)
    for k, v in tables:
        name = f"{prefix}{k}"
        out += f"\n\n[{name}]\n" + _to_toml(v, name + ".")
    return out.strip() + "\n" if not prefix else out
