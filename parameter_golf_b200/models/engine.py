"""CUDA engine: explicit forward, backward and optimizer step on the sm_100a kernels.

One engine instance owns, on one GPU: fp32 master parameters (banks + flat Adam groups), their
gradients, bf16 compute copies of the weights, and every saved activation of one micro-batch. The
forward/backward is written out kernel by kernel (no autograd), following the block structure of
``parameter-golf-rs/crates/pg-model/src/gpu.rs:6041-6908`` (forward) and ``:4558-5918`` (backward), but with
one execution path per op and the element-wise work folded into GEMM epilogues and fused row kernels:

* residual-mix + RMSNorm, RMSNorm-backward + mix/skip backward: one row kernel each;
* O and MLP-down projections carry the residual add in their epilogue; their per-feature output
  scales (``attn_scale``, ``mlp_scale``) are folded into the bf16 weight copies at cast time, and the
  scale gradients are recovered from the un-scaled weight gradient (``d_scale[n] = sum_k W[n,k] G[n,k]``);
* MLP-up stores the pre-activation and ``leaky_relu(.)^2`` from one accumulator read; the
  down-projection's dX GEMM multiplies by the activation derivative in its epilogue;
* tied-embedding logits are produced in bf16 and overwritten in place by their gradient in the
  soft-capped cross-entropy kernel.

Model variants follow the same path: depth recurrence runs a layer's block twice with per-pass activation slots
(``pg-model/src/model.rs:666-671``), the parallel residual feeds the MLP from the attention branch's normed input
(so its gradient joins the QKV input gradient in that GEMM's epilogue), the attention-output and sparse attention
gates are one head kernel pair (``pg-kernels/src/gpu_kernels.rs:4973-5413``), and an untied output head is a second
bf16 weight copy with its own AdamW group.

Gradients of bf16 activations are bf16; weight gradients accumulate in fp32 across micro-batches.
"""
from __future__ import annotations

import math
import os
from typing import Dict, List, Optional, Tuple

import torch

from ..ops import native as N
from ..ops import reference as R
from ..optim.muon import ns_coeff
from ..spec import ModelSpec, RunSpec
from ..utils.logging import nvtx_range
from . import gpt

BF = torch.bfloat16
EMB_NAMES = ("tok_emb", "bigram_embed", "ve_embed")


CANARY_BYTE = 0xA5


def _unsupported(m: ModelSpec) -> Optional[str]:
    only_autograd = [k for k, on in (("value_residual", m.value_residual), ("mtp_num_heads", m.mtp_num_heads > 0), ("dtg", m.dtg),
                                     ("embed_dim", m.embed_dim > 0), ("softcap_kind", m.softcap_kind != "tanh"),
                                     ("activation=swiglu", m.activation == "swiglu"), ("normed_out_proj", m.normed_out_proj),
                                     ("block_smear", m.block_smear), ("vocab_bias", m.vocab_bias),
                                     ("recurrence.effective_depth", m.cycled), ("gated_attention", m.gated_attention),
                                     ("bigram.trigram", m.bigram.enabled and m.bigram.trigram),
                                     ("recurrence.repeats", m.recurrence.enabled and m.recurrence.repeats != 2)) if on]
    if only_autograd:
        return "model options of the autograd path (" + ", ".join(only_autograd) + ")"
    if m.model_dim % 64 or m.kv_dim % 64 or m.mlp_dim % 64 or m.head_dim % 8 or m.vocab_size % 64:
        return "dims that are not multiples of 64"
    if m.bigram.enabled and (m.bigram.dim % 64 or m.bigram.dim == m.model_dim):
        return "bigram dim not a multiple of 64 (or equal to model_dim)"
    return None


class CudaEngine:
    def __init__(self, spec: RunSpec, params: Optional[Dict[str, torch.Tensor]], device, micro_batch: int, seq_len: int, train: bool = True,
                 share: Optional["CudaEngine"] = None):
        """``share``: another engine of the same spec and device whose parameters, gradients, optimizer state and bf16 weight
        copies this one aliases (everything that does not depend on the batch shape); only the activation buffers are new.
        Evaluation and test-time training switch between a scoring shape and a training shape many times per second, and
        rebuilding an engine per switch (parameters through the host included) used to dominate their time."""
        bad = _unsupported(spec.model)
        if bad:
            raise NotImplementedError(f"the CUDA engine does not cover {bad}; use the cpu backend for this variant")
        self.C = N.load()
        self.spec, self.m, self.t = spec, spec.model, spec.train
        self.dev = torch.device(device)
        self.B, self.S = micro_batch, seq_len
        self.T = micro_batch * seq_len
        self.train = train
        self.qat = False
        m = self.m
        self.n, self.d, self.kv, self.mlp, self.H, self.Hkv, self.hd = m.num_layers, m.model_dim, m.kv_dim, m.mlp_dim, m.num_heads, m.num_kv_heads, m.head_dim
        self.qkvw = self.d + 2 * self.kv
        self.slope = m.leaky_slope if m.activation == "leaky_relu_sq" else 0.0
        self.enc = self.n // 2
        self.sched = gpt.layer_schedule(m)                     # (layer, pass) per activation slot
        self.nslots = len(self.sched)
        self.last_slot = {l: j for j, (l, _) in enumerate(self.sched)}
        self.first_slot = {}
        for j, (l, _) in enumerate(self.sched):
            self.first_slot.setdefault(l, j)
        # Activation checkpointing (saved-activation policies of pg-model/src/gpu.rs:1159-1201, 1742-1744): slots whose
        # block activations are not kept share ONE set of buffers and the block is run again from its kept input right
        # before its backward. Block outputs (T x d per slot) are always kept: they are the recompute inputs and skips.
        self.saved = self._saved_slots(getattr(spec.train, "save_layer_acts", "all")) if train else [False] * self.nslots
        self.act_slot, nsaved = [], 0
        for keep in self.saved:
            self.act_slot.append(nsaved if keep else -1)
            nsaved += int(keep)
        self.nact = nsaved + (0 if all(self.saved) else 1)     # number of activation buffer sets
        self.act_slot = [a if a >= 0 else self.nact - 1 for a in self.act_slot]
        self.block_in = [None] * self.nslots                   # (x, skip, skip weight) each slot's block consumed
        self.parallel = m.parallel
        self.gates = []                                        # (weight name, bias name or None, scale, multiplier)
        if m.attn_out_gate.enabled:
            self.gates.append(("attn_gate_weight", "attn_gate_bias", 1.0, 2.0))
        if m.sparse_attn_gate.enabled:
            self.gates.append(("sparse_attn_gate_weight", None, float(m.sparse_attn_gate.scale), 1.0))
        self.unet = m.skip_topology == "unet" and "skip_weights" in (share.p if share is not None else params)
        self.eps = R.RMS_EPS
        if share is not None:
            assert share.dev == self.dev and share.train == train and share.m == self.m
            for name in ("p", "g", "groups", "Wqkv", "Wo", "Wup", "Wd", "Wo_u", "Wd_u", "E", "LM", "BE", "BP", "VE", "VP", "ve_eff", "ema", "mom",
                         "ns", "Gd", "Go", "Gbp", "Gvp"):
                if hasattr(share, name):
                    setattr(self, name, getattr(share, name))
        else:
            self._alloc_params(params)
        self._alloc_acts()
        # Pinned staging for the per-step hyper-parameters: a ring of buffers, each guarded by the event recorded after its
        # asynchronous upload, so that a host that runs ahead of the stream (no per-step synchronisation, graph replay)
        # never rewrites a buffer whose copy has not executed yet.
        self.hp_ring = [torch.zeros(8, dtype=torch.float32).pin_memory() for _ in range(4)]
        self.hp_ring_events = [None] * len(self.hp_ring)
        self.hp_ring_pos = 0
        self.hp_host = self.hp_ring[0]
        self.hp = torch.zeros(8, dtype=torch.float32, device=self.dev)
        self.hp_host[0], self.hp_host[4] = 1.0, 1.0
        self.hp.copy_(self.hp_host)
        self.stats = torch.zeros(4, dtype=torch.float32, device=self.dev)
        self.loss_sum = torch.zeros(1, dtype=torch.float32, device=self.dev)
        self.pair_w_table = self.tok_w = self.w_total = None       # complementary training, see `set_token_weight_table`
        # Called as ``backward_observer(layer, slot)`` right after the backward of each block has been enqueued: every
        # gradient of that layer is then final for this micro-batch unless the layer runs again in an earlier slot. Hook
        # for per-layer gradient reduction overlapped with the rest of the backward (role of `GpuBackwardLayerObserver`,
        # pg-model/src/gpu.rs:517-525).
        self.backward_observer = None
        self.adam_t = 0
        self.layer_flags = None          # set by the sharded optimizer: per-layer weight-ready counters
        self.layer_flag_value = 0
        self.layer_wait_needed = False   # set after a sharded update: the next forward gates each layer with a one-thread wait kernel
        self.lora = None                 # Q-LoRA adapter {"a": [n, r, d], "b": [n, d, r], "alpha", "trainable"} (test-time training); see `set_lora`
        self._lora_rank = 0
        self.param_generation = 0        # bumped by every write to the fp32 master parameters
        self.cast_generation = -1        # generation the bf16 compute copies were made from
        if share is not None:            # the shared bf16 copies are already current
            self.hp, self.hp_host, self.stats = share.hp, share.hp_host, share.stats
            self.hp_ring, self.hp_ring_events, self.hp_ring_pos = share.hp_ring, share.hp_ring_events, 0
            self.adam_t, self.qat = share.adam_t, share.qat
            self.param_generation, self.cast_generation = share.param_generation, share.cast_generation
        else:
            self.cast_weights()

    # ---- storage -----------------------------------------------------------------------------------------------
    def _saved_slots(self, mode: str) -> List[bool]:
        """Which activation slots keep their block activations between forward and backward. ``all`` (default: 180 GB of
        HBM holds every layer of the record shape many times over), ``edges`` (layers 0-2 and the last two, single-pass
        layers only; layers 3-8 and repeated layers recompute), ``inner`` (the complement of the edge rule: layers 3-8),
        ``recurrent`` (only layers that run more than once), ``none`` (every block recomputes)."""
        mode = str(mode).lower()
        passes = {}
        for l, _ in self.sched:
            passes[l] = passes.get(l, 0) + 1
        inner = lambda l: 3 <= l <= 8
        if mode in ("all", "1", "true"):
            return [True] * self.nslots
        if mode in ("none", "0", "false", "off"):
            return [False] * self.nslots
        if mode in ("edges", "checkpoint"):
            return [(not inner(l)) and passes[l] == 1 for l, _ in self.sched]
        if mode in ("inner", "checkpointed"):
            return [inner(l) for l, _ in self.sched]
        if mode == "recurrent":
            return [passes[l] > 1 for l, _ in self.sched]
        raise ValueError(f"train.save_layer_acts: unknown mode {mode!r}")

    def _alloc_params(self, params):
        dev, m = self.dev, self.m
        shapes = gpt.param_shapes(m)
        self.p: Dict[str, torch.Tensor] = {}
        self.g: Dict[str, torch.Tensor] = {}
        for k in gpt.BANKS:
            self.p[k] = params[k].detach().to(dev, torch.float32).contiguous()
            if self.train:
                self.g[k] = torch.zeros_like(self.p[k])
        emb = [k for k in EMB_NAMES if k in shapes]
        head = [k for k in ("lm_head",) if k in shapes]
        sca = [k for k in shapes if k not in gpt.BANKS and k not in emb and k not in head]
        self.groups = []
        plan = [(emb, self.t.tied_embed_lr if m.tie_embeddings else self.t.embed_lr), (sca, self.t.scalar_lr)]
        if head:
            plan.append((head, self.t.head_lr))
        for names, lr in plan:
            total = sum(-(-math.prod(shapes[k]) // 4) * 4 for k in names)
            flat_p = torch.zeros(total, dtype=torch.float32, device=dev)
            flat_g = torch.zeros(total, dtype=torch.float32, device=dev) if self.train else None
            off = 0
            for k in names:
                nel = math.prod(shapes[k])
                self.p[k] = flat_p[off:off + nel].view(shapes[k])
                self.p[k].copy_(params[k].detach().to(dev, torch.float32))
                if self.train:
                    self.g[k] = flat_g[off:off + nel].view(shapes[k])
                off += -(-nel // 4) * 4
            grp = {"names": names, "lr": lr, "p": flat_p, "g": flat_g}
            if self.train:
                grp["m"], grp["v"] = torch.zeros_like(flat_p), torch.zeros_like(flat_p)
            self.groups.append(grp)
        n, d, kv, mlp = self.n, self.d, self.kv, self.mlp
        self.Wqkv = torch.empty(n, self.qkvw, d, dtype=BF, device=dev)
        self.Wo = torch.empty(n, d, d, dtype=BF, device=dev)
        self.Wup = torch.empty(n, mlp, d, dtype=BF, device=dev)
        self.Wd = torch.empty(n, d, mlp, dtype=BF, device=dev)
        self.Wo_u = torch.empty(n, d, d, dtype=BF, device=dev)       # un-scaled copies: only read by the scale-gradient fold
        self.Wd_u = torch.empty(n, d, mlp, dtype=BF, device=dev)
        self.E = torch.empty(m.vocab_size, d, dtype=BF, device=dev)
        self.LM = self.E if m.tie_embeddings else torch.empty(m.vocab_size, d, dtype=BF, device=dev)   # output projection
        if m.bigram.enabled:
            self.BE = torch.empty(m.bigram.vocab_size, m.bigram.dim, dtype=BF, device=dev)
            self.BP = torch.empty(d, m.bigram.dim, dtype=BF, device=dev)
        if m.value_embedding.enabled:
            ve = m.value_embedding
            self.VE = torch.empty(m.vocab_size, ve.dim, dtype=BF, device=dev)
            self.VP = torch.empty(len(ve.layers), kv, ve.dim, dtype=BF, device=dev)
            self.ve_eff = torch.zeros(len(ve.layers), dtype=torch.float32, device=dev)
        if self.train:
            self.ema: Optional[Dict[str, torch.Tensor]] = None
            self.mom = {k: torch.zeros_like(self.p[k]) for k in gpt.BANKS}
            self.ns = {}
            for k in gpt.BANKS:
                Bk, Mk, Nk = self.p[k].shape
                r = min(Mk, Nk)
                self.ns[k] = {"U": torch.empty(Bk, Mk, Nk, dtype=BF, device=dev), "X0": torch.empty(Bk, Mk, Nk, dtype=BF, device=dev),
                              "X1": torch.empty(Bk, Mk, Nk, dtype=BF, device=dev), "A": torch.empty(Bk, r, r, dtype=BF, device=dev),
                              "Bm": torch.empty(Bk, r, r, dtype=BF, device=dev), "sq": torch.zeros(Bk, dtype=torch.float32, device=dev)}
            self.Gd = torch.zeros(d, mlp, dtype=torch.float32, device=dev)
            self.Go = torch.zeros(d, d, dtype=torch.float32, device=dev)
            if m.bigram.enabled:
                self.Gbp = torch.zeros(d, m.bigram.dim, dtype=torch.float32, device=dev)
            if m.value_embedding.enabled:
                self.Gvp = torch.zeros(kv, m.value_embedding.dim, dtype=torch.float32, device=dev)

    def _alloc_acts(self):
        dev, T, d, n = self.dev, self.T, self.d, self.n

        poison = os.environ.get("PGB_POISON", "0") not in ("", "0")
        canary = os.environ.get("PGB_CANARY", "0") not in ("", "0")
        self._canaries: List[Tuple[str, torch.Tensor]] = []

        def buf(*shape, dtype=BF):
            # debug aids. PGB_POISON: activations start as NaN, so a kernel that reads a buffer before its producer ran shows up
            # as a NaN loss instead of silently using stale data (role of the reference's poison fill, pg-model/src/gpu.rs:637-733).
            # PGB_CANARY: every buffer sits between two 512-byte guard zones filled with a byte pattern; `check_canaries` finds
            # the kernel output that ran past its end (the stand-in for a memory checker, which this pool does not offer).
            if canary:
                n = 1
                for x in shape:
                    n *= int(x)
                esz = torch.empty(0, dtype=dtype).element_size()
                nbytes = -(-n * esz // 512) * 512
                raw = torch.full((nbytes + 1024,), CANARY_BYTE, dtype=torch.uint8, device=dev)
                body = raw[512:512 + n * esz].view(dtype).view(*shape)
                if poison and dtype in (BF, torch.float32):
                    body.fill_(float("nan"))
                self._canaries.append((f"buffer {len(self._canaries)} {tuple(shape)} {dtype}", raw, n * esz))
                return body
            if poison and dtype in (BF, torch.float32):
                return torch.full(shape, float("nan"), dtype=dtype, device=dev)
            return torch.empty(*shape, dtype=dtype, device=dev)

        m = self.m
        self.ids = torch.zeros(T, dtype=torch.int32, device=dev)
        self.tgt = torch.zeros(T, dtype=torch.int32, device=dev)
        self.e = buf(T, d)
        self.xe = buf(T, d) if m.bigram.enabled else self.e
        if m.bigram.enabled:
            self.bg = buf(T, m.bigram.dim)
        if m.value_embedding.enabled:
            self.ve_e = buf(T, m.value_embedding.dim)
        self.x0 = buf(T, d)
        L = self.nact if self.train else 1    # inference reuses one slot's worth of buffers

        def per_layer(*shape):
            return [buf(*shape) for _ in range(L)]

        self.x_in, self.h = per_layer(T, d), per_layer(T, d)
        self.qkv_pre, self.qk_post = per_layer(T, self.qkvw), per_layer(T, self.qkvw)
        self.y, self.x_mid = per_layer(T, d), per_layer(T, d)
        self.mm = self.h if self.parallel else per_layer(T, d)      # parallel residual: the MLP reads the attention branch's normed input
        xsa_sets = {self.act_slot[j] for j, (l, _) in enumerate(self.sched) if l in m.xsa_layers()} if self.train else ({0} if m.xsa_last_n > 0 else set())
        self.z = [buf(T, d) if i in xsa_sets else None for i in range(L)]
        self.yg = [[buf(T, d) for _ in range(L)] for _ in self.gates]          # gated attention outputs, one list per gate
        self.gv = [[torch.empty(T, self.H, dtype=torch.float32, device=dev) for _ in range(L)] for _ in self.gates]
        self.zz = [None] * L                 # what the output projection consumed in each slot
        self.hu, self.a = per_layer(T, self.mlp), per_layer(T, self.mlp)
        self.x_out = [buf(T, d) for _ in range(self.nslots)]
        self.lse = [None] * L
        self.hf = buf(T, d)
        from ..plan import logit_chunk_rows
        self.logit_rows = logit_chunk_rows(T, m.vocab_size, self.t.logit_chunk_rows)      # < T: the head runs per chunk of rows
        self.logits = buf(self.logit_rows, m.vocab_size)
        self._logits_full = None                   # only for callers that ask for every logit (`forward(targets=None)`) while chunking
        self._head_grads_done = False
        self.nll = buf(T, dtype=torch.float32)
        rd = m.rope_dims
        if rd > 0:
            cos, sin = R.model_rope_tables(m, self.S)
            self.cos, self.sin = cos.contiguous().to(dev), sin.contiguous().to(dev)
        else:
            self.cos = self.sin = None
        if self.train:
            self.dx, self.dx_mid, self.d_m, self.d_z, self.d_y, self.d_h = (buf(T, d) for _ in range(6))
            self.d_hu = buf(T, self.mlp)
            self.d_qk_post, self.d_qkv_pre = buf(T, self.qkvw), buf(T, self.qkvw)
            self.d_x0 = buf(T, d)
            if self.gates and not self.parallel:
                self.d_hx = torch.zeros(T, d, dtype=BF, device=dev)     # only its first `width` columns are ever written
            self.dsum = torch.empty(self.B, self.H, self.S, dtype=torch.float32, device=dev)
            # fp32 dQ accumulator of the single-pass attention backward: zero between calls (the kernels restore that)
            self.dq_acc = None if self.t.reproducible_backward else torch.zeros(self.B * self.H * self.S * self.hd, dtype=torch.float32, device=dev)
            self.d_skip = [buf(T, d) for _ in range(max(self.enc - 1, 0))] if self.unet else []
            self.d_xe = buf(T, d)
            if m.bigram.enabled:
                self.d_bg = buf(T, m.bigram.dim)

    def check_canaries(self):
        """With ``PGB_CANARY=1``: raise if any byte of a guard zone around an activation / scratch buffer was overwritten."""
        torch.cuda.synchronize(self.dev)
        for name, raw, used in getattr(self, "_canaries", []):
            head, tail = raw[:512], raw[512 + used:]
            if not (bool((head == CANARY_BYTE).all()) and bool((tail == CANARY_BYTE).all())):
                where = "before" if not bool((head == CANARY_BYTE).all()) else "after"
                raise RuntimeError(f"guard zone {where} {name} was overwritten")

    # ---- weights --------------------------------------------------------------------------------------------------
    def cast_weights(self, banks: bool = True):
        """fp32 master -> bf16 compute copies (packed QKV, output scales folded in, optional int6 fake-quant).
        With ``banks=False`` only the replicated tables are refreshed (the sharded optimizer pushes bank weights itself)."""
        C, p, n, d, kv = self.C, self.p, self.n, self.d, self.kv
        q = self.qat
        self.cast_generation = self.param_generation
        if banks:
            for i in range(n):       # packed [q; k; v] rows per layer
                C.cast_rows(p["qo_bank"][i], self.Wqkv[i, :d], None, 0, 1, q)
                C.cast_rows(p["kv_bank"][i], self.Wqkv[i, d:d + kv], None, 0, 1, q)
                C.cast_rows(p["kv_bank"][n + i], self.Wqkv[i, d + kv:], None, 0, 1, q)
            C.cast_rows(p["qo_bank"][n:], self.Wo, p["attn_scale"], 1, n * d, q)
            C.cast_rows(p["mlp_up_bank"], self.Wup, None, 0, 1, q)
            C.cast_rows(p["mlp_down_bank"], self.Wd, p["mlp_scale"], 1, n * d, q)
            C.cast_rows(p["qo_bank"][n:], self.Wo_u, None, 0, 1, q)
            C.cast_rows(p["mlp_down_bank"], self.Wd_u, None, 0, 1, q)
        C.cast_rows(p["tok_emb"], self.E, None, 0, 1, False)
        if not self.m.tie_embeddings:
            C.cast_rows(p["lm_head"], self.LM, None, 0, 1, False)
        if self.m.bigram.enabled:
            C.cast_rows(p["bigram_embed"], self.BE, None, 0, 1, False)
            C.cast_rows(p["bigram_proj"], self.BP, p["bigram_scale"], 0, 1, False)
        if self.m.value_embedding.enabled:
            C.cast_rows(p["ve_embed"], self.VE, None, 0, 1, False)
            torch.mul(p["ve_layer_scales"], p["ve_scale"], out=self.ve_eff)
            for li in range(self.VP.shape[0]):
                C.cast_rows(p["ve_proj"], self.VP[li], self.ve_eff[li:li + 1], 0, 1, False)

    def params_changed(self):
        self.param_generation += 1
        self.cast_weights()

    def mark_params_dirty(self):
        """Call after writing to ``self.p`` directly; the next `forward` refuses to run on the stale bf16 copies until
        `cast_weights` (or `params_changed`) has refreshed them. Same role as the reference's BF16 freshness stamps
        (``pg-model/src/gpu.rs:637-733``)."""
        self.param_generation += 1

    # ---- weight-gradient products ----------------------------------------------------------------------------------------------
    def _dw(self, dY: torch.Tensor, X: torch.Tensor, G: torch.Tensor, segs=()):
        """``G += dY^T X`` (both operands token-major; ``segs`` scatters row ranges of the result into further matrices).
        Default: one split-K launch whose CTAs add their partial tiles with fp32 `red.add` (order depends on scheduling).
        With ``train.reproducible_backward`` the reduction over tokens is cut into equal chunks computed as a BATCHED product
        into a partial buffer (one CTA per partial tile, fixed K order) and summed in ascending chunk order by a second
        kernel, so two runs give the same bits (the fixed-order fp32 reduction the reference's parity mode relies on,
        ``parameter-golf-rs/crates/pg-bench/src/bin/parity_step.rs:9-14``)."""
        if not self.t.reproducible_backward:
            N.gemm(dY, X, G, False, False, N.EPI_F32_ATOMIC, segs=segs)
            return
        T, M, Nn = dY.shape[0], dY.shape[1], X.shape[1]
        splits = 1
        for cand in (32, 16, 8, 4, 2):
            if T % cand == 0 and (T // cand) % 64 == 0:
                splits = cand
                break
        need = splits * M * Nn
        if getattr(self, "_dw_ws", None) is None or self._dw_ws.numel() < need:
            self._dw_ws = torch.empty(need, dtype=torch.float32, device=self.dev)
        ws = self._dw_ws[:need].view(splits, M, Nn)
        N.gemm(dY.unflatten(0, (splits, T // splits)), X.unflatten(0, (splits, T // splits)), ws, False, False, N.EPI_F32)
        bounds = [(G, 0)] + [(t_, r_) for r_, t_ in segs if t_ is not None]
        for i, (dst, start) in enumerate(bounds):            # row range [start, end) of every partial goes to `dst`
            self.C.sum_splits_add(self._dw_ws, start * Nn, splits, M * Nn, dst)

    # ---- Q-LoRA (test-time training) ---------------------------------------------------------------------------------------
    def set_lora(self, lora: Optional[dict]):
        """Attach (or with ``None`` detach) a low-rank adapter on the query projection: ``q += (alpha / r) (h A^T) B^T`` with
        ``A = lora["a"][layer]`` [r, d] and ``B = lora["b"][layer]`` [d, r] (fp32 masters owned by the caller, re-read on every
        forward). Counterpart of the reference's GPU Q-LoRA path (``parameter-golf-rs/crates/pg-model/src/gpu.rs:2035-2114``,
        ``:3312-3513``, LoRA GEMMs ``:3861-3999``): two skinny products through the same tcgen05 GEMM in the forward, four in the
        backward (dB, the gradient of the rank-r activations, dA, and the adapter's share of the input gradient)."""
        self.lora = lora
        if lora is None:
            return
        r = int(lora["a"].shape[1])
        if r % 8 or r > 256:
            raise ValueError("LoRA rank must be a multiple of 8 and at most 256")
        if r != self._lora_rank:
            n, d, dev = self.n, self.d, self.dev
            L = self.nact if self.train else 1
            self._lora_rank = r
            self.lora_a_bf = torch.empty(n, r, d, dtype=BF, device=dev)
            self.lora_b_bf = torch.empty(n, d, r, dtype=BF, device=dev)
            self.lora_t = [torch.empty(self.T, r, dtype=BF, device=dev) for _ in range(L)]
            if self.train:
                self.lora_dt = torch.empty(self.T, r, dtype=BF, device=dev)
                self.g_lora_a = torch.zeros(n, r, d, dtype=torch.float32, device=dev)
                self.g_lora_b = torch.zeros(n, d, r, dtype=torch.float32, device=dev)

    def _lora_refresh(self):
        self.lora_a_bf.copy_(self.lora["a"])
        self.lora_b_bf.copy_(self.lora["b"])

    def _lora_fwd(self, l, li):
        d = self.d
        s = float(self.lora["alpha"]) / self._lora_rank
        qv = self.qkv_pre[li][:, :d]
        N.gemm(self.h[li], self.lora_a_bf[l], self.lora_t[li])                                                   # t = h A^T      [T, r]
        N.gemm(self.lora_t[li], self.lora_b_bf[l], qv, epi=N.EPI_AXPBY_BF16, alpha=s, beta=1.0, aux=qv)          # q += s t B^T

    def _lora_bwd(self, l, aj):
        """Adapter gradients of layer l and the adapter's share of d_h (added in place). ``d_qkv_pre[:, :d]`` holds dL/dq_pre."""
        d = self.d
        s = float(self.lora["alpha"]) / self._lora_rank
        dq = self.d_qkv_pre[:, :d]
        A = N.EPI_F32_ATOMIC
        if self.lora.get("trainable", False):
            N.gemm(dq, self.lora_t[aj], self.g_lora_b[l], False, False, A, alpha=s)                             # dB += s dq^T t  [d, r]
        N.gemm(dq, self.lora_b_bf[l], self.lora_dt, True, False, alpha=s)                                        # d_t = s dq B    [T, r]
        if self.lora.get("trainable", False):
            N.gemm(self.lora_dt, self.h[aj], self.g_lora_a[l], False, False, A)                                  # dA += d_t^T h   [r, d]
        N.gemm(self.lora_dt, self.lora_a_bf[l], self.d_h, True, False, N.EPI_AXPBY_BF16, alpha=1.0, beta=1.0, aux=self.d_h)   # d_h += d_t A

    # ---- attention -----------------------------------------------------------------------------------------------------
    def _attn_fwd(self, l, li):
        d, kv, B, S, H, Hkv, hd = self.d, self.kv, self.B, self.S, self.H, self.Hkv, self.hd
        q = self.qk_post[li][:, :d]
        k = self.qk_post[li][:, d:d + kv]
        v = self.qkv_pre[li][:, d + kv:]
        # exclusive self attention: the projection off the token's own value vector is applied to the accumulator in the
        # attention kernel's output stage, which writes both y (the backward needs it) and z
        z = self.z[li] if l in self.m.xsa_layers() else None
        self.lse[li] = N.attn_fwd(q, k, v, self.y[li], B, S, H, Hkv, hd, self.lse[li], z, 1e-8)

    def _attn_bwd(self, l, j):
        d, kv, B, S, H, Hkv, hd = self.d, self.kv, self.B, self.S, self.H, self.Hkv, self.hd
        q = self.qk_post[j][:, :d]
        k = self.qk_post[j][:, d:d + kv]
        v = self.qkv_pre[j][:, d + kv:]
        dq, dk = self.d_qk_post[:, :d], self.d_qk_post[:, d:d + kv]
        dv = self.d_qkv_pre[:, d + kv:]
        xsa = l in self.m.xsa_layers()
        # in XSA layers `xsa_bwd` has just produced d_y and, in the same pass, the -rowsum(d_y * y) term of the single-pass form
        N.attn_bwd(q, k, v, self.y[j], self.d_y, self.lse[j], dq, dk, dv, B, S, H, Hkv, hd, accumulate_dv=xsa, dsum=self.dsum,
                   dq_acc=self.dq_acc, reproducible=self.t.reproducible_backward, dsum_ready=xsa and not self.t.reproducible_backward)

    def _block_fwd(self, j: int, x, skip, sw, recompute: bool = False):
        """Block of activation slot ``j`` on input ``x`` (with the U-Net skip it consumes, if any); returns the block output.
        ``recompute`` is the second run of a checkpointed block inside the backward pass: it refills the shared activation
        buffers and leaves out the last product, whose output is still in ``x_out[j]``."""
        C, m, p = self.C, self.m, self.p
        d, kv, S = self.d, self.kv, self.S
        l, rep = self.sched[j]
        li = self.act_slot[j] if self.train else 0
        s_l = gpt.layer_ln_scale(m, l)
        C.mix_norm_fwd(x, self.x0, skip, sw, p["resid_mix"][l], self.x_in[li], self.h[li], s_l, self.eps)
        # Per-head RMSNorm, partial RoPE and the query gain run in the output stage of the QKV product unless something has to
        # touch the raw queries first (a Q-LoRA adapter) or the shape is outside what that stage handles.
        fused_qk = self.lora is None and N.qkv_epilogue_supported(self.hd, m.rope_dims)
        wait = {}
        if self.layer_flags is not None and not recompute:
            if self.layer_wait_needed:
                # First forward after a sharded update: the layer's weights may still be on their way (this rank's own
                # Newton-Schulz chain included, which needs SMs). A one-thread kernel waits for the ready counter here, so
                # the persistent GEMM behind it never spins while holding every SM.
                C.comm_wait_flag(self.layer_flags[l:l + 1], self.layer_flag_value, N.status_word(self.dev))
                if l == self.n - 1:
                    self.layer_wait_needed = False
            wait = dict(wait_flag=self.layer_flags[l:l + 1], wait_value=self.layer_flag_value)
        if fused_qk:
            N.gemm_qkv_norm_rope(self.h[li], self.Wqkv[l], self.qkv_pre[li], self.qk_post[li], self.cos, self.sin, p["q_gain"][l], self.H, self.Hkv,
                                 m.rope_dims, S, self.eps, **wait)
        else:
            N.gemm(self.h[li], self.Wqkv[l], self.qkv_pre[li], **wait)
        if m.value_embedding.enabled and l in m.value_embedding.layers:
            vi = m.value_embedding.layers.index(l)
            vview = self.qkv_pre[li][:, d + kv:]
            N.gemm(self.ve_e, self.VP[vi], vview, epi=N.EPI_AXPBY_BF16, alpha=1.0, beta=1.0, aux=vview)
        if self.lora is not None:
            self._lora_fwd(l, li)
        if not fused_qk:
            C.qk_norm_rope_fwd(self.qkv_pre[li], self.qk_post[li], self.cos, self.sin, p["q_gain"][l], self.H, self.Hkv, self.hd, m.rope_dims, S, self.eps)
        self._attn_fwd(l, li)
        zz = self.z[li] if l in m.xsa_layers() else self.y[li]
        for gi, (wname, bname, gscale_, gmult) in enumerate(self.gates):
            out = self.yg[gi][li]
            C.head_gate_fwd(zz, self.h[li], p[wname][l], p[bname][l] if bname else None, out, self.gv[gi][li], self.H, self.hd, gscale_, gmult)
            zz = out
        self.zz[li] = zz
        N.gemm(zz, self.Wo[l], self.x_mid[li], epi=N.EPI_AXPBY_BF16, alpha=1.0, beta=1.0, aux=self.x_in[li])
        if not self.parallel:
            C.mix_norm_fwd(self.x_mid[li], None, None, None, None, None, self.mm[li], s_l, self.eps)
        N.gemm(self.mm[li], self.Wup[l], self.hu[li], epi=N.EPI_ACT_SQ, slope=self.slope, D2=self.a[li])
        xo = self.x_out[j]
        if not recompute:
            N.gemm(self.a[li], self.Wd[l], xo, epi=N.EPI_AXPBY_BF16, alpha=1.0, beta=1.0, aux=self.x_mid[li])
        return xo

    # ---- forward -------------------------------------------------------------------------------------------------------------
    def forward(self, ids: torch.Tensor, targets: Optional[torch.Tensor], gscale: float = 0.0, want_grad: bool = False):
        """Runs the model on one micro-batch. With ``want_grad`` the logits buffer ends up holding
        ``gscale * dL/dlogits``. Per-token NLL lands in ``self.nll``; the sum is added to ``self.loss_sum``."""
        C, m, p = self.C, self.m, self.p
        d, kv, S = self.d, self.kv, self.S
        if self.cast_generation != self.param_generation:
            raise RuntimeError(f"stale bf16 weights: parameters are at generation {self.param_generation}, the compute copies at "
                               f"{self.cast_generation}; call cast_weights() after changing parameters")
        if self.lora is not None:
            self._lora_refresh()
        if ids is not None:                       # otherwise self.ids / self.tgt were filled by `load_span`
            self.ids.copy_(ids.reshape(-1))
            if targets is not None and targets is not True:
                self.tgt.copy_(targets.reshape(-1))
        C.embed_gather(self.ids, self.E, self.e, 0, S, N.status_word(self.dev))
        if m.bigram.enabled:
            C.embed_gather(self.ids, self.BE, self.bg, m.bigram.vocab_size, S, N.status_word(self.dev))
            N.gemm(self.bg, self.BP, self.xe, epi=N.EPI_AXPBY_BF16, alpha=1.0, beta=1.0, aux=self.e)
        if m.value_embedding.enabled:
            C.embed_gather(self.ids, self.VE, self.ve_e, 0, S, N.status_word(self.dev))
        bid = m.smear_gate_boundary_token_id
        C.norm_smear_fwd(self.xe, p["smear_gate"] if m.smear_gate else None, self.ids if (m.smear_gate and bid is not None) else None, self.x0,
                         S, -1 if bid is None else bid, self.eps)
        x = self.x0
        skips: List[torch.Tensor] = []
        xsa_layers = m.xsa_layers()
        for j, (l, rep) in enumerate(self.sched):
            skip = sw = None
            if self.unet and l >= self.enc and rep == 0 and skips:
                skip, sw = skips.pop(), p["skip_weights"][l - self.enc]
            self.block_in[j] = (x, skip, sw)
            x = self._block_fwd(j, x, skip, sw)
            last_pass = j + 1 == self.nslots or self.sched[j + 1][0] != l
            if self.unet and l < self.enc and last_pass:
                skips.append(x)
        self.x_last = x
        C.mix_norm_fwd(x, None, None, None, None, None, self.hf, 1.0, self.eps)
        weighted = targets is not None and self.pair_w_table is not None and want_grad
        if weighted:
            # complementary training: the loss of this micro-batch is sum(w l) / sum(w), w looked up per (input, target) pair
            C.pair_weights(self.ids, self.tgt, self.pair_w_table, self.tok_w, self.w_total)
        self._head_grads_done = False
        R, T = self.logit_rows, self.T
        if R >= T or targets is None:
            logits = self.logits
            if R < T:                              # every logit was asked for: a full buffer, allocated on first use
                if self._logits_full is None:
                    self._logits_full = torch.empty(T, m.vocab_size, dtype=BF, device=self.dev)
                logits = self._logits_full
            N.gemm(self.hf, self.LM, logits)
            if targets is not None:
                C.softcap_ce(logits, self.tgt, self.nll, logits if want_grad else None, self.loss_sum, m.logit_softcap, gscale,
                             self.tok_w if weighted else None, self.w_total if weighted else None)
            return
        # Chunked head: projection, cross-entropy and (when training) the two products that consume the logits gradient, one
        # chunk of rows at a time; the [T, V] logits never exist. The backward pass then starts at the final norm.
        gW = (self.g["tok_emb"] if m.tie_embeddings else self.g["lm_head"]) if want_grad else None
        for r0 in range(0, T, R):
            r1 = min(r0 + R, T)
            lg = self.logits[:r1 - r0]
            N.gemm(self.hf[r0:r1], self.LM, lg)
            C.softcap_ce(lg, self.tgt[r0:r1], self.nll[r0:r1], lg if want_grad else None, self.loss_sum, m.logit_softcap, gscale,
                         self.tok_w[r0:r1] if weighted else None, self.w_total if weighted else None, T)
            if want_grad:
                N.gemm(lg, self.LM, self.d_h[r0:r1], True, False)          # d_hf rows
                self._dw(lg, self.hf[r0:r1], gW)
        self._head_grads_done = want_grad

    def set_token_weight_table(self, table) -> None:
        """Install (or with ``None`` remove) the ``[V, V]`` fp32 table of training-loss weights per (previous token, target)
        pair (`ops.complementary.weight_table`). Training steps then minimise the weighted mean; scoring (`want_grad=False`)
        is never weighted."""
        if table is None:
            self.pair_w_table = None
            return
        V = self.m.vocab_size
        t = torch.as_tensor(table, dtype=torch.float32).reshape(V, V).contiguous().to(self.dev)
        self.pair_w_table = t
        if self.tok_w is None:
            self.tok_w = torch.empty(self.T, dtype=torch.float32, device=self.dev)
            self.w_total = torch.zeros(1, dtype=torch.float32, device=self.dev)

    # ---- backward ---------------------------------------------------------------------------------------------------------------
    def backward(self):
        """Consumes the logits gradient left by `forward(..., want_grad=True)`; accumulates into ``self.g``."""
        C, m, p, g = self.C, self.m, self.p, self.g
        n, d, kv, S = self.n, self.d, self.kv, self.S
        A = N.EPI_F32_ATOMIC
        if not self._head_grads_done:              # the chunked head has already produced d_hf and the output-embedding gradient
            N.gemm(self.logits, self.LM, self.d_h, True, False)                              # d_hf
            self._dw(self.logits, self.hf, g["tok_emb"] if m.tie_embeddings else g["lm_head"])
        C.mix_norm_bwd(self.d_h, None, self.x_last, None, None, None, None, None, None, self.dx, None, None, None, None, False, 1.0, self.eps)
        self.d_x0.zero_()
        xsa_layers = m.xsa_layers()
        for j in range(self.nslots - 1, -1, -1):
            l, rep = self.sched[j]
            s_l = gpt.layer_ln_scale(m, l)
            aj = self.act_slot[j]
            if not self.saved[j]:
                self._block_fwd(j, *self.block_in[j], recompute=True)
            # ---- MLP
            self.Gd.zero_()
            self._dw(self.dx, self.a[aj], self.Gd)
            C.fold_scaled_grad_bf16(self.Gd, self.Wd_u[l], p["mlp_scale"][l], 1, d, g["mlp_down_bank"][l], g["mlp_scale"][l])
            N.gemm(self.dx, self.Wd[l], self.d_hu, True, False, N.EPI_MUL_ACTGRAD, slope=self.slope, aux=self.hu[aj])
            self._dw(self.d_hu, self.mm[aj], g["mlp_up_bank"][l])
            N.gemm(self.d_hu, self.Wup[l], self.d_m, True, False)
            if self.parallel:
                dx_mid, dx_next = self.dx, self.dx_mid      # no norm between x_mid and the MLP: the residual gradient passes through
                d_hx = self.d_m                             # and the MLP-input gradient joins the QKV-input gradient below
            else:
                C.mix_norm_bwd(self.d_m, self.dx, self.x_mid[aj], None, None, None, None, None, None, self.dx_mid, None, None, None, None, False, s_l, self.eps)
                dx_mid, dx_next = self.dx_mid, self.dx
                d_hx = self.d_hx if self.gates else None
            # ---- attention output projection
            zz = self.zz[aj]
            self.Go.zero_()
            self._dw(dx_mid, zz, self.Go)
            C.fold_scaled_grad_bf16(self.Go, self.Wo_u[l], p["attn_scale"][l], 1, d, g["qo_bank"][n + l], g["attn_scale"][l])
            vview = self.qkv_pre[aj][:, d + kv:]
            dv = self.d_qkv_pre[:, d + kv:]
            xsa = l in xsa_layers
            d_att = self.d_z if xsa else self.d_y            # gradient of what the gates / the output projection consumed
            N.gemm(dx_mid, self.Wo[l], d_att, True, False)
            for gi in range(len(self.gates) - 1, -1, -1):
                wname, bname, gscale_, gmult = self.gates[gi]
                gate_in = self.yg[gi - 1][aj] if gi > 0 else (self.z[aj] if xsa else self.y[aj])
                first_writer = (not self.parallel) and gi == len(self.gates) - 1
                C.head_gate_bwd(d_att, gate_in, self.h[aj], p[wname][l], self.gv[gi][aj], g[wname][l], g[bname][l] if bname else None, d_hx,
                                not first_writer, self.H, self.hd, gscale_, gmult)
            if xsa:
                if self.t.reproducible_backward:
                    C.xsa_bwd(self.d_z, self.y[aj], vview, self.d_y, dv, False, self.Hkv, self.H // self.Hkv, self.hd, 1e-8)
                else:
                    C.xsa_bwd(self.d_z, self.y[aj], vview, self.d_y, dv, False, self.Hkv, self.H // self.Hkv, self.hd, 1e-8, self.dsum, S)
            self._attn_bwd(l, aj)
            C.qk_norm_rope_bwd(self.d_qk_post, self.qkv_pre[aj], self.d_qkv_pre, self.cos, self.sin, p["q_gain"][l], g["q_gain"][l], self.H, self.Hkv,
                               self.hd, m.rope_dims, S, self.eps)
            if m.value_embedding.enabled and l in m.value_embedding.layers:
                vi = m.value_embedding.layers.index(l)
                self.Gvp.zero_()
                N.gemm(dv, self.ve_e, self.Gvp, False, False, A)                         # d(ve_eff * ve_proj)
                ds = (self.Gvp * p["ve_proj"]).sum()
                g["ve_proj"].add_(self.Gvp * self.ve_eff[vi])
                g["ve_layer_scales"][vi] += ds * p["ve_scale"][0]
                g["ve_scale"][0] += ds * p["ve_layer_scales"][vi]
                if not hasattr(self, "d_ve_e"):
                    self.d_ve_e = torch.empty_like(self.ve_e)
                    self.d_ve_acc = torch.zeros_like(self.ve_e, dtype=torch.float32)
                N.gemm(dv, self.VP[vi], self.d_ve_e, True, False)
                self.d_ve_acc.add_(self.d_ve_e)
            # one weight-gradient product for the packed QKV rows, written to the Q, K and V slots of the gradient banks
            self._dw(self.d_qkv_pre, self.h[aj], g["qo_bank"][l], segs=((d, g["kv_bank"][l]), (d + kv, g["kv_bank"][n + l])))
            if d_hx is not None:
                N.gemm(self.d_qkv_pre, self.Wqkv[l], self.d_h, True, False, N.EPI_AXPBY_BF16, alpha=1.0, beta=1.0, aux=d_hx)
            else:
                N.gemm(self.d_qkv_pre, self.Wqkv[l], self.d_h, True, False)
            if self.lora is not None:
                self._lora_bwd(l, aj)
            # ---- block input: RMSNorm backward, residual mix, U-Net skip
            x_prev = self.x_out[j - 1] if j > 0 else self.x0
            skip = sw = d_skip = d_sw = add_grad = None
            self_pair = False
            e_idx = 2 * self.enc - 1 - l                         # encoder layer whose output a decoder layer's first pass consumed
            if self.unet and l >= self.enc and rep == 0 and e_idx >= 0:
                e_slot = self.last_slot[e_idx]
                skip, sw, d_sw = self.x_out[e_slot], p["skip_weights"][l - self.enc], g["skip_weights"][l - self.enc]
                self_pair = e_slot == j - 1
                if not self_pair:
                    d_skip = self.d_skip[e_idx]
            if self.unet and j > 0:
                lp = self.sched[j - 1][0]                        # x_prev is the (last-pass) output of an encoder layer whose skip
                if lp != l and lp < self.enc and self.first_slot.get(2 * self.enc - 1 - lp, -1) not in (-1, j):   # consumer is further up
                    add_grad = self.d_skip[lp]
            C.mix_norm_bwd(self.d_h, dx_mid, self.x_in[aj], x_prev, self.x0, skip, sw, p["resid_mix"][l], add_grad, dx_next, self.d_x0, d_skip,
                           g["resid_mix"][l], d_sw, self_pair, s_l, self.eps)
            if self.parallel:
                self.dx, self.dx_mid = self.dx_mid, self.dx
            if self.backward_observer is not None:
                self.backward_observer(l, j)
        self.dx.add_(self.d_x0)
        bid = m.smear_gate_boundary_token_id
        C.norm_smear_bwd(self.dx, self.xe, p["smear_gate"] if m.smear_gate else None, self.ids if (m.smear_gate and bid is not None) else None,
                         self.d_xe, g["smear_gate"] if m.smear_gate else None, S, -1 if bid is None else bid, self.eps)
        C.embed_scatter_add(self.ids, self.d_xe, g["tok_emb"], 0, S)
        if m.bigram.enabled:
            self.Gbp.zero_()
            self._dw(self.d_xe, self.bg, self.Gbp)
            C.fold_scaled_grad(self.Gbp, p["bigram_proj"], p["bigram_scale"], 0, 1, g["bigram_proj"], g["bigram_scale"], False)
            N.gemm(self.d_xe, self.BP, self.d_bg, True, False)
            C.embed_scatter_add(self.ids, self.d_bg, g["bigram_embed"], m.bigram.vocab_size, S)
        if m.value_embedding.enabled and hasattr(self, "d_ve_acc"):
            self.d_ve_e.copy_(self.d_ve_acc)
            self.d_ve_acc.zero_()
            C.embed_scatter_add(self.ids, self.d_ve_e, g["ve_embed"], 0, S)

    # ---- public pieces -----------------------------------------------------------------------------------------------------------
    def zero_grads(self):
        if self.lora is not None and self.train:
            self.g_lora_a.zero_()
            self.g_lora_b.zero_()
        for k in gpt.BANKS:
            self.g[k].zero_()
        for grp in self.groups:
            grp["g"].zero_()
        self.loss_sum.zero_()

    def load_span(self, span_u16: torch.Tensor):
        """Upload path: a uint16 span of T+1 tokens (device tensor) is expanded into inputs and shifted targets."""
        self.C.expand_span_u16(span_u16, self.ids, self.tgt)

    def micro_step_span(self, span_u16: torch.Tensor, accum: int):
        self.load_span(span_u16)
        with nvtx_range("forward"):
            self.forward(None, True, gscale=1.0 / (self.T * accum), want_grad=True)
        with nvtx_range("backward"):
            self.backward()

    def micro_step(self, ids, targets, accum: int):
        """One micro-batch forward+backward; gradients are scaled so that `accum` of them sum to the mean."""
        with nvtx_range("forward"):
            self.forward(ids, targets, gscale=1.0 / (self.T * accum), want_grad=True)
        with nvtx_range("backward"):
            self.backward()

    def set_hp(self, lr_scale: float, momentum: float):
        self.adam_t += 1
        i = self.hp_ring_pos = (self.hp_ring_pos + 1) % len(self.hp_ring)
        if self.hp_ring_events[i] is not None:
            self.hp_ring_events[i].synchronize()          # the upload that last used this buffer has executed
        h = self.hp_host = self.hp_ring[i]
        h[0], h[1] = lr_scale, momentum
        h[2] = 1.0 - self.t.adam_beta1 ** self.adam_t
        h[3] = 1.0 - self.t.adam_beta2 ** self.adam_t
        h[4] = 1.0
        self.hp.copy_(h, non_blocking=True)
        ev = self.hp_ring_events[i] or torch.cuda.Event()
        ev.record()
        self.hp_ring_events[i] = ev

    def clip(self, extra_sumsq: Optional[torch.Tensor] = None):
        """Global-norm clip factor into hp[4] (all gradient buffers of this engine)."""
        if self.t.grad_clip_norm <= 0:
            return
        C = self.C
        for k in gpt.BANKS:
            C.sumsq(self.g[k].view(-1), 1.0, self.stats)
        for grp in self.groups:
            C.sumsq(grp["g"], 1.0, self.stats)
        C.clip_factor(self.stats, self.hp, 1.0, self.t.grad_clip_norm)

    def enable_ema(self):
        self.ema = {k: v.clone() for k, v in self.p.items() if k in gpt.BANKS}
        for gi, grp in enumerate(self.groups):
            grp["ema"] = grp["p"].clone()

    def newton_schulz(self, key: str, Bcount: Optional[int] = None) -> torch.Tensor:
        """Orthogonalise the momentum update ns[key]["U"] (bf16, NOT normalised; ns[key]["sq"] holds each matrix's sum of
        squares) and return the result buffer. The first iteration folds the normalisation X0 = U / (|U| + 1e-7) into its
        GEMM epilogues as a per-matrix factor (A = X0 X0^T = UU^T / |U|^2, X1 = a X0 + B X0 = (a U + B U) / |U|), so no
        pass over the shard is spent on dividing by the norm (the reference normalises in a kernel of its own,
        ``pg-kernels/src/gpu_kernels.rs:4520``)."""
        st = self.ns[key]
        X, Xn, Am, Bm, Xalt, sq = st["U"], st["X1"], st["A"], st["Bm"], st["X0"], st["sq"]
        if Bcount is not None:
            X, Xn, Am, Bm, Xalt, sq = X[:Bcount], Xn[:Bcount], Am[:Bcount], Bm[:Bcount], Xalt[:Bcount], sq[:Bcount]
        tall = X.shape[1] > X.shape[2]
        for s in range(self.t.muon_ns_steps):
            a, b, c = ns_coeff(self.t.muon_ns_profile, s)
            first = s == 0
            if tall:
                N.gemm(X, X, Am, False, False, batch_sumsq=sq if first else None, sumsq_pow=2)                 # A = X^T X
            else:
                N.gemm(X, X, Am, True, True, batch_sumsq=sq if first else None, sumsq_pow=2)                   # A = X X^T
            N.gemm(Am, Am, Bm, True, True, N.EPI_AXPBY_BF16, alpha=c, beta=b, aux=Am)    # B = b A + c A A   (A symmetric)
            if tall:
                N.gemm(X, Bm, Xn, True, True, N.EPI_AXPBY_BF16, alpha=1.0, beta=a, aux=X, batch_sumsq=sq if first else None)    # X = a X + X B
            else:
                N.gemm(Bm, X, Xn, True, False, N.EPI_AXPBY_BF16, alpha=1.0, beta=a, aux=X, batch_sumsq=sq if first else None)   # X = a X + B X
            X, Xn = Xn, (Xalt if first else X)           # U itself is never overwritten: later iterations ping-pong between X1 and X0
        return X

    def optimizer_step(self):
        """Replicated step: AdamW on the flat groups, Muon on the banks, then refresh the bf16 weights."""
        C, t = self.C, self.t
        decay = t.ema_decay
        for grp in self.groups:
            if grp["p"].numel():
                C.adamw(grp["p"], grp["g"], grp["m"], grp["v"], grp.get("ema"), self.hp, grp["lr"], t.adam_beta1, t.adam_beta2, t.adam_eps, t.adam_wd, decay)
        for k in gpt.BANKS:
            st = self.ns[k]
            st["sq"].zero_()
            C.muon_momentum(self.g[k], self.mom[k], st["U"], st["sq"], self.hp, True)
            X = self.newton_schulz(k)
            scale = max(1.0, self.p[k].shape[-2] / self.p[k].shape[-1]) ** 0.5
            C.muon_apply(self.p[k].view(-1), X.view(-1), self.ema[k].view(-1) if self.ema else None, self.hp, t.matrix_lr, t.muon_wd, scale, decay)
        self.param_generation += 1
        self.cast_weights()

    def export_params(self, ema: bool = False) -> Dict[str, torch.Tensor]:
        out = {}
        for k, v in self.p.items():
            out[k] = v.detach().float().cpu().clone()
        if ema and self.train and self.ema is not None:
            for k in gpt.BANKS:
                out[k] = self.ema[k].detach().cpu().clone()
            for grp in self.groups:
                off = 0
                for k in grp["names"]:
                    nel = self.p[k].numel()
                    out[k] = grp["ema"][off:off + nel].view(self.p[k].shape).detach().cpu().clone()
                    off += -(-nel // 4) * 4
        return out

    def load_params(self, params: Dict[str, torch.Tensor]):
        for k, v in params.items():
            self.p[k].copy_(v.to(self.dev, torch.float32))
        self.param_generation += 1
        self.cast_weights()


class EngineRunner:
    """Runner interface (see `parameter_golf_b200.models.runner`) on the CUDA engine, for evaluation and TTT."""

    def __init__(self, spec: RunSpec, params: Dict[str, torch.Tensor], device, batch: Optional[int] = None, train: bool = True):
        self.spec, self.model = spec, spec.model
        self.device = torch.device(device)
        self.batch = batch or spec.eval.batch_windows
        self.engines: Dict[Tuple[int, int], CudaEngine] = {}
        self._params = {k: v.detach().float() for k, v in params.items()}
        self.train = train
        self.lora = None

    MAX_LIVE_SHAPES = 3

    def _engine(self, B: int, S: int) -> CudaEngine:
        """Engine for a batch shape. All shapes of one runner alias the first engine's parameters and bf16 weights
        (`CudaEngine(share=...)`), so switching between the scoring and the training shape costs nothing; the least recently
        created activation set is dropped beyond `MAX_LIVE_SHAPES`."""
        key = (B, S)
        if key not in self.engines:
            if not self.engines:
                self.engines[key] = CudaEngine(self.spec, self._params, self.device, B, S, train=self.train)
            else:
                first = next(iter(self.engines.values()))
                if len(self.engines) >= self.MAX_LIVE_SHAPES:
                    del self.engines[list(self.engines)[1]]           # never the first: it owns nothing the others lack, but keeps order simple
                self.engines[key] = CudaEngine(self.spec, None, self.device, B, S, train=self.train, share=first)
        return self.engines[key]

    @property
    def params(self):
        if self.engines:
            return next(iter(self.engines.values())).p
        return self._params

    def params_changed(self):
        es = list(self.engines.values())
        if es:
            es[0].cast_weights()                 # every shape aliases the same bf16 weight buffers
            for e in es[1:]:
                e.cast_generation = e.param_generation

    @torch.no_grad()
    def nll(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        e = self._engine(ids.shape[0], ids.shape[1])
        e.set_lora(self.lora)
        e.forward(ids.to(self.device, torch.int32), targets.to(self.device, torch.int32))
        return e.nll.view(ids.shape).clone()

    @torch.no_grad()
    def logits(self, ids: torch.Tensor) -> torch.Tensor:
        e = self._engine(ids.shape[0], ids.shape[1])
        e.set_lora(self.lora)
        e.forward(ids.to(self.device, torch.int32), None)
        z = (e.logits if e.logit_rows >= e.T else e._logits_full).view(*ids.shape, -1).float()
        return self.model.logit_softcap * torch.tanh(z / self.model.logit_softcap)

    @torch.no_grad()
    def loss_and_grads(self, ids, targets, qat: bool = False, names=None):
        e = self._engine(ids.shape[0], ids.shape[1])
        if e.qat != qat:
            e.qat = qat
            e.cast_weights()
        e.set_lora(self.lora)
        e.zero_grads()
        e.micro_step(ids.to(self.device, torch.int32), targets.to(self.device, torch.int32), 1)
        loss = e.loss_sum[0] / e.T
        names = list(e.g) if names is None else list(names)
        grads = {k: e.g[k] for k in names}
        if self.lora is not None and self.lora.get("trainable", False):
            grads["lora.a"], grads["lora.b"] = e.g_lora_a, e.g_lora_b
        return loss.clone(), grads


class EngineBackend:
    """Training backend used by `parameter_golf_b200.train.VariantRunner` for the CUDA backends."""

    def __init__(self, spec: RunSpec, params: Dict[str, torch.Tensor], overlap_optimizer: bool = True):
        import os
        from ..train import step_batch_plan
        self.spec = spec
        t = spec.train
        self.device = torch.device(f"cuda:{int(os.environ.get('LOCAL_RANK', 0))}")
        torch.cuda.set_device(self.device)
        tokens, accum = step_batch_plan(spec, spec.mode)
        micro_tokens = tokens // (t.world_size * accum)
        self.accum = accum
        self.engine = CudaEngine(spec, params, self.device, micro_tokens // t.seq_len, t.seq_len, train=True)
        if t.ema_decay > 0:
            self.engine.enable_ema()
        self.dist = None
        if t.world_size > 1:
            from ..parallel.dist_engine import DistributedStep
            self.dist = DistributedStep(self.engine, spec, overlap=overlap_optimizer)

    def set_token_weight_table(self, table) -> None:
        self._graph_state = None      # a captured micro-step would keep replaying the unweighted loss kernel
        self.engine.set_token_weight_table(table)

    def train_step(self, batches, lr_scale: float, momentum: float, qat: bool) -> float:
        e = self.engine
        if qat != e.qat:
            e.qat = qat
            e.cast_weights()
        e.zero_grads()
        e.set_hp(lr_scale, momentum)
        for i, (ids, tgt) in enumerate(batches):
            if self.dist is not None and i == len(batches) - 1:
                self.dist.arm()            # the last backward hands finished layers to the gradient reduction
            e.micro_step(ids.to(self.device, torch.int32, non_blocking=True), tgt.to(self.device, torch.int32, non_blocking=True), len(batches))
        if self.dist is not None:
            self.dist.step()
        else:
            e.clip()
            e.optimizer_step()
        return self._read_loss_and_status(len(batches))

    def host_spans(self, count: int):
        """Pinned host staging buffers for `count` micro-batch spans of T+1 uint16 tokens (stored as int16)."""
        if not hasattr(self, "_span_host") or len(self._span_host) < count:
            self._span_host = [torch.empty(self.engine.T + 1, dtype=torch.int16).pin_memory() for _ in range(count)]
        return self._span_host[:count]

    def stage_spans(self, spans):
        """Copy uint16 spans (pinned host or device tensors of T+1 tokens, viewed as int16) into device staging buffers."""
        e = self.engine
        if not hasattr(self, "_span_dev") or len(self._span_dev) < len(spans):
            self._span_dev = [torch.empty(e.T + 1, dtype=torch.int16, device=self.device) for _ in range(len(spans))]
        for dst, src in zip(self._span_dev, spans):
            dst.copy_(src, non_blocking=True)
        return self._span_dev[:len(spans)]

    def train_step_spans(self, spans, lr_scale: float, momentum: float, qat: bool = False, read_loss: bool = True, staged: bool = False):
        """One optimizer step from `len(spans)` micro-batches given as uint16 token spans of T+1 tokens each.
        ``staged`` means the spans already live on this device. Returns the mean loss (host float) when ``read_loss``."""
        e = self.engine
        if qat != e.qat:
            e.qat = qat                 # every rank must flip at the same step (the trainer agrees on the LR scale first)
            if self.dist is not None:
                self.dist.repush_weights()
            else:
                e.cast_weights()
        e.zero_grads()
        e.set_hp(lr_scale, momentum)
        dev_spans = spans if staged else self.stage_spans(spans)
        for i, sp in enumerate(dev_spans):
            if self.dist is not None and i == len(dev_spans) - 1:
                self.dist.arm()            # the last backward hands finished layers to the gradient reduction
            if self.spec.train.cuda_graph and e.layer_flags is None:
                self._graphed_micro_step(sp, len(dev_spans))
            else:
                e.micro_step_span(sp, len(dev_spans))
        with nvtx_range("optimizer"):
            if self.dist is not None:
                self.dist.step()
            else:
                e.clip()
                e.optimizer_step()
        if read_loss:
            return self._read_loss_and_status(len(dev_spans))
        return None

    def _read_loss_and_status(self, micro_batches: int) -> float:
        """One device->host read of the loss and of the bounded-wait status word. A wait that ran out inside the step (a
        barrier, a gradient or weight-ready flag a peer never set) leaves wrong gradients or weights behind it, so it must
        end the run here: the caller holds `RankHealth.guard()`, which reports the exception to the peers."""
        e = self.engine
        st = N.status_word(self.device)
        if not hasattr(self, "_readback"):
            self._readback = torch.zeros(8, dtype=torch.float32).pin_memory()
        rb = self._readback
        rb[:1].copy_(e.loss_sum[:1], non_blocking=True)
        rb[4:8].view(torch.int32).copy_(st, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        code, block, detail, count = rb[4:8].view(torch.int32).tolist()
        if code:
            st.zero_()
            raise RuntimeError(N.status_message(code, block, detail, count).replace("kernel wait timed out", "kernel wait timed out during the training step")
                               + "; gradients or weights of this step are not trustworthy")
        return float(rb[0]) / (e.T * micro_batches)

    def _graphed_micro_step(self, span: torch.Tensor, accum: int):
        """Forward+backward of one micro-batch replayed from a CUDA graph. The engine allocates nothing per step and
        every kernel argument is a fixed device address (hyper-parameters live in the device array ``hp``), so the
        ~900 launches of a micro-batch are captured once per accumulation count and replayed; the span is copied into
        a static staging buffer first. The first call runs eagerly (it also warms every lazily created buffer), the
        second captures. Same idea as the reference's captured no-loss backward
        (``parameter-golf-rs/crates/pg-train/src/lib.rs:2063-2133``), extended to the whole micro-step.
        The sharded optimizer's weight-ready counters are compared against a host-side step count, so that path stays
        eager (see `CudaEngine.forward`)."""
        e = self.engine
        st = getattr(self, "_graph_state", None)
        if st is None or st["accum"] != accum:
            st = self._graph_state = {"accum": accum, "graph": None, "calls": 0,
                                      "span": torch.empty(e.T + 1, dtype=torch.int16, device=self.device)}
        st["span"].copy_(span, non_blocking=True)
        if st["calls"] == 0:
            n0 = N.launch_count()
            e.micro_step_span(st["span"], accum)
            st["kernels"] = N.launch_count() - n0          # kernel nodes of one replay, for the launch counter
        else:
            if st["graph"] is None:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    e.micro_step_span(st["span"], accum)
                st["graph"] = g
            st["graph"].replay()
            N.load().launches += st["kernels"]
        st["calls"] += 1

    fused_ema = True

    def sync_params(self):
        return self.engine.p

    def final_params(self, ema: bool = False):
        """CPU fp32 parameter dict (EMA weights when requested), with sharded banks gathered from their owners."""
        e = self.engine
        if self.dist is not None and self.dist.sharded:
            for k, v in self.dist.gather_banks(e.p).items():
                e.p[k].copy_(v)
            if ema and e.ema is not None:
                for k, v in self.dist.gather_banks(e.ema).items():
                    e.ema[k].copy_(v)
        return e.export_params(ema=ema)

    def params_changed(self):
        self.engine.cast_weights()

    def state_dict(self):
        """Full optimizer state on the host. A COLLECTIVE when the optimizer is sharded: every rank must call it at the same
        step, because the fp32 master weights, the momentum and the EMA shadow of a bank slot are current only on the rank
        that owns the slot and are gathered from the owners here (the master weights land in ``engine.p``, which the
        caller saves next)."""
        e = self.engine
        mom = e.mom
        ema_banks = e.ema
        if self.dist is not None and self.dist.sharded:
            for k, v in self.dist.gather_banks(e.p).items():
                e.p[k].copy_(v)
            mom = self.dist.gather_banks(e.mom)
            if e.ema is not None:
                ema_banks = self.dist.gather_banks(e.ema)
        st = {"mom": {k: v.cpu() for k, v in mom.items()}, "adam_t": e.adam_t,
              "m": [g["m"].cpu() for g in e.groups], "v": [g["v"].cpu() for g in e.groups]}
        if e.ema is not None:
            st["ema_banks"] = {k: v.cpu() for k, v in ema_banks.items()}
            st["ema_groups"] = [g["ema"].cpu() for g in e.groups]
        return st

    def load_state_dict(self, st):
        e = self.engine
        for k, v in st["mom"].items():
            e.mom[k].copy_(v)
        e.adam_t = int(st["adam_t"])
        for g, mm, vv in zip(e.groups, st["m"], st["v"]):
            g["m"].copy_(mm)
            g["v"].copy_(vv)
        if e.ema is not None:
            if "ema_banks" not in st:
                raise RuntimeError("the checkpoint holds no EMA state but this run averages weights (train.ema_decay > 0)")
            for k, v in st["ema_banks"].items():
                e.ema[k].copy_(v)
            for g, sh in zip(e.groups, st["ema_groups"]):
                g["ema"].copy_(sh)
