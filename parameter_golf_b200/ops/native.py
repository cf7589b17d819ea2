"""Loader of the native extension and thin Python entry points over it.

The extension is built in-tree (`parameter_golf_b200.ops.build`). On a machine with a GPU a missing or stale
library is an error after one rebuild attempt: there is no fallback implementation of the CUDA ops.
"""
from __future__ import annotations

import importlib
import importlib.util
import os

import torch

from . import build as _build

_C = None

EPI_BF16, EPI_F32, EPI_F32_ATOMIC, EPI_AXPBY_BF16, EPI_RESID_BF16, EPI_ACT_SQ, EPI_MUL_ACTGRAD = range(7)

STATUS_NAMES = {0: "ok", 1: "wait_full", 2: "wait_empty", 3: "wait_tmem_full", 4: "wait_tmem_empty", 5: "wait_flag", 6: "bad_arg", 7: "wait_misc",
                8: "bad_index"}


def status_message(code: int, block: int, detail: int, count: int) -> str:
    """What a non-zero status word means, for the exception the host raises."""
    if code == 8:
        return (f"a token id outside its embedding table reached a kernel (row {detail} of the micro-batch, {count} reports); "
                f"the row was read as zeros. Check the shards against model.vocab_size")
    return f"kernel wait timed out: {STATUS_NAMES.get(code, code)} (block {block}, detail {detail}, {count} reports)"


def load():
    """Import (building if needed) and return the extension module."""
    global _C
    if _C is not None:
        return _C
    if not _build.is_current():
        _build.build()
    spec = importlib.util.spec_from_file_location("parameter_golf_b200._C", _build.LIB)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _C = _Counting(mod)
    return _C


class _Counting:
    """Forwards to the extension and counts kernel launches issued through it (`launch_count`)."""

    _PER_CALL = {"attn_bwd": 2, "attn_bwd_fused": 3}

    def __init__(self, mod):
        self._mod = mod
        self.launches = 0
        self.timing = None           # list of (key, start event, end event) while per-op timing is on

    def __getattr__(self, name):
        fn = getattr(self._mod, name)
        n = self._PER_CALL.get(name, 1)

        def call(*a, **k):
            # the single-pass attention backward skips its first kernel when the caller supplies the per-query term
            self.launches += n - 1 if (name == "attn_bwd_fused" and len(a) >= 19 and a[18]) else n
            if self.timing is None:
                return fn(*a, **k)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*a, **k)
            e1.record()
            self.timing.append((_timing_key(name, a, k), e0, e1))
            return out

        self.__dict__[name] = call
        return call


_EPI_NAMES = {0: "bf16", 1: "f32", 2: "f32_atomic", 3: "axpby", 4: "resid", 5: "act_sq", 6: "mul_actgrad"}


def _timing_key(name, a, k):
    if name == "gemm":           # (A, B, D, a_kmajor, b_kmajor, epi, ...): tell the products of the step apart
        A, B, D = a[0], a[1], a[2]
        kdim = A.shape[-1] if a[3] else A.shape[-2]
        mdim = A.shape[-2] if a[3] else A.shape[-1]
        seg = f" M={mdim} (row segments)" if len(a) > 17 and a[17] is not None else ""
        return f"gemm {_EPI_NAMES.get(int(a[5]), a[5])} N={D.shape[-1]} K={kdim} {'T' if a[3] else 'N'}{'T' if a[4] else 'N'}{seg}"
    return name


def enable_timing(on: bool = True) -> None:
    """Per-op device timing: every call through the extension is bracketed by two CUDA events on the current stream
    (no synchronisation is added; `timing_report` reads them afterwards). A development aid for step breakdowns."""
    load().timing = [] if on else None


def timing_report(reset: bool = True):
    """{key: (calls, total_ms)} of the calls recorded since `enable_timing`."""
    C = load()
    torch.cuda.synchronize()
    out = {}
    for key, e0, e1 in C.timing or []:
        c, t = out.get(key, (0, 0.0))
        out[key] = (c + 1, t + e0.elapsed_time(e1))
    if reset and C.timing is not None:
        C.timing = []
    return out


def load_raw():
    """The extension module itself (classes and host-only helpers; nothing here counts as a kernel launch)."""
    return load()._mod


def launch_count() -> int:
    return 0 if _C is None else _C.launches


def available() -> bool:
    return os.path.exists(_build.LIB)


_status = {}


def status_word(device=None) -> torch.Tensor:
    """Per-device int32[4] status word that bounded waits write to: [code, block, detail, count]."""
    dev = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
    if dev.type == "cuda" and dev.index is None:          # "cuda" and "cuda:N" must name the same word
        dev = torch.device("cuda", torch.cuda.current_device())
    if dev not in _status:
        _status[dev] = torch.zeros(4, dtype=torch.int32, device=dev)
    return _status[dev]


def check_status(device=None, reset: bool = True):
    """Raise if any kernel recorded a timed-out wait or a rejected index since the last check (synchronises the device)."""
    st = status_word(device)
    code, block, detail, count = st.tolist()
    if reset and code:
        st.zero_()
    if code:
        raise RuntimeError(status_message(code, block, detail, count))


def gemm(A, B, D, a_kmajor=True, b_kmajor=True, epi=EPI_BF16, alpha=1.0, beta=0.0, slope=0.0, aux=None, colscale=None, D2=None, splits=0,
         wait_flag=None, wait_value=0, segs=(), batch_sumsq=None, sumsq_pow=1):
    """``segs``: up to two ``(first_row, tensor)`` pairs; with an fp32 epilogue the output rows from ``first_row`` on land in that
    tensor instead of ``D`` (one product feeding several gradient matrices).
    ``batch_sumsq``: fp32 ``[batch]``; the output of batch ``b`` (alpha and beta terms alike) is scaled by
    ``(1 / (sqrt(batch_sumsq[b]) + 1e-7)) ** sumsq_pow``."""
    s0 = segs[0] if len(segs) > 0 else (0, None)
    s1 = segs[1] if len(segs) > 1 else (0, None)
    load().gemm(A, B, D, a_kmajor, b_kmajor, epi, alpha, beta, slope, aux, colscale, D2, splits, status_word(A.device), wait_flag, wait_value,
                s0[0], s0[1], s1[0], s1[1], batch_sumsq, sumsq_pow)
    return D


def gemm_qkv_norm_rope(h, W, pre, post, cos, sin, gain, H, Hkv, rope_dims, seq_len, eps, wait_flag=None, wait_value=0):
    """QKV projection whose output stage also applies the per-head RMSNorm, the partial RoPE and the query gain: ``pre`` = h W^T
    for all heads (the backward of the norm and the attention read it), ``post`` = the normalised, rotated, gain-scaled query
    and key heads. Heads of 64; ``rope_dims`` in {0, 16, 32, 64}."""
    load().gemm_qkv_norm_rope(h, W, pre, post, cos, sin, gain, H, Hkv, rope_dims, seq_len, eps, status_word(h.device), wait_flag, wait_value)
    return post


def qkv_epilogue_supported(hd, rope_dims):
    return hd == 64 and rope_dims in (0, 16, 32, 64)


def attn_fwd(q, k, v, y, B, S, H, Hkv, hd, lse=None, z=None, xsa_eps=1e-8):
    """Causal GQA attention forward; q/k/v are [B*S, heads*hd] (row-strided views allowed). Returns the side output [B, H, S] = -(log2-domain log-sum-exp), which `attn_bwd` consumes.
    With ``z`` the kernel also writes the exclusive-self-attention output z_h = y_h - (<y_h, v> / (|v|^2 + eps)) v from the
    accumulator it already holds (`xsa_fwd` as a separate pass is then not needed)."""
    if lse is None:
        lse = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
    load().attn_fwd(q, k, v, y, lse, B, S, H, Hkv, hd, status_word(q.device), z, xsa_eps)
    return lse


_DQ_ACC = {}


def attn_dq_scratch(device, B, S, H, hd=64):
    """Zero-filled fp32 accumulator of the single-pass attention backward, one per device, grown on demand. The kernels
    leave it zero, so every call on the device can share it (calls on one device are stream-ordered)."""
    need = B * H * S * hd
    key = torch.device(device).index
    buf = _DQ_ACC.get(key)
    if buf is None or buf.numel() < need:
        buf = torch.zeros(need, dtype=torch.float32, device=device)
        _DQ_ACC[key] = buf
    return buf


def attn_bwd(q, k, v, o, d_o, lse, dq, dk, dv, B, S, H, Hkv, hd, accumulate_dv=False, dsum=None, dq_acc=None, reproducible=False,
             dsum_ready=False):
    """Causal GQA attention backward. Writes dq, dk and dv (dv is added to when ``accumulate_dv``).

    Default: the single-pass kernel (scores computed once per tile pair; dQ summed in an fp32 accumulator with `red.add`,
    so its last fp32 bits depend on scheduling). ``reproducible=True`` runs the two-kernel form, which recomputes the
    scores for dQ and is bit-reproducible. ``dsum_ready``: ``dsum`` already holds -rowsum(d_o * o) (`xsa_bwd` writes it on
    request), so the single-pass form skips its own pass over d_o and o."""
    if dsum is None:
        dsum_ready = False
        dsum = torch.empty(B, H, S, dtype=torch.float32, device=q.device)
    if reproducible:
        load().attn_bwd(q, k, v, o, d_o, lse, dsum, dq, dk, dv, B, S, H, Hkv, hd, accumulate_dv, status_word(q.device))
        return dsum
    if dq_acc is None:
        dq_acc = attn_dq_scratch(q.device, B, S, H, hd)
    load().attn_bwd_fused(q, k, v, o, d_o, lse, dsum, dq_acc, dq, dk, dv, B, S, H, Hkv, hd, accumulate_dv, status_word(q.device), dsum_ready)
    return dsum


def gptq_rows(Wp, U, scales, bits, block=128):
    """GPTQ row kernel (one clip candidate): int8 codes for the permuted rows ``Wp`` given the Cholesky factor ``U``."""
    if block != 128:
        raise ValueError("the GPTQ kernel works on 128-column blocks")
    Q = torch.empty(Wp.shape, dtype=torch.int8, device=Wp.device)
    load().gptq_rows(Wp.contiguous().float(), U.contiguous().float(), scales.contiguous().float(), Q, bits)
    return Q
