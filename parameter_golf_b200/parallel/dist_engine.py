"""Distributed optimizer step on peer memory: sharded Parallel Muon and the replicated all-reduce variant.

Sharded Parallel Muon (``distributed_optimizer_backend = "sharded_parallel_muon"``). Three kinds of streams: the main
stream runs forward and backward; one communication stream runs the gradient reduction and the replicated part of the
optimizer; one stream per bank runs that bank's Muon chain. Events hand work from one to the next, and every
cross-rank dependency is a counter in the symmetric signal pad that the consuming kernel polls itself (bounded), so no
global barrier is left in the step.

During the backward pass of the last micro-batch (`backward_observer`):

1. as soon as a layer's backward is queued, the communication stream bumps that layer's "gradients final" counter on
   every rank (`comm_flag_add`, release at system scope) and queues one `comm_reduce_peers` per bank slot of the layer
   that this rank owns. The kernel waits for the counter to reach ``world * step``, then sums the slot straight out of
   every peer's fp32 gradient buffer (reduce-scatter, 1/world scale and global-norm partial in one pass) into a
   reduced-shard buffer of its own. The NVLink traffic of layer l hides under the backward of layers l-1 .. 0.

After the last backward:

2. the same for the small replicated gradients (one-shot all-reduce, gated by a "tail" counter);
3. `comm_scalar_allreduce`: exact global gradient norm; it also tells every rank that its gradients were consumed;
4. clip factor, AdamW on the replicated parameters (identical on every rank), refresh of their bf16 copies. The main
   stream waits for this point only, then starts the next step;
5. per bank, on the bank's own stream: clip factor + momentum + Nesterov + sum of squares in one kernel writing the
   bf16 Newton-Schulz input, Newton-Schulz with the normalisation folded into its first products, update of the owned
   fp32 master slots, and `comm_push_cast_slots`: the owner writes the new bf16 compute weights (packed QKV rows, output
   scales folded in, optional int6 fake-quant) into EVERY rank's weight buffer and bumps that layer's ready counter on
   every rank. The four chains are independent and their GEMMs are tiny (a few tiles each), so they run side by side.
6. the next forward polls each layer's ready counter: a one-thread kernel in front of the layer's QKV GEMM the first
   time after an update (a persistent GEMM that spun on the counter itself would hold every SM while this rank's own
   Newton-Schulz kernels still need some), and the GEMM's producer warp again before its first TMA load (free by then).

Ownership follows the reference: a bank of B slots is padded to a multiple of world and cut in contiguous chunks of
``ceil(B/world)`` slots (``parameter-golf-rs/crates/pg-train/src/lib.rs:577-591,733-813``; Python
``records/track_10min_16mb/2026-03-23_LeakyReLU_LegalTTT_ParallelMuon/train_gpt.py:152-166``). The overlap of the
reduction with the backward is the reference's ``after_layer`` observer (``pg-train/src/lib.rs:3155-3243``), the
apply-when-it-lands schedule its Python record's (``…/train_gpt.py:172-266``).

The replicated variant all-reduces every gradient with the same kernels (two-shot for the banks) and then runs the
single-GPU optimizer on every rank.
"""
from __future__ import annotations

import math
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist

from ..models import gpt
from ..ops import native as N
from ..spec import RunSpec
from .symm import SymmetricBuffer

BF = torch.bfloat16
SIG_BARRIER, SIG_SCALAR, SIG_BARRIER2, SIG_LAYER, SIG_GRAD = 0, 32, 64, 128, 512      # slots in the int32 signal pad


from ..optim.muon import shard_range  # noqa: E402,F401  ([start, end) slots of a bank owned by a rank; shared with the CPU-rank form)


def slot_layer(bank: str, s: int, n: int) -> int:
    """The layer whose ready counter slot ``s`` of ``bank`` bumps when its new weights have been pushed. ``qo_bank`` holds the
    ``n`` query matrices and then the ``n`` output projections, ``kv_bank`` the keys and then the values, the MLP banks one
    matrix per layer; every layer therefore collects six bumps per step, from whichever ranks own those slots."""
    if bank in ("qo_bank", "kv_bank"):
        return s % n
    return s


class DistributedStep:
    def __init__(self, engine, spec: RunSpec, group=None, overlap: bool = True):
        """``overlap=False`` queues the whole sharded step on the caller's stream after the backward pass (the serial
        schedule; kept so that the overlap can be measured against it, `bench/dist_tail_profile.py`)."""
        self.e, self.spec, self.group = engine, spec, group
        self.overlap = overlap
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.sharded = spec.train.distributed_optimizer_backend == "sharded_parallel_muon"
        self.C = N.load()
        self.epoch = 0
        self.steps_done = 0
        self.repushes = 0
        e = engine
        # ---- re-home gradients into one symmetric fp32 region: [banks ... | flat groups ...] ---------------------
        self.g_off: Dict[str, int] = {}
        off = 0
        for k in gpt.BANKS:
            self.g_off[k] = off
            off += e.g[k].numel()
        self.grp_off: List[int] = []
        for grp in e.groups:
            self.grp_off.append(off)
            off += grp["g"].numel()
        self.g_total = off
        self.gbuf = SymmetricBuffer(off * 4, group)
        for k in gpt.BANKS:
            new = self.gbuf.view(self.g_off[k] * 4, e.g[k].shape, torch.float32)
            new.copy_(e.g[k])
            e.g[k] = new
        for gi, grp in enumerate(e.groups):
            flat = self.gbuf.view(self.grp_off[gi] * 4, (grp["g"].numel(),), torch.float32)
            flat.copy_(grp["g"])
            grp["g"] = flat
            o = 0
            for name in grp["names"]:
                nel = e.p[name].numel()
                e.g[name] = flat[o:o + nel].view(e.p[name].shape)
                o += -(-nel // 4) * 4
            grp["g_red"] = torch.zeros_like(flat) if self.sharded else flat
        # ---- re-home the bf16 bank weights into a symmetric region -------------------------------------------------------
        self.w_off: Dict[str, int] = {}
        off = 0
        for name in ("Wqkv", "Wo", "Wup", "Wd", "Wo_u", "Wd_u"):
            self.w_off[name] = off
            off += getattr(e, name).numel()
        self.wbuf = SymmetricBuffer(off * 2, group)
        for name in ("Wqkv", "Wo", "Wup", "Wd", "Wo_u", "Wd_u"):
            old = getattr(e, name)
            new = self.wbuf.view(self.w_off[name] * 2, old.shape, BF)
            new.copy_(old)
            setattr(e, name, new)
        self.sig = SymmetricBuffer(1024 * 4, group)
        self.val = SymmetricBuffer(256 * 4, group)
        self.sig_local = self.sig.view(0, (1024,), torch.int32)
        e.layer_flags = self.sig_local[SIG_LAYER:SIG_LAYER + e.n] if self.sharded else None
        e.layer_flag_value = 0
        self.own = {k: shard_range(e.p[k].shape[0], self.rank, self.world) for k in gpt.BANKS}
        # one descriptor row per owned slot: where its bf16 rows go on every rank, where the un-scaled twin goes, which row
        # scales apply, and which per-layer ready counter it bumps; a whole bank shard is then pushed by one launch
        self.push_desc: Dict[str, torch.Tensor] = {}
        if self.sharded:
            for k in gpt.BANKS:
                s0, s1 = self.own[k]
                rows = [self._slot_desc(k, s) for s in range(s0, s1)]
                self.push_desc[k] = torch.tensor(rows, dtype=torch.int64, device="cuda").reshape(-1, 4)
        if self.sharded:
            self._init_overlap()
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def _init_overlap(self):
        """Streams, events and buffers of the overlapped sharded step."""
        e = self.e
        dev = e.dev
        self.bank_order = sorted(gpt.BANKS, key=lambda b: -e.p[b].numel())
        if self.overlap:
            self.comm_stream = torch.cuda.Stream(device=dev, priority=-1)
            self.bank_streams = {k: torch.cuda.Stream(device=dev, priority=-1) for k in self.bank_order}
        else:
            self.comm_stream = torch.cuda.current_stream(dev)
            self.bank_streams = {k: self.comm_stream for k in self.bank_order}
        self.ev_layer = [torch.cuda.Event() for _ in range(e.n + 1)]          # index n: end of the backward pass
        self.ev_clip, self.ev_adam = torch.cuda.Event(), torch.cuda.Event()
        self.ev_bank = {k: torch.cuda.Event() for k in self.bank_order}
        self.bank_pending = False
        # reduced gradients of the owned slots: the symmetric gradient buffer itself is zeroed by the next step while the
        # bank chains may still be reading
        self.red = {}
        for k in gpt.BANKS:
            s0, s1 = self.own[k]
            self.red[k] = torch.zeros((max(s1 - s0, 0),) + tuple(e.p[k].shape[1:]), dtype=torch.float32, device=dev)
        # which owned slots belong to which layer
        n = e.n
        self.layer_slots = [[] for _ in range(n)]
        for k in gpt.BANKS:
            s0, s1 = self.own[k]
            for sl in range(s0, s1):
                self.layer_slots[sl % n].append((k, sl))
        self.first_slot_of_layer = {}
        for j, (l, _) in enumerate(e.sched):
            self.first_slot_of_layer.setdefault(l, j)
        # hyper-parameters are double-buffered: the bank chains of step t still read theirs while step t + 1 uploads
        self.hp_pair = [e.hp, e.hp.clone()]
        self.armed = False
        self.timing = None          # list of (name, event) while per-phase timing is on (`enable_timing`)

    # ---- pieces ------------------------------------------------------------------------------------------------------------
    def _barrier(self, slot):
        self.C.comm_barrier(self.sig.table, self.rank, self.world, slot, self.epoch, N.status_word())

    def _slot_desc(self, bank: str, s: int):
        """(destination offset, un-scaled twin offset or -1, address of the row scales or 0, ready-counter index) of a slot."""
        e = self.e
        n, d, kv, mlp = e.n, e.d, e.kv, e.mlp
        per = e.p[bank][0].numel()
        layer = slot_layer(bank, s, n)
        flag = SIG_LAYER + layer
        if bank == "qo_bank" and s < n:
            return [self.w_off["Wqkv"] + s * e.qkvw * d, -1, 0, flag]
        if bank == "qo_bank":
            return [self.w_off["Wo"] + layer * d * d, self.w_off["Wo_u"] + layer * per, e.p["attn_scale"][layer].data_ptr(), flag]
        if bank == "kv_bank":
            return [self.w_off["Wqkv"] + layer * e.qkvw * d + (d if s < n else d + kv) * d, -1, 0, flag]
        if bank == "mlp_up_bank":
            return [self.w_off["Wup"] + s * mlp * d, -1, 0, flag]
        return [self.w_off["Wd"] + s * d * mlp, self.w_off["Wd_u"] + s * per, e.p["mlp_scale"][s].data_ptr(), flag]

    def _push_bank(self, bank: str):
        """Write the bf16 compute rows of every owned slot of ``bank`` into every rank (one launch) and bump the ready
        counters of the layers they belong to (one more)."""
        s0, s1 = self.own[bank]
        if s1 <= s0:
            return
        e, C = self.e, self.C
        C.comm_push_cast_slots(e.p[bank][s0:s1], self.wbuf.table, self.world, self.push_desc[bank], e.p[bank].shape[-1], e.qat)
        C.comm_flag_add_slots(self.sig.table, self.world, self.push_desc[bank], 1)

    def repush_weights(self):
        """Re-publish the bf16 weights of the owned slots without an update (used when the fake-quant setting changes).
        Every rank must call it at the same step."""
        if not self.sharded:
            self.e.cast_weights()
            return
        for k in gpt.BANKS:
            self._push_bank(k)
        self.e.cast_weights(banks=False)
        self.repushes += 1
        self.e.layer_flag_value = 6 * (self.steps_done + self.repushes)
        self.e.layer_wait_needed = True

    def step(self):
        if self.sharded:
            self._step_sharded()
        else:
            self._step_replicated()
        self.steps_done += 1

    def enable_timing(self, on: bool = True):
        """Record a CUDA event at every phase boundary of the sharded step (`phase_times` reads them)."""
        self.timing = [] if on else None

    def _mark(self, name: str, stream=None):
        if self.timing is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(stream if stream is not None else torch.cuda.current_stream())
            self.timing.append((name, ev))

    def phase_times(self):
        """[(phase, milliseconds since the end of the backward pass)] of the last timed step; synchronises."""
        torch.cuda.synchronize()
        t = dict(self.timing or [])
        if "backward_end" not in t:
            return []
        return [(name, t["backward_end"].elapsed_time(ev)) for name, ev in (self.timing or []) if name != "backward_end"]

    def arm(self):
        """Call before the last micro-batch of a step: its backward pass then hands every finished layer to the
        communication stream (`_layer_done`)."""
        if not self.sharded or not self.overlap:
            return
        self.armed = True
        self.e.backward_observer = self._layer_done
        if self.timing is not None:
            self.timing = []

    def _expected(self) -> int:
        return self.world * (self.steps_done + 1)

    def _layer_done(self, l: int, j: int):
        """Backward of activation slot j (layer l) has been queued on the main stream. When that was the layer's last pass, its
        bank gradients are final on this rank: tell every rank and queue the reduction of the slots owned here."""
        if not self.armed or self.first_slot_of_layer[l] != j:
            return
        e, C, w = self.e, self.C, self.world
        ev = self.ev_layer[l]
        ev.record()
        cs = self.comm_stream
        with torch.cuda.stream(cs):
            if self.bank_pending:                  # the previous step's bank chains read `red`: let them finish first
                for k in self.bank_order:
                    cs.wait_event(self.ev_bank[k])
                self.bank_pending = False
            cs.wait_event(ev)
            C.comm_flag_add(self.sig.table, w, SIG_GRAD + l, 1, 1)
            flag = self.sig_local[SIG_GRAD + l:SIG_GRAD + l + 1]
            for k, sl in self.layer_slots[l]:
                per = e.p[k][0].numel()
                s0 = self.own[k][0]
                C.comm_reduce_peers(self.gbuf.table, w, self.g_off[k] + sl * per, per, self.red[k][sl - s0], 1.0 / w, e.stats, 1.0,
                                    flag, self._expected(), N.status_word())

    def _step_sharded(self):
        e, C, t = self.e, self.C, self.spec.train
        w, n = self.world, e.n
        if not self.armed:                          # single call without `arm` (tests, one micro-batch drivers): nothing overlapped
            self.armed = True
            for l in range(n - 1, -1, -1):
                self._layer_done(l, self.first_slot_of_layer[l])
        self.armed = False
        e.backward_observer = None
        main = torch.cuda.current_stream()
        self._mark("backward_end", main)
        ev_tail = self.ev_layer[n]
        ev_tail.record(main)
        cs = self.comm_stream
        decay = t.ema_decay
        self.epoch += 1
        with torch.cuda.stream(cs):
            cs.wait_event(ev_tail)
            C.comm_flag_add(self.sig.table, w, SIG_GRAD + n, 1, 1)
            flag = self.sig_local[SIG_GRAD + n:SIG_GRAD + n + 1]
            for gi, grp in enumerate(e.groups):
                C.comm_reduce_peers(self.gbuf.table, w, self.grp_off[gi], grp["g"].numel(), grp["g_red"], 1.0 / w, e.stats, 1.0 / w,
                                    flag, self._expected(), N.status_word())
            self._mark("reduce", cs)
            C.comm_scalar_allreduce(self.val.table, self.sig.table, self.rank, w, 0, SIG_SCALAR, self.epoch, e.stats, N.status_word())
            C.clip_factor(e.stats, e.hp, 1.0, max(t.grad_clip_norm, 0.0))
            self.ev_clip.record(cs)
            self._mark("norm_allreduce", cs)
            for grp in e.groups:
                if grp["p"].numel():
                    C.adamw(grp["p"], grp["g_red"], grp["m"], grp["v"], grp.get("ema"), e.hp, grp["lr"], t.adam_beta1, t.adam_beta2, t.adam_eps, t.adam_wd, decay)
            e.cast_weights(banks=False)
            self.ev_adam.record(cs)
            self._mark("adamw", cs)
        for k in self.bank_order:
            s0, s1 = self.own[k]
            bs = self.bank_streams[k]
            with torch.cuda.stream(bs):
                bs.wait_event(self.ev_clip)
                if s1 > s0:
                    cnt = s1 - s0
                    st = e.ns[k]
                    st["sq"].zero_()
                    C.muon_momentum(self.red[k], e.mom[k][s0:s1], st["U"][:cnt], st["sq"][:cnt], e.hp, True)
                    X = e.newton_schulz(k, cnt)
                    scale = max(1.0, e.p[k].shape[-2] / e.p[k].shape[-1]) ** 0.5
                    C.muon_apply(e.p[k][s0:s1].view(-1), X.reshape(-1), e.ema[k][s0:s1].view(-1) if e.ema else None, e.hp, t.matrix_lr, t.muon_wd, scale, decay)
                    self._push_bank(k)
                self.ev_bank[k].record(bs)
                self._mark("bank_" + k, bs)
        self.bank_pending = True
        main.wait_event(self.ev_adam)               # peers have consumed this rank's gradients; replicated weights are current
        self._mark("main stream resumes", main)
        e.layer_flag_value = 6 * (self.steps_done + 1 + self.repushes)
        e.layer_wait_needed = True                  # the next forward gates each layer on its ready counter with a one-thread kernel
        # the bank chains keep reading this step's hyper-parameters; the next step uploads into the other buffer
        e.hp = self.hp_pair[(self.steps_done + 1) & 1]

    def synchronize(self):
        """Host wait for everything this step queued on the communication and bank streams."""
        if self.sharded:
            self.comm_stream.synchronize()
            for bs in self.bank_streams.values():
                bs.synchronize()

    def _step_replicated(self):
        """Two-shot all-reduce of every gradient (reduce my slice from all peers, write it back to all peers), then the
        ordinary replicated optimizer on every rank."""
        e, C, t = self.e, self.C, self.spec.train
        w = self.world
        self.epoch += 1
        self._barrier(SIG_BARRIER)
        n4 = self.g_total // 4
        a, b = (n4 * self.rank // w) * 4, (n4 * (self.rank + 1) // w) * 4
        mine = self.gbuf.view(a * 4, (b - a,), torch.float32)
        C.comm_reduce_peers(self.gbuf.table, w, a, b - a, mine, 1.0 / w, None, 0.0, None, 0, None)
        self._barrier(SIG_BARRIER2)                      # every slice is reduced before anyone overwrites a peer's copy
        C.comm_push_copy(mine, self.gbuf.table, w, self.rank, a)
        self.epoch += 1
        self._barrier(SIG_BARRIER)
        e.clip()
        e.optimizer_step()

    # ---- parameter gathering for export / evaluation --------------------------------------------------------------------------------
    def gather_banks(self, source: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """Full fp32 banks on every rank from the owners' authoritative slots (control-plane collective, end of run)."""
        torch.cuda.synchronize()                    # the bank chains of the last step run on streams of their own
        out = {}
        for k in gpt.BANKS:
            full = source[k].clone()
            if self.sharded:
                for r in range(self.world):
                    s0, s1 = shard_range(full.shape[0], r, self.world)
                    if s1 > s0:
                        dist.broadcast(full[s0:s1], src=dist.get_global_rank(self.group, r) if self.group else r, group=self.group)
            out[k] = full
        return out

    def close(self):
        for b in (self.gbuf, self.wbuf, self.sig, self.val):
            b.close()
