"""Muon (Newton–Schulz orthogonalised momentum) on parameter banks, AdamW, EMA/SWA, LR schedules.

Update rule (``parameter-golf-rs/crates/pg-optim/src/muon.rs:250-298``; Python
``records/track_10min_16mb/2026-03-23_LeakyReLU_LegalTTT_ParallelMuon/train_gpt.py:127-266``):
``buf = mu*buf + g; u = g + mu*buf (Nesterov); u = NS(u); p = (1 - lr*wd)*p - lr*scale*u`` with
``scale = max(1, rows/cols)^0.5``. Newton–Schulz normalises by the Frobenius norm (+1e-7), works on the
transposed matrix when rows > cols, and iterates ``A = X X^T; B = b A + c A^2; X = a X + B X`` with one
of three coefficient profiles (``muon.rs:44-63``).

These are the torch statements used on CPU and as the oracle of the fused CUDA optimizer.
"""
from __future__ import annotations

import math
from typing import Dict, Iterable, List, Optional

import torch

NS_COEFFS = {
    "simple": [(3.4445, -4.7750, 2.0315)],
    "quintic": [
        (4.0848, -6.8946, 2.9270),
        (3.9505, -6.3029, 2.6377),
        (3.7418, -5.5913, 2.3037),
        (2.8769, -3.1427, 1.2046),
        (2.8366, -3.0525, 1.2012),
    ],
    "polar_express": [
        (8.2051, -22.9019, 16.4607),
        (4.0664, -2.8612, 0.5184),
        (3.9096, -2.8234, 0.5250),
        (3.2856, -2.4153, 0.4853),
        (2.2779, -1.6198, 0.3985),
        (1.8726, -1.2307, 0.3585),
        (1.8564, -1.2132, 0.3568),
        (1.8750, -1.2500, 0.3750),
    ],
}


def ns_coeff(profile: str, step: int):
    tab = NS_COEFFS[profile]
    if profile == "simple":
        return tab[0]
    if profile == "quintic":
        return tab[step % len(tab)]
    return tab[min(step, len(tab) - 1)]


def newton_schulz(g: torch.Tensor, steps: int = 5, profile: str = "quintic", eps: float = 1e-7,
                  compute_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Batched NS orthogonalisation of ``g`` [..., M, N]; returns the same shape and dtype as
    ``compute_dtype`` (default: g's dtype)."""
    x = g.to(compute_dtype) if compute_dtype is not None else g.clone()
    was_2d = x.ndim == 2
    if was_2d:
        x = x[None]
    transposed = x.shape[-2] > x.shape[-1]
    if transposed:
        x = x.mT
    x = x / (x.float().norm(dim=(-2, -1), keepdim=True) + eps).to(x.dtype)
    for s in range(steps):
        a, b, c = ns_coeff(profile, s)
        A = x @ x.mT
        Bm = b * A + c * (A @ A)
        x = a * x + Bm @ x
    if transposed:
        x = x.mT
    return x[0] if was_2d else x


def muon_scale(shape) -> float:
    return max(1.0, shape[-2] / shape[-1]) ** 0.5


class Muon:
    """Replicated Muon over a list of bank tensors (each [B, M, N] or [M, N]). Gradients are passed
    explicitly so the same object serves autograd (CPU) and the manual-backward engine."""

    def __init__(self, params: List[torch.Tensor], lr: float, momentum: float, ns_steps: int = 5,
                 ns_profile: str = "quintic", weight_decay: float = 0.0, nesterov: bool = True,
                 ns_dtype: Optional[torch.dtype] = None):
        self.params = params
        self.lr, self.momentum, self.ns_steps, self.ns_profile = lr, momentum, ns_steps, ns_profile
        self.weight_decay, self.nesterov, self.ns_dtype = weight_decay, nesterov, ns_dtype
        self.bufs = [torch.zeros_like(p, dtype=torch.float32) for p in params]

    @torch.no_grad()
    def step(self, grads: List[torch.Tensor], lr: Optional[float] = None, momentum: Optional[float] = None):
        lr = self.lr if lr is None else lr
        mu = self.momentum if momentum is None else momentum
        for p, g, buf in zip(self.params, grads, self.bufs):
            g = g.float()
            buf.mul_(mu).add_(g)
            u = g.add(buf, alpha=mu) if self.nesterov else buf
            u = newton_schulz(u, self.ns_steps, self.ns_profile, compute_dtype=self.ns_dtype).float()
            if self.weight_decay > 0:
                p.mul_(1.0 - lr * self.weight_decay)
            p.add_(u.to(p.dtype), alpha=-lr * muon_scale(p.shape))

    def state_dict(self):
        return {"bufs": [b.clone() for b in self.bufs]}

    def load_state_dict(self, st):
        for b, s in zip(self.bufs, st["bufs"]):
            b.copy_(s)


def shard_range(slots: int, rank: int, world: int):
    """[start, end) of the leading-axis slots of a bank that ``rank`` owns: equal chunks of ceil(slots / world), the last
    ranks may own fewer or none (the reference's ``chunk_batch``, ``pg-train/src/lib.rs:577-591``)."""
    chunk = -(-slots // world)
    s0 = min(rank * chunk, slots)
    return s0, min(s0 + chunk, slots)


class ShardedMuon:
    """Parallel Muon over a process group, on any backend `torch.distributed` offers (gloo for CPU ranks): the reference form of
    the sharded optimizer the CUDA path runs with peer-memory kernels (``records/.../2026-03-23_.../train_gpt.py:127-266``,
    ``pg-train/src/lib.rs:3259-3772``).

    Every bank ``[slots, M, N]`` is split along its first axis. A rank receives the sum of all ranks' gradients for the slots it
    owns (one reduce per owner), keeps momentum for those slots only, orthogonalises and applies the update to them, and the
    updated slots are all-gathered so that every rank ends the step with identical full banks."""

    def __init__(self, params: List[torch.Tensor], lr: float, momentum: float, ns_steps: int = 5, ns_profile: str = "quintic",
                 weight_decay: float = 0.0, nesterov: bool = True, group=None):
        import torch.distributed as dist
        self.params, self.group = params, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.lr, self.momentum, self.ns_steps, self.ns_profile = lr, momentum, ns_steps, ns_profile
        self.weight_decay, self.nesterov = weight_decay, nesterov
        self.own = [shard_range(p.shape[0], self.rank, self.world) for p in params]
        self.bufs = [torch.zeros_like(p[s0:s1], dtype=torch.float32) for p, (s0, s1) in zip(params, self.own)]

    @torch.no_grad()
    def reduce_to_owners(self, grads: List[torch.Tensor]) -> List[torch.Tensor]:
        """Mean over ranks of the gradient slots each rank owns (the other slots of ``grads`` are left as they are)."""
        import torch.distributed as dist
        out = []
        for g, p in zip(grads, self.params):
            mine = None
            for r in range(self.world):
                s0, s1 = shard_range(p.shape[0], r, self.world)
                if s1 <= s0:
                    continue
                part = g[s0:s1].float().contiguous()
                dist.reduce(part, dst=dist.get_global_rank(self.group, r) if self.group is not None else r, group=self.group)
                if r == self.rank:
                    mine = part / self.world
            s0, s1 = self.own[len(out)]
            out.append(mine if mine is not None else g[s0:s1].float())
        return out

    @torch.no_grad()
    def step(self, own_grads: List[torch.Tensor], lr: Optional[float] = None, momentum: Optional[float] = None):
        """``own_grads[i]`` is the reduced gradient of the owned slots of bank i (what `reduce_to_owners` returns, possibly
        rescaled by the clip factor). Updates the owned slots, then exchanges them."""
        import torch.distributed as dist
        lr = self.lr if lr is None else lr
        mu = self.momentum if momentum is None else momentum
        for p, g, buf, (s0, s1) in zip(self.params, own_grads, self.bufs, self.own):
            if s1 > s0:
                buf.mul_(mu).add_(g)
                u = g.add(buf, alpha=mu) if self.nesterov else buf
                u = newton_schulz(u, self.ns_steps, self.ns_profile).float()
                if self.weight_decay > 0:
                    p[s0:s1].mul_(1.0 - lr * self.weight_decay)
                p[s0:s1].add_(u.to(p.dtype), alpha=-lr * muon_scale(p.shape))
            chunk = -(-p.shape[0] // self.world)
            send = torch.zeros((chunk,) + tuple(p.shape[1:]), dtype=p.dtype)
            send[: s1 - s0].copy_(p[s0:s1])
            recv = [torch.empty_like(send) for _ in range(self.world)]
            dist.all_gather(recv, send, group=self.group)
            for r, t in enumerate(recv):
                r0, r1 = shard_range(p.shape[0], r, self.world)
                if r1 > r0 and r != self.rank:
                    p[r0:r1].copy_(t[: r1 - r0])

    def own_sumsq(self, own_grads: List[torch.Tensor]) -> torch.Tensor:
        return sum((g.float().pow(2).sum() for g in own_grads), torch.zeros(()))

    def state_dict(self):
        """Full momentum buffers, gathered from the owners (a collective: every rank calls it)."""
        import torch.distributed as dist
        full = []
        for p, buf, (s0, s1) in zip(self.params, self.bufs, self.own):
            chunk = -(-p.shape[0] // self.world)
            send = torch.zeros((chunk,) + tuple(p.shape[1:]), dtype=torch.float32)
            send[: s1 - s0].copy_(buf)
            recv = [torch.empty_like(send) for _ in range(self.world)]
            dist.all_gather(recv, send, group=self.group)
            f = torch.zeros_like(p, dtype=torch.float32)
            for r, t in enumerate(recv):
                r0, r1 = shard_range(p.shape[0], r, self.world)
                f[r0:r1].copy_(t[: r1 - r0])
            full.append(f)
        return {"bufs": full}

    def load_state_dict(self, st):
        for buf, s, (s0, s1) in zip(self.bufs, st["bufs"], self.own):
            buf.copy_(s[s0:s1])


class AdamW:
    """Decoupled-weight-decay Adam with bias correction (``pg-optim/src/adamw.rs:46-70``); one lr per group."""

    def __init__(self, groups: List[dict], betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.0):
        self.groups = groups  # each: {"params": [tensors], "lr": float, "names": [...]}
        self.b1, self.b2 = betas
        self.eps, self.weight_decay = eps, weight_decay
        self.t = 0
        self.m = [[torch.zeros_like(p, dtype=torch.float32) for p in g["params"]] for g in groups]
        self.v = [[torch.zeros_like(p, dtype=torch.float32) for p in g["params"]] for g in groups]

    @torch.no_grad()
    def step(self, grads: List[List[torch.Tensor]], lr_scale: float = 1.0):
        self.t += 1
        c1 = 1.0 - self.b1 ** self.t
        c2 = 1.0 - self.b2 ** self.t
        for gi, g in enumerate(self.groups):
            lr = g["lr"] * lr_scale
            for pi, p in enumerate(g["params"]):
                gr = grads[gi][pi].float()
                m, v = self.m[gi][pi], self.v[gi][pi]
                m.mul_(self.b1).add_(gr, alpha=1 - self.b1)
                v.mul_(self.b2).addcmul_(gr, gr, value=1 - self.b2)
                if self.weight_decay > 0:
                    p.mul_(1.0 - lr * self.weight_decay)
                p.addcdiv_((m / c1).to(p.dtype), ((v / c2).sqrt() + self.eps).to(p.dtype), value=-lr)

    def state_dict(self):
        return {"t": self.t, "m": [[x.clone() for x in g] for g in self.m], "v": [[x.clone() for x in g] for g in self.v]}

    def load_state_dict(self, st):
        self.t = int(st["t"])
        for dst, src in ((self.m, st["m"]), (self.v, st["v"])):
            for gd, gs in zip(dst, src):
                for a, b in zip(gd, gs):
                    a.copy_(b)


class Ema:
    """Exponential moving average of a parameter dict; the first update copies
    (``pg-optim/src/ema.rs:26-37``)."""

    def __init__(self, decay: float):
        self.decay = decay
        self.shadow: Optional[Dict[str, torch.Tensor]] = None

    @torch.no_grad()
    def update(self, params: Dict[str, torch.Tensor]):
        if self.shadow is None:
            self.shadow = {k: v.detach().float().clone() for k, v in params.items()}
            return
        for k, v in params.items():
            self.shadow[k].mul_(self.decay).add_(v.detach().float(), alpha=1.0 - self.decay)

    def apply_to(self, params: Dict[str, torch.Tensor]):
        if self.shadow is None:
            return
        with torch.no_grad():
            for k, v in params.items():
                v.copy_(self.shadow[k].to(v.dtype))


class Swa:
    """Uniform average of snapshots taken every ``every`` steps while the LR scale is below ``threshold``."""

    def __init__(self, every: int = 50, threshold: float = 0.2):
        self.every, self.threshold = every, threshold
        self.sum: Optional[Dict[str, torch.Tensor]] = None
        self.count = 0

    def should_collect(self, step: int, lr_scale: float) -> bool:
        return self.every > 0 and lr_scale < self.threshold and step % self.every == 0

    @torch.no_grad()
    def collect(self, params: Dict[str, torch.Tensor]):
        if self.sum is None:
            self.sum = {k: v.detach().float().clone() for k, v in params.items()}
        else:
            for k, v in params.items():
                self.sum[k].add_(v.detach().float())
        self.count += 1

    def average(self) -> Optional[Dict[str, torch.Tensor]]:
        if not self.count:
            return None
        return {k: v / self.count for k, v in self.sum.items()}


class Lawa:
    """Latest-weight averaging: a window of the last ``k`` snapshots, one every ``freq`` steps, averaged uniformly at the end of
    training (``records/track_10min_16mb/2026-03-23_LeakyReLU_LegalTTT_ParallelMuon/train_gpt.py:1635,1727-1758``). When it is
    on and holds at least two snapshots its average replaces the EMA weights."""

    def __init__(self, k: int = 10, freq: int = 100):
        from collections import deque
        self.k, self.freq = k, freq
        self.queue = deque(maxlen=max(k, 1))

    def should_collect(self, step: int) -> bool:
        return self.freq > 0 and step % self.freq == 0

    @torch.no_grad()
    def collect(self, params: Dict[str, torch.Tensor]):
        self.queue.append({k: v.detach().float().cpu().clone() for k, v in params.items()})

    @property
    def count(self) -> int:
        return len(self.queue)

    def average(self) -> Optional[Dict[str, torch.Tensor]]:
        if not self.queue:
            return None
        out = {k: torch.zeros_like(v) for k, v in self.queue[0].items()}
        for snap in self.queue:
            for k, v in snap.items():
                out[k].add_(v)
        return {k: v / len(self.queue) for k, v in out.items()}


# ---- schedules --------------------------------------------------------------------------------------

def lr_scale(step: int, warmup: int, total: int, warmdown: int) -> float:
    """Warmup–stable–decay scale in [0, 1] (``pg-optim/src/scheduler.rs:39-52``)."""
    start = max(total - warmdown, 0)
    if step < warmup:
        return step / warmup
    if step < start:
        return 1.0
    if step < total:
        return max((total - step) / warmdown, 0.0)
    return 0.0


def lr_scale_with_floor(step: int, warmup: int, total: int, warmdown: int, min_scale: float) -> float:
    s = lr_scale(step, warmup, total, warmdown)
    return s if step < warmup else max(s, min_scale)


def wsd_lr(step: int, base_lr: float, warmup: int, total: int, warmdown: int) -> float:
    return base_lr * lr_scale(step, warmup, total, warmdown) if step < total else 0.0


def wallclock_lr_scale(step: int, elapsed_ms: float, iterations: int, warmdown_iters: int, max_wallclock_ms: Optional[float]) -> float:
    """Wallclock-aware warmdown of the Python trainer (``train_gpt.py:924-933``): the warmdown window is
    ``warmdown_iters`` average steps long and ends at the wallclock cap."""
    if warmdown_iters <= 0:
        return 1.0
    if not max_wallclock_ms:
        start = max(iterations - warmdown_iters, 0)
        return max((iterations - step) / max(warmdown_iters, 1), 0.0) if start <= step < iterations else 1.0
    step_ms = elapsed_ms / max(step, 1)
    warmdown_ms = warmdown_iters * step_ms
    remaining = max(max_wallclock_ms - elapsed_ms, 0.0)
    return remaining / max(warmdown_ms, 1e-9) if remaining <= warmdown_ms else 1.0


def fraction_lr_scale(step: int, elapsed_ms: float, iterations: int, fraction: float, max_wallclock_ms: Optional[float]) -> float:
    """Warm-down over the last ``fraction`` of the run: of the wall-clock budget when there is one (the scale is the time left
    over the length of that window), else of the step count. It fixes the schedule whose step-counted window was longer than the
    whole capped run, so that the rate decayed from the first step
    (records/track_non_record_16mb/2026-03-19_SwiGLU_WarmdownFix_QuarterBatch_1x5090/README.md "Warmdown Schedule Bug";
    records/track_10min_16mb/2026-03-24_74M_Ternary_.../train_gpt_cuda_ternary.py ``lr_mul``)."""
    if fraction <= 0:
        return 1.0
    if not max_wallclock_ms:
        window = iterations * fraction
        return max((iterations - step) / max(window, 1.0), 0.0) if step >= int(iterations * (1.0 - fraction)) else 1.0
    window_ms = max_wallclock_ms * fraction
    remaining = max(max_wallclock_ms - elapsed_ms, 0.0)
    return remaining / max(window_ms, 1e-9) if remaining <= window_ms else 1.0


def muon_momentum_at(step: int, start: float, end: float, warmup_steps: int) -> float:
    frac = min(step / warmup_steps, 1.0) if warmup_steps > 0 else 1.0
    return (1 - frac) * start + frac * end


def global_grad_norm(grads: Iterable[torch.Tensor]) -> torch.Tensor:
    return torch.sqrt(sum((g.float().pow(2).sum() for g in grads), torch.zeros(())))


def clip_grads_(grads: List[torch.Tensor], max_norm: float) -> float:
    """Scale all gradients by ``min(1, max_norm/(norm+1e-6))``; returns the pre-clip norm."""
    total = math.sqrt(sum(float(g.float().pow(2).sum()) for g in grads))
    if max_norm > 0 and total > max_norm:
        f = max_norm / (total + 1e-6)
        for g in grads:
            g.mul_(f)
    return total
