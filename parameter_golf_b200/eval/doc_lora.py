"""Document-isolated evaluation with per-document LoRA test-time training.

The evaluation of ``records/track_10min_16mb/2026-03-17_LoRA_TTT`` (``train_gpt.py:805-958``): the validation stream is cut into
documents at the boundary (BOS) token; every document is scored on its own, so no token is conditioned on another document;
within a document the predictions are taken chunk by chunk (``chunk`` tokens, each scored inside a context window of up to
``window`` tokens that ends with the chunk), and after a chunk has been scored one Adam step on that chunk's mean loss updates
low-rank adapters on the query and value projections of every block and on the output head. Adapters and optimizer state are
per document and start from scratch for each one (A uniform in ±1/sqrt(d), B zero), so nothing learned on one document reaches
another and every token is scored before anything trains on it.

Documents are processed in batches with an adapter set per batch element (`torch.bmm`), sorted by their number of chunks so
that a batch wastes little padding; each rank takes a contiguous slice of the documents and the three sums are reduced at the
end. With ``rank = 0`` the adapters are absent and the result is the plain document-isolated, strided evaluation (the record's
ablation rows "doc-isolated" and "stride").
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np
import torch

from ..data.bpb import BpbLuts
from ..models import gpt
from ..spec import EvalSpec, ModelSpec


def find_documents(tokens: np.ndarray, boundary_id: int, include_next_boundary: bool = True) -> List[Tuple[int, int]]:
    """``(start, length)`` of every document: it starts at a boundary token and, so that the token count equals the flat stream's,
    takes the next document's boundary token as its last target. Tokens before the first boundary belong to no document;
    documents too short to hold one prediction are dropped."""
    pos = np.flatnonzero(np.asarray(tokens) == boundary_id)
    docs = []
    for i, start in enumerate(pos):
        end = int(pos[i + 1]) if i + 1 < len(pos) else int(len(tokens))
        if include_next_boundary and i + 1 < len(pos):
            end += 1
        if end - int(start) >= 2:
            docs.append((int(start), end - int(start)))
    return docs


def chunk_window(ci: int, pred_len: int, num_chunks: int, chunk: int, window: int) -> Tuple[int, int, int, int]:
    """``(window start, window length, offset of the chunk in the window, chunk length)`` for chunk ``ci`` of a document with
    ``pred_len`` predictions: the window ends where the chunk ends and reaches back at most ``window`` positions."""
    c0 = ci * chunk
    c1 = pred_len if ci == num_chunks - 1 else (ci + 1) * chunk
    w0 = max(0, c1 - window)
    return w0, c1 - w0, c0 - w0, c1 - c0


class DocAdapters:
    """Adapter tensors for a batch of ``bsz`` documents, with their Adam state."""

    def __init__(self, m: ModelSpec, bsz: int, rank: int, device, gen: torch.Generator):
        d, kv, V, n = m.model_dim, m.kv_dim, m.vocab_size, m.num_layers
        bound = 1.0 / math.sqrt(d)

        def a():
            return ((torch.rand(bsz, rank, d, generator=gen) * 2 - 1) * bound).to(device).requires_grad_(True)

        def b(out):
            return torch.zeros(bsz, out, rank, device=device, requires_grad=True)
        self.t: Dict[str, object] = {"q_a": [a() for _ in range(n)], "q_b": [b(d) for _ in range(n)], "v_a": [a() for _ in range(n)],
                                     "v_b": [b(kv) for _ in range(n)], "head_a": a(), "head_b": b(V)}
        self.leaves = self.t["q_a"] + self.t["q_b"] + self.t["v_a"] + self.t["v_b"] + [self.t["head_a"], self.t["head_b"]]
        self.m1 = [torch.zeros_like(x) for x in self.leaves]
        self.m2 = [torch.zeros_like(x) for x in self.leaves]
        self.steps = 0

    @torch.no_grad()
    def adam(self, grads, lr: float, b1: float, b2: float, eps: float = 1e-10):
        self.steps += 1
        c1, c2 = 1 - b1 ** self.steps, 1 - b2 ** self.steps
        for x, g, m1, m2 in zip(self.leaves, grads, self.m1, self.m2):
            if g is None:
                continue
            m1.mul_(b1).add_(g, alpha=1 - b1)
            m2.mul_(b2).addcmul_(g, g, value=1 - b2)
            x.addcdiv_(m1 / c1, (m2 / c2).sqrt_().add_(eps), value=-lr)


def eval_doc_lora_ttt(params: Dict[str, torch.Tensor], model: ModelSpec, tokens: np.ndarray, ev: EvalSpec, luts: BpbLuts, rank: int = 0,
                      world: int = 1, device="cpu", log: Callable = lambda s: None, all_reduce: Optional[Callable] = None,
                      betas=(0.9, 0.95), seed: int = 0) -> Tuple[float, float]:
    """``(val_loss, val_bpb)`` over all documents. ``all_reduce(tensor)`` sums a float64 tensor over ranks in place."""
    docs = find_documents(tokens, ev.doc_boundary_token_id)
    if not docs:
        raise ValueError(f"no document starts with token {ev.doc_boundary_token_id} in the validation stream")
    mine = docs[(len(docs) * rank) // world: (len(docs) * (rank + 1)) // world]
    chunk, window, lora_rank = ev.doc_chunk_size, model.eval_seq_len, ev.doc_lora_rank
    mine.sort(key=lambda d: (d[1] - 2) // chunk)
    p = {k: v.to(device) for k, v in params.items()}
    toks = torch.from_numpy(np.asarray(tokens).astype(np.int64))
    sums = torch.zeros(3, dtype=torch.float64)               # loss, bytes, tokens
    gen = torch.Generator().manual_seed(seed + 7919 * rank)
    for b0 in range(0, len(mine), ev.doc_batch_size):
        batch = mine[b0: b0 + ev.doc_batch_size]
        bsz = len(batch)
        ad = DocAdapters(model, bsz, lora_rank, device, gen) if lora_rank > 0 else None
        pred = [ln - 1 for _, ln in batch]
        nch = [-(-pl // chunk) for pl in pred]
        for ci in range(max(nch)):
            _, ctx, off, _ = chunk_window(ci, (ci + 1) * chunk, ci + 1, chunk, window)      # a full chunk's window: the batch's width
            active = [ci < c for c in nch]
            train = ad is not None and any(ci < c - 1 for c in nch)
            x = torch.zeros(bsz, ctx, dtype=torch.int64)
            y = torch.zeros(bsz, ctx, dtype=torch.int64)
            info = []
            for b in range(bsz):
                if not active[b]:
                    info.append((0, 0, 0))
                    continue
                ds, _ = batch[b]
                w0, wl, co, cl = chunk_window(ci, pred[b], nch[b], chunk, window)
                seg = toks[ds + w0: ds + w0 + wl + 1]
                x[b, :wl], y[b, :wl] = seg[:-1], seg[1:]
                info.append((co, cl, ds + w0))
            with torch.enable_grad() if train else torch.no_grad():
                ptl = gpt.gpt_forward(model, p, x.to(device), y.to(device), lora=ad.t if ad is not None else None, reduction="none").float()
            with torch.no_grad():
                for b in range(bsz):
                    co, cl, g0 = info[b]
                    if cl == 0:
                        continue
                    sums[0] += ptl[b, co: co + cl].double().sum().cpu()
                    positions = g0 + co + 1 + np.arange(cl)             # where the targets sit in the validation stream
                    sums[1] += float(luts.token_bytes(x[b, co: co + cl].numpy(), y[b, co: co + cl].numpy(), positions).sum())
                    sums[2] += cl
            if train:
                # one step on the chunk just scored, for the documents that still have a chunk to come
                mask = torch.tensor([float(ci < c - 1) for c in nch], device=ptl.device)
                loss = (ptl[:, off: off + chunk].mean(dim=-1) * mask).sum()
                grads = torch.autograd.grad(loss, ad.leaves, allow_unused=True)
                ad.adam(grads, ev.doc_lora_lr, betas[0], betas[1])
        log(f"doc_lora_ttt: rank {rank} documents {min(b0 + bsz, len(mine))}/{len(mine)}")
    if all_reduce is not None and world > 1:
        all_reduce(sums)
    return float(sums[0] / sums[2]), float(sums[0] / math.log(2.0) / sums[1])
