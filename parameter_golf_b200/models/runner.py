"""Model runners: one interface over the autograd oracle (any device) and the CUDA engine.

Evaluation, test-time training, calibration and the trainer talk to a runner, never to a model
implementation directly:

* ``params``: name -> tensor (fp32 master weights),
* ``nll(ids, targets)`` -> per-token negative log-likelihood [B, T] (no grad),
* ``loss_and_grads(ids, targets, qat=False)`` -> (mean loss tensor, name -> gradient),
* ``logits(ids)`` -> soft-capped logits [B, T, V] (no grad).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..spec import ModelSpec
from . import gpt


class OracleRunner:
    """Autograd implementation on plain torch ops; the CPU backend and the numerical oracle."""

    def __init__(self, model: ModelSpec, params: Dict[str, torch.Tensor], compute_dtype: Optional[torch.dtype] = None):
        self.model = model
        self.params = params
        self.compute_dtype = compute_dtype
        self.lora = None
        self.temperature = 1.0           # evaluation-time scaling of the capped logits (`eval.temperature`); training never uses it

    @property
    def device(self):
        return self.params["tok_emb"].device

    def _p(self):
        if self.compute_dtype is None:
            return self.params
        return {k: v.to(self.compute_dtype) if v.ndim >= 2 else v for k, v in self.params.items()}

    @torch.no_grad()
    def nll(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        return gpt.gpt_forward(self.model, self._p(), ids, targets, lora=self.lora, dtype=self.compute_dtype, reduction="none",
                               temperature=self.temperature).float()

    @torch.no_grad()
    def logits(self, ids: torch.Tensor) -> torch.Tensor:
        return gpt.gpt_logits(self.model, self._p(), ids, lora=self.lora, dtype=self.compute_dtype)

    def loss_and_grads(self, ids, targets, qat: bool = False, names=None, token_weights=None, mtp: bool = False,
                       train: bool = False) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
        names = list(self.params) if names is None else list(names)
        leaves = {k: self.params[k].detach().requires_grad_(True) for k in names}
        p = dict(self.params)
        p.update(leaves)
        if self.compute_dtype is not None:
            p = {k: v.to(self.compute_dtype) if v.ndim >= 2 else v for k, v in p.items()}
        lora = self.lora
        lora_leaves = None
        if lora is not None and lora.get("trainable", False):
            lora_leaves = {"a": lora["a"].detach().requires_grad_(True), "b": lora["b"].detach().requires_grad_(True)}
            lora = dict(lora, **lora_leaves)
        loss = gpt.gpt_forward(self.model, p, ids, targets, qat=qat, lora=lora, dtype=self.compute_dtype, token_weights=token_weights, mtp=mtp,
                               train=train)
        wanted = list(leaves.values()) + (list(lora_leaves.values()) if lora_leaves else [])
        gs = torch.autograd.grad(loss, wanted, allow_unused=True)
        grads = {k: (g if g is not None else torch.zeros_like(leaves[k])) for k, g in zip(names, gs[: len(names)])}
        if lora_leaves:
            grads["lora.a"], grads["lora.b"] = gs[len(names)], gs[len(names) + 1]
        return loss.detach(), grads

    def hidden_taps(self, ids, taps):
        with torch.no_grad():
            gpt.gpt_hidden(self.model, self._p(), ids, dtype=self.compute_dtype, taps=taps)
