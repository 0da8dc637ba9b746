"""AdamW for bf16 parameters with fp32 master weights and moments, one fused kernel per tensor."""
from __future__ import annotations

from typing import Optional

import torch

from .. import runtime


class FusedAdamW:
    """``step()`` updates every parameter that has a gradient. ``step_param`` updates one parameter
    from an explicit gradient tensor, optionally on another stream: the MoE layer uses it to apply a
    weight's update as soon as its gradient exists, under the remaining backward GEMMs
    (optimizer-in-backward); such parameters are then skipped by the next ``step()``."""

    def __init__(self, params, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0):
        self.params = [p for p in params if p.requires_grad]
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.state = {}
        self.steps = {}
        self._stepped_early = set()
        for p in self.params:
            assert p.dtype == torch.bfloat16 and p.numel() % 8 == 0 and p.is_contiguous(), "FusedAdamW wants contiguous bf16 tensors (numel % 8 == 0)"
            self.state[p] = (p.detach().float().clone(), torch.zeros_like(p, dtype=torch.float32), torch.zeros_like(p, dtype=torch.float32))
            self.steps[p] = 0

    def owns(self, p) -> bool:
        return p in self.state

    def zero_grad(self, set_to_none: bool = True):
        for p in self.params:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()

    @torch.no_grad()
    def step_param(self, p, grad: torch.Tensor, grad_scale: float = 1.0, stream: Optional[torch.cuda.Stream] = None, early: bool = False):
        master, m, v = self.state[p]
        self.steps[p] += 1
        g = grad if grad.dtype == torch.bfloat16 else grad.to(torch.bfloat16)
        if stream is None:
            runtime.ext().adamw(p.data, master, m, v, g.contiguous(), self.lr, self.betas[0], self.betas[1], self.eps, self.wd, self.steps[p], grad_scale)
        else:
            with torch.cuda.stream(stream):
                runtime.ext().adamw(p.data, master, m, v, g.contiguous(), self.lr, self.betas[0], self.betas[1], self.eps, self.wd, self.steps[p], grad_scale)
        if early:
            self._stepped_early.add(p)

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0):
        for p in self.params:
            if p in self._stepped_early or p.grad is None:
                continue
            self.step_param(p, p.grad, grad_scale)
        self._stepped_early.clear()
