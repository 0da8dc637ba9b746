"""AdamW for bf16 parameters with fp32 master weights and moments, one fused kernel per tensor."""
from __future__ import annotations

import torch

from .. import runtime


class FusedAdamW:
    def __init__(self, params, lr=1e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0):
        self.params = [p for p in params if p.requires_grad]
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.step_count = 0
        self.state = {}
        for p in self.params:
            assert p.dtype == torch.bfloat16 and p.numel() % 8 == 0 and p.is_contiguous(), "FusedAdamW wants contiguous bf16 tensors (numel % 8 == 0)"
            self.state[p] = (p.detach().float().clone(), torch.zeros_like(p, dtype=torch.float32), torch.zeros_like(p, dtype=torch.float32))

    def zero_grad(self, set_to_none: bool = True):
        for p in self.params:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0):
        C = runtime.ext()
        self.step_count += 1
        for p in self.params:
            if p.grad is None:
                continue
            master, m, v = self.state[p]
            g = p.grad if p.grad.dtype == torch.bfloat16 else p.grad.to(torch.bfloat16)
            C.adamw(p.data, master, m, v, g.contiguous(), self.lr, self.betas[0], self.betas[1], self.eps, self.wd, self.step_count, grad_scale)
