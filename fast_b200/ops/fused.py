"""Small fused autograd ops around the MoE block: embedding with a segmented-sum backward, and the
mean-square loss of a residual sum computed without materialising fp32 copies."""
from __future__ import annotations

import torch

from .. import runtime


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        ctx.save_for_backward(ids)
        ctx.shape = table.shape
        return torch.nn.functional.embedding(ids, table)

    @staticmethod
    def backward(ctx, grad_out):
        (ids,) = ctx.saved_tensors
        grad_table = torch.zeros(ctx.shape, dtype=grad_out.dtype, device=grad_out.device)
        # positions grouped by id by this library's counting sort (stable, cost independent of duplicates)
        sorted_ids, perm = runtime.ext().embedding_index(ids.reshape(-1).contiguous(), ctx.shape[0])
        runtime.ext().embedding_bwd(sorted_ids, perm, grad_out.reshape(-1, ctx.shape[1]).contiguous(), grad_table)
        return None, grad_table


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """``table[ids]`` (bf16 table); backward sums duplicate ids in position order (deterministic)."""
    return _Embedding.apply(ids, table)


class _ResidualMeanSquare(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        C = runtime.ext()
        a, b = a.contiguous(), b.contiguous()
        partial = torch.empty(148 * 8, dtype=torch.float32, device=a.device)
        out = torch.empty(1, dtype=torch.float32, device=a.device)
        C.sumsq_add(a, b, 1.0 / a.numel(), partial, out)
        ctx.save_for_backward(a, b)
        return out.reshape(())

    @staticmethod
    def backward(ctx, grad_loss):
        a, b = ctx.saved_tensors
        g = torch.empty_like(a)
        runtime.ext().scaled_sum(a, b, grad_loss.reshape(1).float().contiguous(), 2.0 / a.numel(), g)
        return g, g


def residual_mean_square(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """mean((a + b)^2) with the sum rounded to bf16, as a scalar fp32 tensor (bf16 inputs)."""
    return _ResidualMeanSquare.apply(a, b)
