"""Differentiable all-to-all(v): the backward pass is the transposed collective.

The reference plans the reverse exchange with ``schedule(workload, backward=1)``
(amd/flash.cpp:400-408) and leaves calling it to the framework; here one autograd function ties
the two plans together, so a model can use the scheduled collective like any other layer.
"""
from __future__ import annotations

import torch

from .comm import Communicator, Schedule


class _AllToAllV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, comm: Communicator, fwd: Schedule, bwd: Schedule) -> torch.Tensor:
        ctx.comm, ctx.bwd, ctx.in_shape, ctx.dtype = comm, bwd, x.shape, x.dtype
        row = tuple(x.shape[1:])
        row_bytes = fwd.unit_bytes
        out = torch.empty((fwd.output_bytes // row_bytes, *row), dtype=x.dtype, device=x.device)
        comm.all_to_all_v(out, x.contiguous(), fwd)
        return out

    @staticmethod
    def backward(ctx, grad_out: torch.Tensor):
        grad_in = torch.empty(ctx.in_shape, dtype=ctx.dtype, device=grad_out.device)
        ctx.comm.all_to_all_v(grad_in, grad_out.contiguous(), ctx.bwd)
        return grad_in, None, None, None


def all_to_all_v(x: torch.Tensor, comm: Communicator, matrix, kind="auto") -> torch.Tensor:
    """``x`` holds this rank's rows for rank 0..n-1 back to back (``matrix[i, j]`` rows from i to j);
    returns the rows received from rank 0..n-1. Gradients flow back through the transposed plan.
    Both plans are cached by the communicator, so repeated calls with the same matrix plan once."""
    row_bytes = x.element_size() * (x.numel() // max(x.shape[0], 1)) if x.dim() > 1 else x.element_size()
    fwd = comm.schedule(matrix, unit_bytes=row_bytes, kind=kind)
    bwd = comm.schedule(matrix, unit_bytes=row_bytes, kind=kind, transpose=True)
    return _AllToAllV.apply(x, comm, fwd, bwd)
