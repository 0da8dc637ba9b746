"""``torch.ops.fast_b200.*``: the stateless kernels registered as PyTorch custom operators, so that
they carry schemas, show up in traces and profiles under their own names, and can sit inside code
that is traced with fake tensors (shape propagation without running a kernel).

The reference registers its entry points the same way (a ``TORCH_LIBRARY`` class and op,
nvidia/alltoall_nvshmem.cpp:646-660). The stateful collectives (``Communicator``,
``ExpertParallel``) stay Python objects: they own symmetric memory and epochs. Operator arguments
carry no defaults (mutated optional arguments must be passed explicitly).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch.library import custom_op

from .. import runtime
from . import gemm


@custom_op("fast_b200::grouped_gemm_fwd", mutates_args=("out", "gate_up_out"))
def grouped_gemm_fwd(a: torch.Tensor, w: torch.Tensor, group_off: torch.Tensor, out: torch.Tensor, swiglu: bool,
                     gate_up_out: Optional[torch.Tensor]) -> None:
    """out[rows of g] = a[rows of g] @ w[g].T, optionally with the SwiGLU epilogue (see ops.gemm)."""
    gemm.grouped_gemm_fwd(a, w, group_off, out, swiglu=swiglu, gate_up_out=gate_up_out)


@custom_op("fast_b200::grouped_gemm_dgrad", mutates_args=("out",))
def grouped_gemm_dgrad(dy: torch.Tensor, w: torch.Tensor, group_off: torch.Tensor, out: torch.Tensor,
                       swiglu_bwd_of: Optional[torch.Tensor]) -> None:
    """out[rows of g] = dy[rows of g] @ w[g]; with ``swiglu_bwd_of`` the epilogue writes d(gate|up)."""
    gemm.grouped_gemm_dgrad(dy, w, group_off, out, swiglu_bwd_of=swiglu_bwd_of)


@custom_op("fast_b200::grouped_gemm_wgrad", mutates_args=("out",))
def grouped_gemm_wgrad(dy: torch.Tensor, x: torch.Tensor, group_off: torch.Tensor, out: torch.Tensor) -> None:
    """out[g] = dy[rows of g].T @ x[rows of g]."""
    gemm.grouped_gemm_wgrad(dy, x, group_off, out)


@custom_op("fast_b200::route_topk", mutates_args=())
def route_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Softmax(logits + bias) top-k: (expert indices int32 [T, k], weights float32 [T, k], renormalised over the k)."""
    C = runtime.ext()
    T, E = logits.shape
    idx = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    wts = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    nb = (T + C.ROUTE_TOKENS_PER_BLOCK - 1) // C.ROUTE_TOKENS_PER_BLOCK
    slot = torch.empty(nb * C.ROUTE_TOKENS_PER_BLOCK, k, dtype=torch.int32, device=logits.device)
    cnt = torch.empty(nb, E, dtype=torch.int32, device=logits.device)
    C.route_topk(logits.contiguous(), bias, k, idx, wts, slot, cnt)
    return idx, wts


@route_topk.register_fake
def _route_topk_fake(logits, bias, k):
    T = logits.shape[0]
    return logits.new_empty((T, k), dtype=torch.int32), logits.new_empty((T, k), dtype=torch.float32)
