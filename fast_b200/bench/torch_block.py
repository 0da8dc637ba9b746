"""The Mixtral-shaped MoE block of ``bench.py`` built from library pieces only: torch ops (cuBLAS
GEMMs, eager element-wise kernels), ``torch.distributed`` all-to-all over NCCL for dispatch and
combine, and ``torch.optim.AdamW(fused=True)``. It is the box's NCCL + cuBLAS arm that the
training number is set against: same shapes, same data, same work per step (forward, backward
through the reversed all-to-all, optimizer step), none of this package's kernels.

The reference itself has no MoE block (its repository is the all-to-all transport only); the way
it is meant to be used - a framework's expert-parallel layer calling an all-to-all(v) around
per-expert GEMMs (amd/README.md:58, amd/flash.cpp:552-568 ``all_to_all_v``) - is what this file
does with the stock collective.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


class _AllToAll(torch.autograd.Function):
    """``all_to_all_single`` with row splits; backward is the same collective with the splits swapped."""

    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.out_splits, ctx.in_splits, ctx.group = out_splits, in_splits, group
        out = torch.empty(sum(out_splits), *x.shape[1:], dtype=x.dtype, device=x.device)
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        else:
            out.copy_(x)
        return out

    @staticmethod
    def backward(ctx, g):
        back = torch.empty(sum(ctx.in_splits), *g.shape[1:], dtype=g.dtype, device=g.device)
        if dist.is_initialized() and dist.get_world_size(ctx.group) > 1:
            dist.all_to_all_single(back, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        else:
            back.copy_(g)
        return back, None, None, None


class TorchMixtralBlock(nn.Module):
    """Embedding -> RMSNorm -> top-k routed SwiGLU experts (expert-parallel over ``group``) + residual
    -> mean-square loss, all in stock PyTorch."""

    def __init__(self, vocab=32000, hidden=4096, inter=14336, num_experts=8, top_k=2, group=None, device="cuda", seed=0):
        super().__init__()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.E, self.K, self.El = num_experts, top_k, num_experts // self.world
        g = torch.Generator(device=device).manual_seed(seed + 100)
        bf = torch.bfloat16
        self.embed = nn.Parameter((torch.randn(vocab, hidden, generator=g, device=device) * 0.02).to(bf))
        self.norm_w = nn.Parameter(torch.ones(hidden, device=device, dtype=bf))
        self.gate = nn.Parameter((torch.randn(num_experts, hidden, generator=g, device=device) * 0.02).to(bf))
        ge = torch.Generator(device=device).manual_seed(seed + 1 + self.rank)
        self.w1 = nn.Parameter((torch.randn(self.El, inter, hidden, generator=ge, device=device) * 0.02).to(bf))
        self.w3 = nn.Parameter((torch.randn(self.El, inter, hidden, generator=ge, device=device) * 0.02).to(bf))
        self.w2 = nn.Parameter((torch.randn(self.El, hidden, inter, generator=ge, device=device) * 0.02).to(bf))

    def replicated_parameters(self):
        return [self.embed, self.norm_w, self.gate]

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        h = F.embedding(token_ids.reshape(-1), self.embed)
        x = F.rms_norm(h, (h.shape[-1],), self.norm_w, 1e-5)
        T, K, W, El = x.shape[0], self.K, self.world, self.El
        logits = (x @ self.gate.t()).float()
        idx = logits.topk(K, dim=-1).indices
        w = torch.softmax(logits.gather(1, idx), dim=-1)
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)           # entries grouped by expert, hence by owner rank
        tok = order // K
        counts = torch.bincount(flat, minlength=self.E)
        recv_counts = torch.empty_like(counts)
        if W > 1:
            dist.all_to_all_single(recv_counts, counts, group=self.group)
        else:
            recv_counts.copy_(counts)
        in_splits = counts.view(W, El).sum(1).tolist()      # host round trip, as every stock expert-parallel layer has
        rc = recv_counts.view(W, El)
        out_splits = rc.sum(1).tolist()
        per_e = rc.sum(0).tolist()
        recv = _AllToAll.apply(x[tok], out_splits, in_splits, self.group)
        eid = torch.repeat_interleave(torch.arange(El, device=x.device).repeat(W), rc.reshape(-1))
        perm = torch.argsort(eid, stable=True)              # rows arrive by (source, expert); regroup by expert
        hx = recv[perm]
        outs, start = [], 0
        for e in range(El):
            seg = hx[start:start + per_e[e]]
            outs.append((F.silu(seg @ self.w1[e].t()) * (seg @ self.w3[e].t())) @ self.w2[e].t())
            start += per_e[e]
        y = torch.cat(outs) if outs else hx
        back = torch.empty_like(y).index_copy(0, perm, y)
        ret = _AllToAll.apply(back, in_splits, out_splits, self.group)
        moe = torch.zeros(T, x.shape[1], dtype=torch.float32, device=x.device).index_add(0, tok, ret.float() * w.reshape(-1)[order].unsqueeze(1))
        return (h + moe.to(h.dtype)).float().pow(2).mean()


def measure(ids_list, steps: int, warmup: int, hidden=4096, inter=14336, num_experts=8, top_k=2, vocab=32000, group=None) -> dict:
    """Times ``steps`` training steps (forward, backward, gradient averaging of the replicated
    parameters, fused AdamW) with CUDA events, max over ranks. Returns ms per step and tokens/s."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    model = TorchMixtralBlock(vocab, hidden, inter, num_experts, top_k, group=group)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.01, fused=True)

    def step(ids):
        opt.zero_grad(set_to_none=True)
        loss = model(ids)
        loss.backward()
        if world > 1:
            for p in model.replicated_parameters():
                dist.all_reduce(p.grad, op=dist.ReduceOp.AVG, group=group)
        opt.step()
        return loss

    for i in range(warmup):
        step(ids_list[i % len(ids_list)])
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier(group=group)
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        loss = step(ids_list[i % len(ids_list)])
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    ms = float(t[0])
    tokens = ids_list[0].numel() * world
    last = float(loss.item())
    del model, opt
    torch.cuda.empty_cache()
    return {"impl": "torch ops (cuBLAS) + NCCL all_to_all_single + torch.optim.AdamW(fused)", "ms_per_step": round(ms, 3),
            "tokens_per_s": round(tokens / (ms * 1e-3), 1), "steps": steps, "warmup": warmup, "last_loss": last}
