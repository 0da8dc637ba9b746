"""MoE layer and the Mixtral-shaped block model built on the expert-parallel engine.

Weight layout (framework-owned): ``w13`` is [experts_local, 2*inter, hidden] where every group of
256 rows holds 128 gate rows followed by the 128 up rows of the same features (so that one GEMM
tile carries both halves of SwiGLU); ``w2`` is [experts_local, hidden, inter].
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..ops import fused
from ..parallel.comm import Communicator
from ..parallel.ep import ExpertParallel


def interleave_gate_up(w1: torch.Tensor, w3: torch.Tensor) -> torch.Tensor:
    """[E, I, H] gate and up projections -> [E, 2I, H] in tiles of [128 gate | 128 up]."""
    E, I, H = w1.shape
    return torch.stack([w1.view(E, I // 128, 128, H), w3.view(E, I // 128, 128, H)], dim=2).reshape(E, 2 * I, H).contiguous()


def split_gate_up(w13: torch.Tensor):
    E, I2, H = w13.shape
    t = w13.view(E, I2 // 256, 2, 128, H)
    return t[:, :, 0].reshape(E, I2 // 2, H), t[:, :, 1].reshape(E, I2 // 2, H)


class _MoEFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weights, w13, w2, engine, rs):
        engine.dispatch(x, rs)
        engine.experts_forward(w13, w2, rs)
        out = engine.combine(rs, weights.detach().float().contiguous())
        ctx.engine, ctx.rs, ctx.w2_param = engine, rs, w2
        ctx.save_for_backward(weights, w13, w2)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        weights, w13, w2 = ctx.saved_tensors
        gx, gw, dw13, dw2 = _experts_backward(ctx.engine, grad_out, ctx.rs, weights.detach().float().contiguous(), w13, w2, ctx.w2_param)
        return gx, gw.to(weights.dtype), dw13, dw2, None, None


def _experts_backward(eng, grad_out, rs, weights, w13, w2, w2_param):
    """Backward of dispatch -> experts -> combine through the engine. Returns (grad_x, grad_weights, dW13,
    dW2 or None); dW2 is None when an attached optimizer applied W2's update inside the pass."""
    if not hasattr(eng, "_dw13") or eng._dw13.shape != w13.shape:
        eng._dw13, eng._dw2 = torch.empty_like(w13), torch.empty_like(w2)
    opt = getattr(eng, "optimizer_in_backward", None)
    early = opt is not None and opt.owns(w2_param)
    after = None
    if early:
        # W2's update runs on a side stream under the remaining GEMMs (W13 dgrad / wgrad): after the
        # W2 wgrad nothing in this pass reads W2 any more.
        main = torch.cuda.current_stream()
        if not hasattr(eng, "_opt_stream"):
            eng._opt_stream = torch.cuda.Stream(device=grad_out.device)

        def after():
            ev = torch.cuda.Event()
            ev.record(main)
            eng._opt_stream.wait_event(ev)
            opt.step_param(w2_param, eng._dw2, stream=eng._opt_stream, early=True)

    gx, gw = eng.backward(grad_out.contiguous(), rs, weights, w13, w2, eng._dw13, eng._dw2, after_dw2=after)
    if early:
        done = torch.cuda.Event()
        done.record(eng._opt_stream)
        torch.cuda.current_stream().wait_event(done)  # the next kernels on this stream may read W2 / reuse dW2
    return gx, gw, eng._dw13, (None if early else eng._dw2)


class _NormRouteMoEFunction(torch.autograd.Function):
    """h -> RMSNorm -> router -> dispatch -> experts -> combine, with the router front end fused into one
    kernel each way (no library GEMM, layer-norm, gather or softmax kernel on the path)."""

    @staticmethod
    def forward(ctx, h, norm_w, gate, w13, w2, engine, eps, layer):
        rs, hn, rstd, _ = engine.route_fused(h, norm_w, gate, eps, layer.router_bias)
        layer.last_route = rs
        engine.dispatch(hn, rs)
        engine.experts_forward(w13, w2, rs)
        out = engine.combine(rs, rs.topk_w)
        ctx.engine, ctx.rs, ctx.w2_param = engine, rs, w2
        ctx.save_for_backward(h, norm_w, gate, rstd, w13, w2)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        h, norm_w, gate, rstd, w13, w2 = ctx.saved_tensors
        eng, rs = ctx.engine, ctx.rs
        gx, gw, dw13, dw2 = _experts_backward(eng, grad_out, rs, rs.topk_w, w13, w2, ctx.w2_param)
        grad_h = torch.empty_like(h)
        d_gate = torch.zeros(gate.shape, dtype=torch.float32, device=h.device)
        d_nw = torch.zeros(norm_w.shape, dtype=torch.float32, device=h.device)
        eng._C.norm_gate_bwd(h, norm_w, gate, rstd, rs.topk_idx, rs.topk_w, gw, gx, grad_h, d_gate, d_nw)
        return grad_h, d_nw.to(norm_w.dtype), d_gate.to(gate.dtype), dw13, dw2, None, None, None


class MoELayer(nn.Module):
    """Top-k softmax-routed SwiGLU experts, expert-parallel over the communicator's ranks."""

    def __init__(self, comm: Communicator, hidden: int, inter: int, num_experts: int, top_k: int, max_tokens: int, fp8_dispatch: bool = False,
                 router_bias: bool = False, training: bool = True, capacity_rows: Optional[int] = None, init_std: float = 0.02, seed: int = 0,
                 overlap_dispatch: bool = False, graph_mode: bool = False, fp8_direct: bool = False):
        super().__init__()
        self.comm, self.hidden, self.inter, self.num_experts, self.top_k = comm, hidden, inter, num_experts, top_k
        El = num_experts // comm.world
        dev = comm.device
        g = torch.Generator(device=dev).manual_seed(seed)
        self.gate = nn.Parameter((torch.randn(num_experts, hidden, generator=g, device=dev) * init_std).to(torch.bfloat16))
        ge = torch.Generator(device=dev).manual_seed(seed + 1 + comm.rank)
        self.w13 = nn.Parameter((torch.randn(El, 2 * inter, hidden, generator=ge, device=dev) * init_std).to(torch.bfloat16))
        self.w2 = nn.Parameter((torch.randn(El, hidden, inter, generator=ge, device=dev) * init_std).to(torch.bfloat16))
        self.router_bias = nn.Parameter(torch.zeros(num_experts, device=dev), requires_grad=False) if router_bias else None
        self.engine = ExpertParallel(comm, num_experts, hidden, inter, top_k, max_tokens, fp8_dispatch=fp8_dispatch, training=training,
                                     capacity_rows=capacity_rows, overlap_dispatch=overlap_dispatch, graph_mode=graph_mode, fp8_direct=fp8_direct)

    @torch.no_grad()
    def capture(self, tokens: int) -> None:
        """Capture the forward-only layer for ``tokens`` rows in a CUDA graph (needs ``graph_mode=True``).
        Collective: every rank captures, and later replays, the same number of times."""
        assert self.engine.graph_mode, "construct the layer with graph_mode=True"
        dev = self.gate.device
        self._gx = torch.zeros(tokens, self.hidden, dtype=torch.bfloat16, device=dev)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):  # warm-up outside the capture: lazy allocations, tensor maps, status blocks
                self._gout = self._infer(self._gx)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(dev)
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._gout = self._infer(self._gx)

    @torch.no_grad()
    def forward_graphed(self, x: torch.Tensor) -> torch.Tensor:
        """Replay the captured layer on ``x`` (same shape as at capture). The result lives in a buffer
        owned by the graph and is overwritten by the next replay."""
        self._gx.copy_(x)
        self._graph.replay()
        return self._gout

    def _infer(self, x: torch.Tensor) -> torch.Tensor:
        logits = (x @ self.gate.t()).float()
        rs = self.engine.route(logits, self.router_bias)
        self.last_route = rs
        self.engine.dispatch(x, rs)
        self.engine.experts_forward(self.w13, self.w2, rs)
        return self.engine.combine(rs, rs.topk_w)

    def forward_from_residual(self, h: torch.Tensor, norm_w: torch.Tensor, eps: float) -> torch.Tensor:
        """MoE(RMSNorm(h; norm_w)) for h [tokens, hidden] bf16. When the layer's shapes allow it the norm,
        the router logits, the top-k and their backward run as one fused kernel each way; otherwise this is
        ``self(rms_norm(h))`` with stock ops in front."""
        fused = self.engine.can_fuse_gate() and torch.is_grad_enabled() and self.training and h.dtype == torch.bfloat16
        if not fused:
            return self(torch.nn.functional.rms_norm(h, (h.shape[-1],), norm_w, eps))
        return _NormRouteMoEFunction.apply(h.contiguous(), norm_w, self.gate, self.w13, self.w2, self.engine, eps, self)

    def attach_optimizer(self, opt) -> None:
        """Optimizer-in-backward: ``opt`` (a FusedAdamW owning ``w2``) applies W2's update as soon as
        its gradient exists, overlapped with the rest of the backward pass; ``opt.step()`` then
        skips it. ``w2.grad`` stays None in that mode."""
        self.engine.optimizer_in_backward = opt

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x: [tokens, hidden] bf16 -> [tokens, hidden] bf16."""
        logits = (x @ self.gate.t()).float()
        rs = self.engine.route(logits.detach(), self.router_bias)
        self.last_route = rs
        if torch.is_grad_enabled() and self.training:
            w = torch.softmax(logits.gather(1, rs.topk_idx.long()), dim=-1)
            return _MoEFunction.apply(x, w, self.w13, self.w2, self.engine, rs)
        self.engine.dispatch(x, rs)
        self.engine.experts_forward(self.w13, self.w2, rs)
        return self.engine.combine(rs, rs.topk_w)


class MixtralBlockModel(nn.Module):
    """Embedding -> RMSNorm -> MoE block (+ residual) -> mean-square loss; Mixtral-8x7B shapes by default."""

    def __init__(self, comm: Communicator, vocab: int = 32000, hidden: int = 4096, inter: int = 14336, num_experts: int = 8, top_k: int = 2,
                 max_tokens: int = 8 * 4096, capacity_rows: Optional[int] = None, seed: int = 0):
        super().__init__()
        dev = comm.device
        g = torch.Generator(device=dev).manual_seed(seed + 100)
        self.embed = nn.Parameter((torch.randn(vocab, hidden, generator=g, device=dev) * 0.02).to(torch.bfloat16))
        self.norm_w = nn.Parameter(torch.ones(hidden, device=dev, dtype=torch.bfloat16))
        self.moe = MoELayer(comm, hidden, inter, num_experts, top_k, max_tokens, capacity_rows=capacity_rows, seed=seed)
        self.eps = 1e-5

    def replicated_parameters(self):
        return [self.embed, self.norm_w, self.moe.gate]

    def expert_parameters(self):
        return [self.moe.w13, self.moe.w2]

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        h = fused.embedding(token_ids.reshape(-1), self.embed)
        return fused.residual_mean_square(h, self.moe.forward_from_residual(h, self.norm_w, self.eps))


@torch.no_grad()
def reference_moe(x, gate, w13_all, w2_all, top_k, bias=None):
    """Plain fp32 PyTorch MoE on one device with ALL experts ([E, 2I, H] interleaved, [E, H, I])."""
    xf = x.float()
    logits = xf @ gate.float().t()
    sel = logits + (bias.float() if bias is not None else 0.0)
    idx = sel.topk(top_k, dim=-1).indices
    w = torch.softmax(logits.gather(1, idx), dim=-1)
    w1, w3 = split_gate_up(w13_all.float())
    out = torch.zeros_like(xf)
    for e in range(w13_all.shape[0]):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        h = xf[tok]
        a = torch.nn.functional.silu(h @ w1[e].t()) * (h @ w3[e].t())
        out.index_add_(0, tok, (a @ w2_all[e].float().t()) * w[tok, slot].unsqueeze(1))
    return out, idx, w
