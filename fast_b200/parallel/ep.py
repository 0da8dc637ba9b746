"""Expert-parallel MoE engine: routing -> count exchange -> fused dispatch -> grouped expert GEMMs
-> fused combine, and the mirrored backward pass, all stream-ordered on the device.

Nothing in the step returns to the host between the gate and the combined output: routing
indices, split counts, receive offsets and GEMM group boundaries are produced and consumed in
device memory, and peers are synchronised by flags and counters in the symmetric heap.

In the reference, the host computes a schedule from a token matrix (amd/flash.cpp:400-420) and
runs the forward all-to-all, and again with ``backward=1`` for the reverse direction; the MoE
layer around it is left to the caller. Here the same two collectives are fused with the permute,
the quantisation, the expert GEMMs and the weighted reduction.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import runtime
from ..ops import gemm
from ..utils.config import nvtx_range
from .comm import Communicator


@dataclass
class RouteState:
    """Per-step routing products kept for combine and for the backward pass."""

    topk_idx: torch.Tensor
    topk_w: torch.Tensor
    dest_row: torch.Tensor
    slot_in_block: torch.Tensor
    block_base: torch.Tensor
    send_base: torch.Tensor
    group_off: torch.Tensor
    group_rows: torch.Tensor
    epoch: int


class ExpertParallel:
    """One MoE layer's expert-parallel state on one rank.

    The receive, activation and gradient buffers belong to the engine and are overwritten by the
    next ``route``: a forward pass must be followed by its backward pass (or be forward-only)
    before the next forward of the same engine; use one engine per layer. Every rank of the
    communicator must call the same sequence of methods (the count exchange inside ``route`` is the
    hand-shake that makes buffer reuse safe across ranks).

    ``overlap_dispatch`` (forward-only layers) sends the rows expert by expert on a side stream while the
    first expert GEMM, gated per 256-row tile, runs on all but ``overlap_reserve_sms`` SMs. It pays with
    bf16 rows (layer -2 % at 2 GPUs, -7 % at 4); with ``fp8_dispatch`` the default receive path
    dequantises the whole buffer before the GEMM, so nothing can start early and the mode only costs.
    """

    def __init__(self, comm: Communicator, num_experts: int, hidden: int, inter: int, top_k: int, max_tokens: int, fp8_dispatch: bool = False,
                 capacity_rows: Optional[int] = None, training: bool = True, comm_ctas: Optional[int] = None, overlap_dispatch: bool = False,
                 graph_mode: bool = False, fp8_direct: bool = False, overlap_reserve_sms: int = 16):
        C = runtime.ext()
        self._C, self.comm = C, comm
        W = comm.world
        assert num_experts % W == 0 and hidden % 256 == 0 and inter % 128 == 0 and top_k <= 8
        assert not training or inter % 256 == 0, "training needs inter % 256 == 0 (dgrad output tiles are 256 wide)"
        self.E, self.El, self.H, self.I, self.K, self.T = num_experts, num_experts // W, hidden, inter, top_k, max_tokens
        self.fp8, self.training = fp8_dispatch, training
        # graph_mode (forward only): the step's epoch lives in device memory and is advanced by the split-scan
        # kernel, and the routing outputs are static buffers, so the whole layer can be captured in a CUDA
        # graph and replayed.
        assert not (graph_mode and training), "graph_mode covers the forward-only layer"
        self.graph_mode = graph_mode
        # overlap_dispatch: rows are sent expert by expert on a side stream while the gated expert GEMM of
        # the main stream already consumes the experts that are complete (forward dispatch only).
        self.overlap = overlap_dispatch
        self.side = torch.cuda.Stream(device=comm.device) if overlap_dispatch else None
        sms = torch.cuda.get_device_properties(comm.device).multi_processor_count
        # dispatch / combine run alone on the stream: fill the machine (4 CTAs of 256 threads per SM)
        self.comm_ctas = comm_ctas or 4 * sms
        # Overlapped dispatch: the gated GEMM is persistent (one CTA per SM, nearly all of its shared memory) and
        # waits for rows that this rank's own dispatch kernel must send, so it may never own every SM: it leaves
        # `reserve` SMs to the dispatch kernel, whose grid is sized for them.
        # SMs the first expert GEMM leaves to the side-stream dispatch in overlap mode (the GEMM is persistent and would
        # otherwise hold every SM): about 16 SMs of copy loops fill 0.87 of an NVLink port, 32 all of it.
        self.overlap_reserve_sms = max(2, int(overlap_reserve_sms)) if overlap_dispatch else 0
        self.gemm1_ctas = (sms - self.overlap_reserve_sms) & ~1
        worst = W * max_tokens * min(top_k, self.El) + 256 * self.El
        self.cap = int(capacity_rows) if capacity_rows else worst
        self.cap = (min(self.cap, worst) + 255) // 256 * 256
        dev = comm.device
        i32 = dict(dtype=torch.int32, device=dev)
        # symmetric: control words
        self.counts = comm.alloc((W, self.E), torch.int32)
        self.flags = comm.alloc((8, 64), torch.int64)  # rows: 0 counts, 1 fwd-ready, 2 bwd-entry, 3 bwd-ready
        # Arrival counters. Training keeps one per local expert and channel (forward / backward dispatch). The
        # forward-only layer counts arrivals per 256-row tile of the receive buffer instead, so that the expert
        # GEMM's producer waits only for the tile it is about to load (CTA-pair kernel: its tiles are 256 rows).
        self.tile_rows = 256 if (not training and gemm.USE_PAIR) else 0
        self.ntiles = self.cap // 256
        # fp8_direct (forward-only layer): e4m3 rows and their scales feed the first expert GEMM as they are (converter
        # warps build the bf16 tiles in shared memory). Measured slower than the separate dequantisation pass followed
        # by the bf16 GEMM (the conversion sits in the GEMM's critical path), so it is an option, not the default.
        self.fp8_direct = bool(fp8_direct and fp8_dispatch and self.tile_rows)
        self.arrive = comm.alloc((2, max(self.El, self.ntiles if self.tile_rows else 0)), torch.int64)
        for t in (self.counts, self.flags, self.arrive):
            t.zero_()
        # symmetric: payload
        if fp8_dispatch:
            self.xq_recv = comm.alloc((self.cap, hidden), torch.uint8)
            self.xs_recv = comm.alloc((self.cap, hidden // 128), torch.float32)
            self.x_recv = None if self.fp8_direct else torch.zeros(self.cap, hidden, dtype=torch.bfloat16, device=dev)
        else:
            self.x_recv = comm.alloc((self.cap, hidden), torch.bfloat16)
        self.y = comm.alloc((self.cap, hidden), torch.bfloat16)
        if self.x_recv is not None:
            self.x_recv.zero_()
        self.y.zero_()
        # local work buffers
        self.act = torch.zeros(self.cap, inter, dtype=torch.bfloat16, device=dev)
        if training:
            self.dy_recv = comm.alloc((self.cap, hidden), torch.bfloat16)
            self.dx_recv = comm.alloc((self.cap, hidden), torch.bfloat16)
            self.dy_recv.zero_()
            self.dx_recv.zero_()
            self.gu = torch.zeros(self.cap, 2 * inter, dtype=torch.bfloat16, device=dev)
            self.dact = torch.zeros(self.cap, inter, dtype=torch.bfloat16, device=dev)
            self.dgu = torch.zeros(self.cap, 2 * inter, dtype=torch.bfloat16, device=dev)
        blocks = (max_tokens + C.ROUTE_TOKENS_PER_BLOCK - 1) // C.ROUTE_TOKENS_PER_BLOCK
        self.blocks = blocks
        self.block_cnt = torch.zeros(blocks, self.E, **i32)
        self.block_base = torch.zeros(blocks, self.E, **i32)
        self.slot_in_block = torch.zeros(blocks * C.ROUTE_TOKENS_PER_BLOCK, top_k, **i32)
        self.send_base = torch.zeros(self.E, **i32)
        self.send_cnt = torch.zeros(self.E, **i32)
        self.send_pos = torch.zeros(self.E, **i32)
        self.send_list = torch.zeros(max_tokens * top_k, **i32) if overlap_dispatch else None
        self._xq_send = self._xs_send = None  # sorted fp8 dispatch: rows quantised once, allocated on first use
        self.group_off = torch.zeros(self.El + 1, **i32)
        self.group_rows = torch.zeros(self.El, **i32)
        self.arrive_target = torch.zeros(2, self.El, dtype=torch.int64, device=dev)
        self.tile_target = torch.zeros(1, self.ntiles, dtype=torch.int64, device=dev) if self.tile_rows else None
        self.traffic = torch.zeros(W, W, **i32)
        self.epoch = 0
        self.epoch_dev = torch.zeros(1, dtype=torch.int64, device=dev)
        if graph_mode:
            self._static_route = (torch.empty(max_tokens, top_k, **i32), torch.empty(max_tokens, top_k, dtype=torch.float32, device=dev),
                                  torch.empty(max_tokens, top_k, **i32))
        self.status = comm.status
        self.timeout_ns = comm.timeout_ns
        torch.cuda.synchronize(dev)
        if W > 1:
            import torch.distributed as dist

            dist.barrier(group=comm.group)

    def close(self) -> None:
        """Return this engine's symmetric allocations to the heap (collective: every rank, same order)."""
        torch.cuda.synchronize(self.comm.device)
        for name in ("dx_recv", "dy_recv", "y", "x_recv", "xs_recv", "xq_recv", "arrive", "flags", "counts"):
            t = getattr(self, name, None)
            if t is not None and hasattr(t, "_symm_off"):
                self.comm.free(t)
                setattr(self, name, None)

    # ---- helpers -----------------------------------------------------------------------------
    def _off(self, t: torch.Tensor) -> int:
        return t._symm_off

    def _flag_off(self, row: int) -> int:
        return self.flags._symm_off + row * 64 * 8

    def _arrive_ptr(self, ch: int) -> int:
        return self.arrive.data_ptr() + ch * self.arrive.shape[1] * 8

    def traffic_matrix(self) -> torch.Tensor:
        """Token traffic matrix [src, dst] of the last routed step (device tensor)."""
        return self.traffic

    # ---- forward ---------------------------------------------------------------------------------
    def route(self, logits: torch.Tensor, bias: Optional[torch.Tensor] = None) -> RouteState:
        C = self._C
        T = logits.shape[0]
        assert T <= self.T and logits.shape[1] == self.E and logits.dtype == torch.float32
        if self.graph_mode:
            topk_idx, topk_w, dest_row = (t[:T] for t in self._static_route)
        else:
            topk_idx = torch.empty(T, self.K, dtype=torch.int32, device=logits.device)
            topk_w = torch.empty(T, self.K, dtype=torch.float32, device=logits.device)
            dest_row = torch.empty(T, self.K, dtype=torch.int32, device=logits.device)
        nb = (T + C.ROUTE_TOKENS_PER_BLOCK - 1) // C.ROUTE_TOKENS_PER_BLOCK
        C.route_topk(logits.contiguous(), bias, self.K, topk_idx, topk_w, self.slot_in_block, self.block_cnt[:nb])
        self.epoch += 1
        ed = self.epoch_dev.data_ptr() if self.graph_mode else 0
        C.splits_scan(self.comm.heap, self._off(self.counts), self._flag_off(0), self.epoch, self.block_cnt[:nb], self.block_base[:nb], self.send_base,
                      self.send_cnt, self.group_off, self.group_rows, self.arrive_target[: 2 if self.training else 1], self.traffic, 2 if self.training else 1,
                      gemm.row_align(), self.cap, self.status,
                      self.timeout_ns, self.send_pos if self.overlap else None, ed, self.tile_target, self.tile_rows)
        return RouteState(topk_idx, topk_w, dest_row, self.slot_in_block, self.block_base, self.send_base, self.group_off, self.group_rows,
                          0 if self.graph_mode else self.epoch)

    def can_fuse_gate(self) -> bool:
        """Whether ``route_fused`` (RMSNorm + router logits + top-k in one kernel) covers this layer."""
        C = self._C
        return self.E <= 32 and self.H <= 8192 and C.norm_gate_smem_bytes(self.E, self.H, self.K, True) <= 220 * 1024 and not self.graph_mode

    def route_fused(self, h: torch.Tensor, norm_w: torch.Tensor, gate: torch.Tensor, eps: float, bias: Optional[torch.Tensor] = None):
        """RMSNorm of ``h``, router logits against ``gate`` and the routing of ``route`` in one kernel:
        returns ``(RouteState, hn, rstd, logits)`` with ``hn`` the normalised rows (the MoE input)."""
        C = self._C
        T = h.shape[0]
        assert T <= self.T and h.shape[1] == self.H and gate.shape == (self.E, self.H)
        dev = h.device
        topk_idx = torch.empty(T, self.K, dtype=torch.int32, device=dev)
        topk_w = torch.empty(T, self.K, dtype=torch.float32, device=dev)
        dest_row = torch.empty(T, self.K, dtype=torch.int32, device=dev)
        hn = torch.empty_like(h)
        rstd = torch.empty(T, dtype=torch.float32, device=dev)
        logits = torch.empty(T, self.E, dtype=torch.float32, device=dev)
        nb = (T + C.ROUTE_TOKENS_PER_BLOCK - 1) // C.ROUTE_TOKENS_PER_BLOCK
        C.norm_gate_route(h, norm_w, gate, bias, self.K, eps, hn, rstd, logits, topk_idx, topk_w, self.slot_in_block, self.block_cnt[:nb])
        self.epoch += 1
        C.splits_scan(self.comm.heap, self._off(self.counts), self._flag_off(0), self.epoch, self.block_cnt[:nb], self.block_base[:nb], self.send_base,
                      self.send_cnt, self.group_off, self.group_rows, self.arrive_target[: 2 if self.training else 1], self.traffic, 2 if self.training else 1,
                      gemm.row_align(), self.cap, self.status, self.timeout_ns, self.send_pos if self.overlap else None, 0, self.tile_target, self.tile_rows)
        rs = RouteState(topk_idx, topk_w, dest_row, self.slot_in_block, self.block_base, self.send_base, self.group_off, self.group_rows, self.epoch)
        return rs, hn, rstd, logits

    def dispatch(self, x: torch.Tensor, rs: RouteState) -> None:
        C = self._C
        send_list = xq = xs = None
        if not self.fp8:
            C.zero_pad_rows(self.x_recv, rs.group_off, rs.group_rows)  # on the main stream: ordered before any consumer
        if self.overlap:
            # The sending order and (fp8) the quantised rows are made on the main stream, with the whole GPU, before the
            # gated GEMM is queued behind them. Only the sends themselves go to the side stream: ordered after routing,
            # concurrent with whatever the main stream queues next (the gated expert GEMM); the main stream re-joins
            # in experts_forward.
            C.build_send_list(rs.topk_idx, rs.slot_in_block, rs.block_base, self.send_pos, self.send_list, self.status)
            send_list = self.send_list
            if self.fp8:
                # Sorted sending gives every (token, slot) entry a warp of its own: quantise each row once, entries copy bytes.
                if self._xq_send is None:
                    self._xq_send = torch.empty(self.T, self.H, dtype=torch.uint8, device=x.device)
                    self._xs_send = torch.empty(self.T, self.H // 128, dtype=torch.float32, device=x.device)
                xq, xs = self._xq_send, self._xs_send
                C.quantise_rows(x, xq, xs, self.comm_ctas)
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            self.side.wait_event(ev)
            x.record_stream(self.side)
            ctx = torch.cuda.stream(self.side)
            ctx.__enter__()
        try:
            if self.fp8:
                C.dispatch_push(self.comm.heap, x, rs.topk_idx, None, rs.slot_in_block, rs.block_base, rs.send_base, rs.dest_row, True, True,
                                self._off(self.xq_recv), self._off(self.xs_recv), self.arrive._symm_off, 0, 0, self.status, self.timeout_ns,
                                4 * self.overlap_reserve_sms if self.overlap else self.comm_ctas, send_list, self.tile_rows, self.ntiles, xq, xs)
            else:
                C.dispatch_push(self.comm.heap, x, rs.topk_idx, None, rs.slot_in_block, rs.block_base, rs.send_base, rs.dest_row, True, False,
                                self._off(self.x_recv), 0, self.arrive._symm_off, 0, 0, self.status, self.timeout_ns,
                                4 * self.overlap_reserve_sms if self.overlap else self.comm_ctas, send_list, self.tile_rows, self.ntiles)
        finally:
            if self.overlap:
                self._dispatch_done = torch.cuda.Event()
                self._dispatch_done.record(self.side)
                ctx.__exit__(None, None, None)

    def _join_dispatch(self) -> None:
        """Main stream waits for the side-stream dispatch (its dest_row table and its use of x)."""
        if self.overlap and getattr(self, "_dispatch_done", None) is not None:
            torch.cuda.current_stream().wait_event(self._dispatch_done)
            self._dispatch_done = None

    def experts_forward(self, w13: torch.Tensor, w2: torch.Tensor, rs: RouteState) -> None:
        C = self._C
        if self.tile_rows:   # forward-only layer: the producer of the first GEMM waits tile by tile
            gate, gate_tile = (self._arrive_ptr(0), self.tile_target[0]), self.tile_rows
        else:
            gate, gate_tile = (self._arrive_ptr(0), self.arrive_target[0]), 0
        if self.fp8_direct:
            # e4m3 rows and their scales go straight into the GEMM: converter warps build the bf16 tiles in
            # shared memory, rows past a group's real end are zeros there. No dequantised copy, no separate wait.
            gemm.grouped_gemm_fwd(self.xq_recv, w13, rs.group_off, self.act, swiglu=True, gate=gate, a_scales=self.xs_recv, group_rows=rs.group_rows,
                                  gate_tile_rows=gate_tile, ctas=self.gemm1_ctas)
        else:
            if self.fp8:
                C.wait_counters(self._arrive_ptr(0), self.tile_target[0] if self.tile_rows else self.arrive_target[0], self.status, self.timeout_ns)
                C.dequant_fp8(self.xq_recv, self.xs_recv, self.x_recv, rs.group_off.data_ptr() + 4 * self.El)
                C.zero_pad_rows(self.x_recv, rs.group_off, rs.group_rows)
                gate = None
            # A gated GEMM leaves SMs to the dispatch it waits for; an ungated one (every row is in) takes them all.
            gemm.grouped_gemm_fwd(self.x_recv, w13, rs.group_off, self.act, swiglu=True, gate_up_out=self.gu if self.training else None, gate=gate,
                                  gate_tile_rows=gate_tile, ctas=self.gemm1_ctas if gate is not None else None)
        gemm.grouped_gemm_fwd(self.act, w2, rs.group_off, self.y)
        self._join_dispatch()
        C.peer_signal(self.comm.heap, self._flag_off(1), rs.epoch, self.epoch_dev.data_ptr() if self.graph_mode else 0)

    def combine(self, rs: RouteState, weights: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        T = rs.topk_idx.shape[0]
        if out is None:
            out = torch.empty(T, self.H, dtype=torch.bfloat16, device=rs.topk_idx.device)
        self._C.combine_pull(self.comm.heap, self.E, rs.topk_idx, rs.dest_row, weights, self._off(self.y), self._flag_off(1), rs.epoch, out, None, None,
                             self.H, self.status, self.timeout_ns, self.comm_ctas, self.epoch_dev.data_ptr() if self.graph_mode else 0)
        return out

    def forward(self, x: torch.Tensor, logits: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, bias: Optional[torch.Tensor] = None,
                weights: Optional[torch.Tensor] = None):
        with nvtx_range("route"):
            rs = self.route(logits, bias)
        with nvtx_range("dispatch"):
            self.dispatch(x, rs)
        with nvtx_range("experts"):
            self.experts_forward(w13, w2, rs)
        with nvtx_range("combine"):
            out = self.combine(rs, rs.topk_w if weights is None else weights)
        return out, rs

    def plan_last_step(self, topo=None, **plan_opts):
        """Host-side view of the last routed step: reads the device traffic matrix (this
        synchronises), converts tokens to bytes and runs the scheduler on it. Returns
        ``(plan, cost)`` with the cost under a 900 GB/s NVLink model - what a planned all-to-all(v)
        of the same dispatch would look like (stages, modeled time, port bound)."""
        from .. import sched

        tokens = self.traffic.cpu().numpy().astype("int64")
        row_bytes = self.H * (1 if self.fp8 else 2)
        topo = topo or sched.Topology.flat(self.comm.world)
        plan = sched.build_plan(tokens * row_bytes, topo, **plan_opts)
        nv = sched.nvlink_model(900.0, 2.0)
        return plan, plan.cost(nv, nv, 1e-6)

    # ---- backward --------------------------------------------------------------------------------
    def backward(self, grad_out: torch.Tensor, rs: RouteState, weights: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, dw13: torch.Tensor,
                 dw2: torch.Tensor, after_dw2=None):
        """Returns (grad_x [T, H], grad_weights [T, K]); fills dw13 / dw2. ``after_dw2()`` is called
        as soon as the W2 gradient kernel is queued (nothing later in the pass reads W2)."""
        C = self._C
        T = rs.topk_idx.shape[0]
        dev = grad_out.device
        grad_w = torch.empty(T, self.K, dtype=torch.float32, device=dev)
        # d(weights): <grad_out[t], y_row(t, j)> - the expert outputs are still in place on the peers.
        C.combine_pull(self.comm.heap, self.E, rs.topk_idx, rs.dest_row, None, self._off(self.y), self._flag_off(1), rs.epoch, None, grad_out, grad_w,
                       self.H, self.status, self.timeout_ns, self.comm_ctas, 0)
        # Transposed combine: push w * grad_out to the expert rows (channel 1).
        C.zero_pad_rows(self.dy_recv, rs.group_off, rs.group_rows)
        C.dispatch_push(self.comm.heap, grad_out, rs.topk_idx, weights, rs.slot_in_block, rs.block_base, rs.send_base, rs.dest_row, False, False,
                        self._off(self.dy_recv), 0, self.arrive._symm_off + self.El * 8, self._flag_off(2), rs.epoch, self.status, self.timeout_ns,
                        self.comm_ctas, None)
        gate = (self._arrive_ptr(1), self.arrive_target[1])
        if gemm.USE_PAIR:  # d(act) never leaves the tensor memory: the dgrad epilogue applies the SwiGLU backward
            gemm.grouped_gemm_dgrad(self.dy_recv, w2, rs.group_off, self.dgu, gate=gate, swiglu_bwd_of=self.gu)
        else:
            gemm.grouped_gemm_dgrad(self.dy_recv, w2, rs.group_off, self.dact, gate=gate)
        gemm.grouped_gemm_wgrad(self.dy_recv, self.act, rs.group_off, dw2)
        if after_dw2 is not None:
            after_dw2()
        if not gemm.USE_PAIR:
            C.swiglu_bwd(self.gu, self.dact, self.dgu, rs.group_off.data_ptr() + 4 * self.El)
        gemm.grouped_gemm_dgrad(self.dgu, w13, rs.group_off, self.dx_recv)
        gemm.grouped_gemm_wgrad(self.dgu, self.x_recv, rs.group_off, dw13)
        C.peer_signal(self.comm.heap, self._flag_off(3), rs.epoch, 0)
        grad_x = torch.empty(T, self.H, dtype=torch.bfloat16, device=dev)
        # Transposed dispatch: every token pulls and sums the gradients of its k rows.
        C.combine_pull(self.comm.heap, self.E, rs.topk_idx, rs.dest_row, None, self._off(self.dx_recv), self._flag_off(3), rs.epoch, grad_x, None, None,
                       self.H, self.status, self.timeout_ns, self.comm_ctas, 0)
        return grad_x, grad_w
