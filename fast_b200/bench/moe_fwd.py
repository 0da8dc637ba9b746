"""MoE expert-parallel forward latency (DeepSeek-V3-like shapes): dispatch, experts, combine.

    torchrun --nproc-per-node N -m fast_b200.bench.moe_fwd [--tokens 4096 --hidden 7168 --inter 2048
        --experts-per-gpu 32 --top-k 8 --fp8]

4096 tokens per rank, 32 routed experts per GPU, top-8 softmax routing of N(0,1) gate logits plus a
per-expert N(0,1.5) bias (skew), dispatch in bf16 or e4m3 with 1x128 scales, SwiGLU experts with
random-init bf16 weights (std 0.02), top-k weighted bf16 combine. Device-timed per phase with CUDA
events, max over ranks. The NCCL column runs the same layer with torch.distributed
all_to_all_single for both exchanges and torch ops for permute / reduce.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .. import runtime
from ..parallel import Communicator
from ..parallel.ep import ExpertParallel
from ..utils.results import ResultLog


def _max_over_ranks(vals, world):
    t = torch.tensor(vals, device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]


def nccl_reference_layer(x, idx, w, w13, w2, world, E):
    """dispatch -> experts -> combine with NCCL all-to-all and torch ops (the baseline path)."""
    from ..models.moe import split_gate_up

    T, K = idx.shape
    El = E // world
    flat = idx.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    tok = order // K
    send = x[tok]
    counts = torch.bincount(flat, minlength=E)
    recv_counts = torch.empty_like(counts)
    if world > 1:
        dist.all_to_all_single(recv_counts, counts)
    else:
        recv_counts.copy_(counts)
    in_splits = counts.view(world, El).sum(1).tolist()
    out_splits = recv_counts.view(world, El).sum(1).tolist()
    recv = torch.empty(sum(out_splits), x.shape[1], dtype=x.dtype, device=x.device)
    if world > 1:
        dist.all_to_all_single(recv, send, out_splits, in_splits)
    else:
        recv.copy_(send)
    # rows arrive grouped by source rank then expert; regroup by expert
    rc = recv_counts.view(world, El)
    eid = torch.repeat_interleave(torch.arange(El, device=x.device).repeat(world), rc.reshape(-1))
    perm = torch.argsort(eid, stable=True)
    h = recv[perm]
    w1, w3 = split_gate_up(w13)
    out = torch.empty_like(h)
    start = 0
    per_e = rc.sum(0).tolist()
    for e in range(El):
        n = per_e[e]
        if n:
            seg = h[start:start + n]
            out[start:start + n] = (torch.nn.functional.silu(seg @ w1[e].t()) * (seg @ w3[e].t())) @ w2[e].t()
        start += n
    back = torch.empty_like(out)
    back[perm] = out
    ret = torch.empty_like(send)
    if world > 1:
        dist.all_to_all_single(ret, back, in_splits, out_splits)
    else:
        ret.copy_(back)
    y = torch.zeros(T, x.shape[1], dtype=torch.float32, device=x.device)
    y.index_add_(0, tok, ret.float() * w.reshape(-1)[order].unsqueeze(1))
    return y.to(x.dtype)


def heap_bytes_needed(world, tokens, hidden, top_k, experts_per_gpu, fp8):
    cap = world * tokens * min(top_k, experts_per_gpu) + 256 * experts_per_gpu
    return int(cap * hidden * (3 if fp8 else 4.2)) + (256 << 20)


def measure(comm, tokens=4096, hidden=7168, inter=2048, experts_per_gpu=32, top_k=8, fp8=False, iters=20, warmup=5, skip_nccl=False, overlap=False, fp8_direct=False, reserve_sms=16):
    """Runs the forward layer on an existing communicator and returns the result dict (every rank)."""
    rank, world = comm.rank, comm.world
    E, K, H, I, T, El = experts_per_gpu * world, top_k, hidden, inter, tokens, experts_per_gpu
    eng = ExpertParallel(comm, E, H, I, K, T, fp8_dispatch=fp8, training=False, overlap_dispatch=overlap, fp8_direct=fp8_direct, overlap_reserve_sms=reserve_sms)
    g = torch.Generator(device="cuda").manual_seed(7)      # same on every rank: the bias is replicated
    bias = torch.randn(E, generator=g, device="cuda") * 1.5
    gr = torch.Generator(device="cuda").manual_seed(100 + rank)
    x = torch.randn(T, H, generator=gr, device="cuda").to(torch.bfloat16)
    logits = torch.randn(T, E, generator=gr, device="cuda")
    w13 = (torch.randn(El, 2 * I, H, generator=gr, device="cuda") * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(El, H, I, generator=gr, device="cuda") * 0.02).to(torch.bfloat16)
    C = runtime.ext()

    ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
    acc = [0.0] * 5  # four phases + whole layer
    out = None
    for it in range(warmup + iters):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ev[0].record()
        rs = eng.route(logits, bias)
        ev[1].record()
        eng.dispatch(x, rs)
        if not overlap:
            # phase boundary for timing only: all rows of this rank's experts have landed
            C.wait_counters(eng._arrive_ptr(0), eng.tile_target[0] if eng.tile_rows else eng.arrive_target[0], eng.status, eng.timeout_ns)
        ev[2].record()
        eng.experts_forward(w13, w2, rs)
        ev[3].record()
        out = eng.combine(rs, rs.topk_w)
        ev[4].record()
        torch.cuda.synchronize()
        if it >= warmup:
            for p in range(4):
                acc[p] += ev[p].elapsed_time(ev[p + 1]) * 1e3 / iters
            acc[4] += ev[0].elapsed_time(ev[4]) * 1e3 / iters
    comm.check()
    # Combine alone: every peer's rows are final by now, so this is the pure pull + reduce time
    # (inside the layer, a rank's combine also absorbs the wait for the slowest peer's experts).
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for _ in range(iters):
        out = eng.combine(rs, rs.topk_w)
    c1.record()
    torch.cuda.synchronize()
    combine_alone_us = _max_over_ranks([c0.elapsed_time(c1) * 1e3 / iters], world)[0]
    route_us, dispatch_us, experts_us, combine_us, layer_us = _max_over_ranks(acc, world)
    tm = eng.traffic_matrix().cpu().numpy()
    res = {"bench": "moe_forward", "world": world, "overlap_dispatch": overlap, "overlap_reserve_sms": eng.overlap_reserve_sms, "tokens_per_rank": T, "hidden": H, "inter": I, "experts": E, "top_k": K,
           "dispatch_dtype": "fp8_e4m3_1x128" if fp8 else "bf16", "expert_feed": "e4m3 rows converted inside the GEMM" if eng.fp8_direct else ("dequantised to bf16 first" if fp8 else "bf16"), "route_us": round(route_us, 1), "dispatch_us": round(dispatch_us, 1),
           "experts_us": round(experts_us, 1), "combine_us": round(combine_us, 1), "combine_alone_us": round(combine_alone_us, 1),
           "dispatch_plus_combine_us": round(dispatch_us + combine_alone_us, 1),
           "layer_us": round(layer_us, 1),  # whole layer per iteration, max over ranks (phase maxima above fall on different ranks)
           "max_rows_in": int(tm.sum(0).max()), "max_rows_out": int(tm.sum(1).max())}
    row_bytes = H * (1 if fp8 else 2) + (H // 128 * 4 if fp8 else 0)
    if world > 1:
        off_in = int((tm.sum(0) - tm.diagonal()).max())
        off_out = int((tm.sum(1) - tm.diagonal()).max())
        res["dispatch_bound_us_at_770GBps"] = round(max(off_in, off_out) * row_bytes / 770e9 * 1e6, 1)
        res["combine_bound_us_at_770GBps"] = round(max(off_in, off_out) * H * 2 / 770e9 * 1e6, 1)
    if not skip_nccl:
        idx, w = rs.topk_idx, rs.topk_w
        for _ in range(2):
            ref = nccl_reference_layer(x, idx, w, w13, w2, world, E)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = max(3, iters // 4)
        e0.record()
        for _ in range(n):
            ref = nccl_reference_layer(x, idx, w, w13, w2, world, E)
        e1.record()
        torch.cuda.synchronize()
        res["nccl_torch_layer_us"] = round(_max_over_ranks([e0.elapsed_time(e1) * 1e3 / n], world)[0], 1)
        err = ((out.float() - ref.float()).abs().max() / (ref.float().abs().max() + 1e-9)).item()
        res["max_rel_err_vs_nccl_torch"] = round(err, 5)
    return res


def measure_graph(comm, tokens, hidden, inter, experts_per_gpu, top_k, iters=50):
    """Whole forward layer (gate GEMM to combined output) launched eagerly vs replayed from one CUDA
    graph; the difference is launch and host overhead, which dominates at small token counts."""
    from ..models import MoELayer

    world = comm.world
    layer = MoELayer(comm, hidden, inter, experts_per_gpu * world, top_k, max_tokens=tokens, training=False, graph_mode=True)
    layer.eval()
    layer.capture(tokens)
    x = torch.randn(tokens, hidden, device="cuda").to(torch.bfloat16)

    def timed(fn):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return _max_over_ranks([e0.elapsed_time(e1) * 1e3 / iters], world)[0]

    with torch.no_grad():
        eager = timed(lambda: layer._infer(x))
        graph = timed(lambda: layer.forward_graphed(x))
    comm.check()
    return {"bench": "moe_forward_graph", "world": world, "tokens_per_rank": tokens, "hidden": hidden, "inter": inter,
            "experts": experts_per_gpu * world, "top_k": top_k, "eager_layer_us": round(eager, 1), "graph_layer_us": round(graph, 1)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--inter", type=int, default=2048)
    ap.add_argument("--experts-per-gpu", type=int, default=32)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--fp8", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--skip-nccl", action="store_true")
    ap.add_argument("--graph", action="store_true", help="time the whole forward layer eagerly and as one CUDA graph replay")
    ap.add_argument("--fp8-direct", action="store_true", help="with --fp8: feed the e4m3 rows to the expert GEMM as they are (converter warps) instead of dequantising first")
    ap.add_argument("--overlap", action="store_true", help="send rows expert by expert on a side stream while the gated GEMM runs (dispatch_us then only times the launch)")
    ap.add_argument("--reserve-sms", type=int, default=16, help="with --overlap: SMs the first expert GEMM leaves to the dispatch kernel")
    ap.add_argument("--out", default="", help="append the result row to this file (JSON lines)")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = Communicator(heap_bytes=heap_bytes_needed(world, a.tokens, a.hidden, a.top_k, a.experts_per_gpu, a.fp8), device=local, timeout_s=20.0)
    if a.graph:
        res = measure_graph(comm, a.tokens, a.hidden, a.inter, a.experts_per_gpu, a.top_k, max(a.iters, 20))
    else:
        res = measure(comm, a.tokens, a.hidden, a.inter, a.experts_per_gpu, a.top_k, a.fp8, a.iters, a.warmup, a.skip_nccl, a.overlap, a.fp8_direct, a.reserve_sms)
    if rank == 0:
        print(json.dumps(res), flush=True)
        ResultLog(a.out or None, "moe_fwd").add(res)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
