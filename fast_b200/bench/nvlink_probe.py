"""One process, two GPUs: rank 0's transport kernels (all-to-all(v) push, fused dispatch, fused combine)
run alone on GPU 0 against real peer memory on GPU 1, so that a profiler can count the NVLink bytes
of a single launch beside the bytes the operation must move.

    python -m fast_b200.bench.nvlink_probe [--mb 256] [--tokens 16384] [--hidden 7168]
    ncu --section Nvlink --metrics nvltx__bytes.sum,nvlrx__bytes.sum,gpu__time_duration.sum --clock-control none \
        -k regex:"a2a_push|dispatch_push|combine_pull" -c 6 python -m fast_b200.bench.nvlink_probe

The peer rank launches nothing: its "buffers may be written" flag is set by hand, nothing is sent
back, so no kernel here waits for another GPU and a profiler may replay each launch. Every number
printed is per launch: algorithmic bytes that must cross the link, CUDA-event time, GB/s.
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

from .. import runtime, sched
from ..sched import PlanKind, Topology


def _time(fn, iters=5, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, default=256, help="bytes rank 0 pushes to rank 1 in the all-to-all(v) case (MiB)")
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--cta-sweep", type=int, nargs="*", default=[], help="also time the all-to-all(v) push with these CTA counts (one CTA per SM)")
    a = ap.parse_args()
    assert torch.cuda.device_count() >= 2, "needs two GPUs in one process"
    C = runtime.ext()
    torch.cuda.set_device(0)
    T, H = a.tokens, a.hidden
    nbytes = a.mb << 20
    heap_bytes = nbytes + 3 * T * H * 2 + (64 << 20)
    h0, h1 = C.SymmHeap.create_device_group([0, 1], heap_bytes)
    status = C.StatusBlock()
    timeout_ns = int(5e9)
    out = {}

    def alloc(n):  # same offset on both ranks
        o0, o1 = h0.alloc(n), h1.alloc(n)
        assert o0 == o1
        return o0

    # ---- all-to-all(v): rank 0 -> rank 1, fan-out plan, rank 1's ready flag preset ------------------------------
    sig_off = alloc(C.SIG_WORDS * 8)
    out_off = alloc(nbytes)
    sig0 = h0.tensor(sig_off, [C.SIG_WORDS], torch.int64)
    sig0[1] = 1 << 40                                          # peer 1 "entered" every epoch this run will use
    m = np.array([[0, nbytes], [0, 0]], dtype=np.int64)
    plan = sched.build_plan(m, Topology.flat(2), kind=PlanKind.FANOUT, split_align=16)
    low = plan.lower(0, 1, 1 << 20)
    prog = C.A2AProgram(torch.from_numpy(low["items"]), [int(x) for x in low["expect_rail_bytes"]], int(low["expect_output_bytes"]),
                        int(low["expect_balance_bytes"]), 0)
    src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda:0")
    epoch = [0]

    def push(bulk=False, ctas=148):
        epoch[0] += 1
        C.a2a_launch(prog, h0, [src.data_ptr(), 0, h0.base_ptr(0), h0.base_ptr(0)], [0, out_off, 0, 0], sig_off, epoch[0], status, timeout_ns,
                     min(ctas, prog.n_items), 512, 0, bulk)

    for name, bulk in (("a2a_push", False), ("a2a_push_bulk_copy", True)):
        ms = _time(lambda: push(bulk), a.iters)
        out[name] = {"link_bytes": nbytes, "ms": round(ms, 4), "GBps": round(nbytes / ms / 1e6, 1)}
    # how many SMs each copy loop needs to fill the link (one CTA per SM): GB/s by CTA count
    out["a2a_push_GBps_by_ctas"] = {str(c): round(nbytes / _time(lambda: push(False, c), a.iters) / 1e6, 1) for c in a.cta_sweep}
    out["a2a_push_bulk_copy_GBps_by_ctas"] = {str(c): round(nbytes / _time(lambda: push(True, c), a.iters) / 1e6, 1) for c in a.cta_sweep}
    got = h1.tensor(out_off, [nbytes], torch.uint8)
    assert torch.equal(got.to("cuda:0"), src), "pushed bytes differ"

    # ---- fused dispatch: every token's row goes to expert 1 (owned by rank 1), bf16 and e4m3 ----------------------
    i32 = dict(dtype=torch.int32, device="cuda:0")
    x = torch.randn(T, H, device="cuda:0").to(torch.bfloat16)
    topk = torch.ones(T, 1, **i32)
    dest = torch.arange(T, **i32).reshape(T, 1)
    zeros = torch.zeros(T, 1, **i32)
    base = torch.zeros(1, 2, **i32)
    send_base = torch.zeros(2, **i32)
    recv_off = alloc(T * H * 2)
    scale_off = alloc(T * (H // 128) * 4)
    arrive_off = alloc(64 * 8)
    y_off = alloc(T * H * 2)
    for name, fp8 in (("dispatch_push_bf16", False), ("dispatch_push_e4m3", True)):
        fn = lambda: C.dispatch_push(h0, x, topk, None, zeros, base, send_base, dest, False, fp8, recv_off, scale_off, arrive_off, 0, 0, status, timeout_ns,
                                     4 * 148, None)
        ms = _time(fn, a.iters)
        b = T * H * (1 if fp8 else 2) + (T * (H // 128) * 4 if fp8 else 0)
        out[name] = {"link_bytes": b, "ms": round(ms, 4), "GBps": round(b / ms / 1e6, 1)}
    # the same e4m3 rows quantised once beforehand: the dispatch entries only copy bytes (sorted order = token order here)
    xq = torch.empty(T, H, dtype=torch.uint8, device="cuda:0")
    xs = torch.empty(T, H // 128, dtype=torch.float32, device="cuda:0")
    send_list = torch.arange(T, **i32)
    ms = _time(lambda: C.quantise_rows(x, xq, xs, 4 * 148), a.iters)
    out["quantise_rows_local"] = {"link_bytes": 0, "ms": round(ms, 4), "GBps_local_read_plus_write": round(T * H * 3 / ms / 1e6, 1)}
    fn = lambda: C.dispatch_push(h0, x, topk, None, zeros, base, send_base, dest, False, True, recv_off, scale_off, arrive_off, 0, 0, status, timeout_ns,
                                 4 * 148, send_list, 0, 0, xq, xs)
    ms = _time(fn, a.iters)
    b = T * H + T * (H // 128) * 4
    out["dispatch_push_e4m3_prequantised"] = {"link_bytes": b, "ms": round(ms, 4), "GBps": round(b / ms / 1e6, 1)}
    # ---- fused combine: every token pulls its one row from rank 1 ----------------------------------------------
    res = torch.empty(T, H, dtype=torch.bfloat16, device="cuda:0")
    w = torch.ones(T, 1, dtype=torch.float32, device="cuda:0")
    ms = _time(lambda: C.combine_pull(h0, 2, topk, dest, w, y_off, arrive_off, 0, res, None, None, H, status, timeout_ns, 4 * 148, 0), a.iters)
    out["combine_pull"] = {"link_bytes": T * H * 2, "ms": round(ms, 4), "GBps": round(T * H * 2 / ms / 1e6, 1)}
    code = status.read()[0]
    assert code == 0, f"a device wait or check reported code {code}"
    print(json.dumps(out))


if __name__ == "__main__":
    main()
