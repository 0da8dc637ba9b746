"""All-to-all(v) bandwidth bench: this runtime's staged and fan-out plans against NCCL.

    torchrun --nproc-per-node N -m fast_b200.bench.a2a --mode uniform|skewed [--sizes ...]

Device-timed with CUDA events on the launching stream, max over ranks, seeded matrices. The
reference's counterpart is its perf loop (nvidia/alltoall_nvshmem.cpp:172-381) and the AMD
tester's sweeps (amd/test_alltoall.cpp:1994-2596); algbw = bytes sent per rank / time.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist

from .. import sched
from ..parallel import Communicator
from ..sched import PlanKind, Topology
from ..utils.results import ResultLog


def _time_ms(fn, iters, warmup, batches=3):
    """Device time of one call of ``fn``: ``batches`` batches of ``iters`` back-to-back calls between CUDA
    events, each batch's mean taken as the max over ranks, the median batch reported. Launch-bound
    collectives on many processes see a late rank now and then; one such batch does not move the figure."""
    for _ in range(warmup):
        fn()
    means = []
    for _ in range(batches):
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        ev[0].record()
        for _ in range(iters):
            fn()
        ev[1].record()
        torch.cuda.synchronize()
        means.append(ev[0].elapsed_time(ev[1]) / iters)
    t = torch.tensor(means, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.median().item())


def _e2e_fresh_ms(comm, out, inp, m, kind, chunk, **opts):
    """Wall-clock cost of a collective on a matrix this communicator has never planned: traffic matrix
    in hand -> ``schedule()`` (hash, plan, validation, lowering, work-list upload) -> launch -> output
    complete. This is what a step with new routing pays; the device-timed columns reuse a schedule."""
    import time

    torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    s = comm.schedule(m, unit_bytes=1, kind=kind, chunk_bytes=chunk, **opts)
    t1 = time.perf_counter()
    comm.all_to_all_v(out, inp, s)
    torch.cuda.synchronize()
    t2 = time.perf_counter()
    t = torch.tensor([(t2 - t0) * 1e3, (t1 - t0) * 1e3], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0]), float(t[1])


def phase_breakdown(comm, out, inp, s, reps: int = 3) -> dict:
    """Per-phase completion of one scheduled collective, from device time stamps: microseconds from
    the rank's kernel start to the first start / last end of its balance, rail (inter-server stage),
    redistribute and direct work, max over ranks and mean over ``reps`` runs (the reference's
    load-balance / cross-node / restore columns, amd/test_alltoall.cpp:1432-1438)."""
    stamps = comm.new_phase_stamps()
    acc = {}
    for _ in range(reps):
        comm.clear_phase_stamps(stamps)
        torch.cuda.synchronize()
        dist.barrier()
        comm.all_to_all_v(out, inp, s, phase_stamps=stamps)
        torch.cuda.synchronize()
        ph = comm.read_phase_stamps(stamps)
        names = ["balance", "rail", "redistribute", "direct", "total"]
        v = torch.tensor([[ph.get(n, (0.0, 0.0))[0], ph.get(n, (0.0, 0.0))[1]] for n in names], device="cuda", dtype=torch.float64)
        lo = v[:, 0].clone()
        dist.all_reduce(v, op=dist.ReduceOp.MAX)
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        for i, n in enumerate(names):
            acc.setdefault(n, []).append((float(lo[i]), float(v[i, 1])))
    return {n: {"first_start_us": round(float(np.mean([x[0] for x in xs])), 1), "last_end_us": round(float(np.mean([x[1] for x in xs])), 1)}
            for n, xs in acc.items() if any(x[1] > 0 for x in xs)}


def nccl_alltoallv(out, inp, in_splits, out_splits):
    dist.all_to_all_single(out, inp, out_splits, in_splits)


def nccl_sendrecv_group(out, inp, in_splits, out_splits, rank, world):
    ops = []
    io = np.concatenate([[0], np.cumsum(in_splits)])
    oo = np.concatenate([[0], np.cumsum(out_splits)])
    for step in range(world):
        d = (rank + step) % world
        s = (rank - step) % world
        if in_splits[d]:
            ops.append(dist.P2POp(dist.isend, inp[io[d]:io[d + 1]], d))
        if out_splits[s]:
            ops.append(dist.P2POp(dist.irecv, out[oo[s]:oo[s + 1]], s))
    for w in dist.batch_isend_irecv(ops):
        w.wait()


def skewed_point(comm, row_bytes: int, skew: float, matrices: int = 3, iters: int = 5, warmup: int = 3, chunk=None):
    """One (row size, skew) point on an existing communicator: mean over seeded matrices of the
    device-timed completion (max over ranks) for NCCL all_to_all_single and for this runtime's
    fan-out and staged plans. Returns a dict of per-variant ms / per-rank algorithm GB/s."""
    rank, world = comm.rank, comm.world
    mats = [sched.workload_zipf_rows(world, skew, row_bytes, 1000 * mi + 7, 16) for mi in range(matrices)]
    need = max(int(m.sum(0).max()) for m in mats) + (1 << 20)
    out = comm.alloc(need, torch.uint8)
    g = torch.Generator(device="cuda").manual_seed(4321 + rank)
    inp = torch.randn(row_bytes // 2, generator=g, device="cuda", dtype=torch.bfloat16).view(torch.uint8)
    nccl_out = torch.empty(need, dtype=torch.uint8, device="cuda")
    acc = {}
    for m in mats:
        in_splits = [int(x) for x in m[rank]]
        out_splits = [int(x) for x in m[:, rank]]
        sent = int(m[rank].sum())
        bound = int(max((m.sum(0) - np.diag(m)).max(), (m.sum(1) - np.diag(m)).max()))
        variants = {"nccl_alltoallv": lambda: nccl_alltoallv(nccl_out[: sum(out_splits)], inp[:sent], in_splits, out_splits)}
        for name, kind in (("ours_fanout", PlanKind.FANOUT), ("ours_staged", PlanKind.STAGED)):
            s = comm.schedule(m, unit_bytes=1, kind=kind, chunk_bytes=chunk)
            variants[name] = (lambda s=s: comm.all_to_all_v(out, inp, s))
        for name, fn in variants.items():
            acc.setdefault(name, []).append((_time_ms(fn, iters, warmup), sent, bound))
    comm.check()
    comm.free(out)
    res = {"row_bytes": row_bytes, "skew": skew, "matrices": matrices, "world": world}
    for name, xs in acc.items():
        res[name] = {"ms": round(float(np.mean([x[0] for x in xs])), 4), "algbw_GBps": round(float(np.mean([x[1] / x[0] / 1e6 for x in xs])), 2),
                     "frac_of_770GBps_port_bound": round(float(np.mean([x[2] / 770e9 / (x[0] * 1e-3) for x in xs])), 4)}
    return res


def run(args):
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl")
    max_row = max(args.sizes)
    # Receive buffers must hold the heaviest column of any matrix that will be drawn.
    need = max_row
    def draw(size, skew, mi):
        if args.mode == "random":
            return sched.workload_uniform(world, 2 * size // world // 16, 1000 * mi + 7, True) * 16
        return sched.workload_zipf_rows(world, skew, size, 1000 * mi + 7, 16)

    if args.mode == "random":
        need = max(int(max(draw(size, None, mi).sum(0).max(), draw(size, None, mi).sum(1).max())) for size in args.sizes for mi in range(args.matrices))
    if args.mode == "skewed":
        for size in args.sizes:
            for skew in args.skews:
                for mi in range(args.matrices):
                    need = max(need, int(sched.workload_zipf_rows(world, skew, size, 1000 * mi + 7, 16).sum(0).max()))
    need = need + (1 << 20)
    # --servers S > 0 runs the two-tier plan (balance, rail stages, redistribute) over S virtual
    # servers of world/S GPUs; its staging needs up to ~2x the payload.
    topo = Topology(args.servers, world // args.servers) if args.servers else Topology.flat(world)
    comm = Communicator(heap_bytes=need * (4 if args.servers else 1) + (128 << 20), topo=topo, ctas=args.ctas or None, threads=args.threads)
    out = comm.alloc(need, torch.uint8)
    g = torch.Generator(device="cuda").manual_seed(1234 + rank)
    inp = torch.randn(max(max_row, need) // 2, generator=g, device="cuda", dtype=torch.bfloat16).view(torch.uint8)
    nccl_out = torch.empty(need, dtype=torch.uint8, device="cuda")
    results = []
    log = ResultLog(getattr(args, "out", "") or None, "a2a", world=world)
    for size in args.sizes:
        skews = args.skews if args.mode == "skewed" else [None]
        for skew in skews:
            acc, e2e, phases = {}, {}, None
            nmat = args.matrices if args.mode != "uniform" else 1
            for mi in range(nmat):
                if args.mode == "uniform":
                    per = max(size // world // 16 * 16, 16)
                    m = np.full((world, world), per, dtype=np.int64)
                else:
                    m = draw(size, skew, mi)
                in_splits = [int(x) for x in m[rank]]
                out_splits = [int(x) for x in m[:, rank]]
                sent = int(m[rank].sum())
                bound_bytes = int(max((m.sum(0) - np.diag(m)).max(), (m.sum(1) - np.diag(m)).max()))
                iters = max(3, min(args.iters, int(2e9 // max(sent, 1))))
                variants = {"nccl_alltoallv": lambda: nccl_alltoallv(nccl_out[: sum(out_splits)], inp[:sent], in_splits, out_splits)}
                if args.sendrecv:
                    variants["nccl_sendrecv"] = lambda: nccl_sendrecv_group(nccl_out, inp, in_splits, out_splits, rank, world)
                for name, kind, opts in [("ours_fanout", PlanKind.FANOUT, {}), ("ours_staged", PlanKind.STAGED, {}),
                                         ("ours_staged_bottleneck", PlanKind.STAGED, {"match": sched.MatchPolicy.BOTTLENECK}),
                                         ("ours_spreadout", PlanKind.SPREAD_OUT, {})] + ([("ours_single_burst", PlanKind.SINGLE_BURST, {})] if args.servers else []) + (
                                         [("ours_staged_pieces", PlanKind.STAGED, {"rail_segment_bytes": args.rail_segment})] if args.servers and args.rail_segment > 0 else []):
                    s = comm.schedule(m, unit_bytes=1, kind=kind, chunk_bytes=args.chunk or None, **opts)
                    variants[name] = (lambda s=s: comm.all_to_all_v(out, inp, s))
                if args.bulk:
                    # the same fan-out plan with the bulk-copy engine doing the transfers (one thread per CTA)
                    sb = comm.schedule(m, unit_bytes=1, kind=PlanKind.FANOUT, chunk_bytes=args.chunk or None)

                    def bulk_run(s=sb):
                        comm.bulk_copy = True
                        try:
                            comm.all_to_all_v(out, inp, s)
                        finally:
                            comm.bulk_copy = False

                    variants["ours_fanout_bulk_copy"] = bulk_run
                if args.p2p_baseline:
                    # The reference's executor style: the staged plan run phase by phase over library
                    # send/recv groups (here NCCL), host-synchronised between phases.
                    from ..parallel.p2p_executor import P2PExecutor

                    pex = P2PExecutor()
                    plan_p2p = sched.build_plan(m, topo, kind=PlanKind.STAGED, split_align=16)
                    prepared = pex.prepare(plan_p2p, 1, inp, nccl_out)  # descriptors built once, outside the timed loop
                    variants["staged_plan_over_nccl_sendrecv"] = prepared.run
                for name, fn in variants.items():
                    ms = _time_ms(fn, iters, args.warmup)
                    acc.setdefault(name, []).append((ms, sent, bound_bytes))
                comm.check()
                if args.e2e and args.mode != "uniform":
                    # a matrix of the same law that no cache has seen (seeds above any used for the timed columns)
                    fresh = draw(size, skew, 100000 + 1000 * len(results) + mi)
                    room = int(fresh.sum(0).max()) <= need and int(fresh.sum(1).max()) <= inp.numel()
                    if room:
                        for name, kind in (("ours_fanout", PlanKind.FANOUT), ("ours_staged", PlanKind.STAGED)):
                            e2e.setdefault(name, []).append(_e2e_fresh_ms(comm, out, inp, fresh, kind, args.chunk or None))
                        comm.check()
                if args.phases and mi == 0:
                    s = comm.schedule(m, unit_bytes=1, kind=PlanKind.STAGED, chunk_bytes=args.chunk or None)
                    phases = phase_breakdown(comm, out, inp, s)
                if mi == 0 and args.verify:
                    s = comm.schedule(m, unit_bytes=1, kind=PlanKind.STAGED, chunk_bytes=args.chunk or None)
                    comm.all_to_all_v(out, inp, s)
                    nccl_alltoallv(nccl_out[: sum(out_splits)], inp[:sent], in_splits, out_splits)
                    torch.cuda.synchronize()
                    assert torch.equal(out[: sum(out_splits)], nccl_out[: sum(out_splits)]), "mismatch vs NCCL"
            row = {"mode": args.mode, "world": world, "servers": args.servers or world, "row_bytes": size, "skew": skew, "matrices": nmat}
            for name, xs in acc.items():
                ms = float(np.mean([x[0] for x in xs]))
                row[name] = {"ms": round(ms, 4), "algbw_GBps": round(float(np.mean([x[1] / x[0] / 1e6 for x in xs])), 2),
                             "bound_frac_770": round(float(np.mean([x[2] / 770e9 / (x[0] * 1e-3) for x in xs])), 4)}
            for name, xs in e2e.items():
                row[name]["e2e_fresh_matrix_ms"] = round(float(np.mean([x[0] for x in xs])), 4)
                row[name]["schedule_ms"] = round(float(np.mean([x[1] for x in xs])), 4)
            if phases is not None:
                row["ours_staged"]["phases"] = phases
            results.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
                log.add(row)
    dist.barrier()
    dist.destroy_process_group()
    return results


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="skewed", choices=["uniform", "skewed", "random"], help="uniform: equal splits; skewed: Zipf rows; random: i.i.d. uniform entries (mean row = size)")
    ap.add_argument("--sizes", type=int, nargs="+", default=[64 << 20])
    ap.add_argument("--skews", type=float, nargs="+", default=[0.0, 0.5, 1.0, 1.5])
    ap.add_argument("--matrices", type=int, default=20, help="fresh seeded matrices per point")
    ap.add_argument("--bulk", action="store_true", help="also time the fan-out plan with bulk copies through shared memory instead of load/store loops")
    ap.add_argument("--e2e", action="store_true", help="also time schedule() + launch + completion on a never-seen matrix per drawn matrix (wall clock, max over ranks)")
    ap.add_argument("--phases", action="store_true", help="per-phase breakdown (balance / rail / redistribute / direct) of the staged plan from device time stamps")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--ctas", type=int, default=0, help="CTAs of the push kernel (0 = one per SM)")
    ap.add_argument("--threads", type=int, default=512)
    ap.add_argument("--chunk", type=int, default=0, help="work-item bytes (0 = chosen from the matrix)")
    ap.add_argument("--sendrecv", action="store_true")
    ap.add_argument("--p2p-baseline", action="store_true", help="also run the staged plan over NCCL send/recv groups (the reference's executor style)")
    ap.add_argument("--servers", type=int, default=0, help="treat the ranks as this many virtual servers (hierarchical FAST plan + single-burst ablation)")
    ap.add_argument("--verify", action="store_true")
    ap.add_argument("--rail-segment", type=int, default=0, help="with --servers: also time the staged plan with one arrival counter per this many bytes of rail staging")
    ap.add_argument("--out", default="", help="append every result row to this file (JSON lines)")
    run(ap.parse_args())


if __name__ == "__main__":
    main()
