"""Child of test_multi_process_bit_exact: one process per GPU, real peer memory."""
import os
import sys

os.environ.setdefault("FASTB_CHECK_SYMM", "1")  # every symmetric allocation is compared across the ranks (read at import)

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from fast_b200 import sched  # noqa: E402
from fast_b200.parallel import Communicator  # noqa: E402
from fast_b200.sched import PlanKind, Topology  # noqa: E402


def compat_on_real_peers(rank, world):
    """The reference-shaped classes on real peers: flash_t's token-unit schedule / all_to_all /
    all_to_all_2 / all_to_all_v against torch.distributed.all_to_all_single, forward and transposed,
    and the tester class with the reference's own workload generator."""
    from fast_b200.compat import FlashAllToAll, FlashComm, code_of

    hidden = 64
    server_n = 2 if world % 2 == 0 and world >= 4 else world
    fa = FlashAllToAll(rank, world, server_n, world // server_n, hidden, code_of(torch.bfloat16), heap_bytes=256 << 20)
    m = sched.workload_zipf_rows(world, 0.8, 3000, 11, 1)        # tokens
    for backward in (0, 1):
        mm = m.T if backward else m
        fa.schedule(m.reshape(-1), backward)
        x = torch.randn(int(mm[rank].sum()), hidden, device="cuda", generator=torch.Generator(device="cuda").manual_seed(100 + rank)).to(torch.bfloat16)
        ref = torch.empty(int(mm[:, rank].sum()), hidden, device="cuda", dtype=torch.bfloat16)
        dist.all_to_all_single(ref, x, [int(v) for v in mm[:, rank]], [int(v) for v in mm[rank]])
        y = torch.zeros_like(ref)
        fa.init_buffers(x, y)                                     # library-owned receive staging
        fa.all_to_all()
        fa.comm.check()
        assert torch.equal(y, ref), f"flash_t.all_to_all backward={backward} rank {rank}"
        fa.free_buffers()
        szs = fa.get_buffer_szs()
        y2 = fa.comm.alloc((max(int(mm.sum(axis=0).max()), 1), hidden), torch.bfloat16)   # caller-owned, symmetric (same size on every rank): written in place by the peers
        lbrecv = fa.comm.alloc((max(int(szs[2]), 1), hidden), torch.bfloat16)
        cros = fa.comm.alloc((max(int(szs[3]), 1), hidden), torch.bfloat16)
        y2.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        fa.all_to_all_2(x, y2, None, None, lbrecv, cros, None, None)
        fa.comm.check()
        assert torch.equal(y2[: ref.shape[0]], ref), f"flash_t.all_to_all_2 backward={backward} rank {rank}"
        y3 = torch.zeros_like(ref)
        fa.all_to_all_v(x, y3, [int(v) for v in mm[rank]], [int(v) for v in mm[:, rank]])
        fa.comm.check()
        assert torch.equal(y3, ref), f"flash_t.all_to_all_v backward={backward} rank {rank}"
        torch.cuda.synchronize()
        dist.barrier()
        for t in (cros, lbrecv, y2):
            fa.comm.free(t)
    fc = FlashComm(rank, world, world, comm=fa.comm, mean_units=1 << 14, generator="glibc", quiet=True)
    r1, r2 = fc.test_flash_alltoall(warmup=2, iters=3), fc.test_basic_alltoall(warmup=2, iters=3)
    assert r1["verified"] and r2["verified"] and r1["time_ms"] > 0, (r1, r2)
    dist.barrier()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    topos = [Topology.flat(world)] + ([Topology(2, world // 2)] if world % 2 == 0 and world >= 4 else [])
    for topo in topos:
        comm = Communicator(heap_bytes=256 << 20, topo=topo, ctas=16, threads=512)
        out = comm.alloc(32 << 20, torch.uint8)
        for kind in (PlanKind.STAGED, PlanKind.FANOUT, PlanKind.SPREAD_OUT, PlanKind.SINGLE_BURST):
            for seed in range(3):
                m = sched.workload_zipf_rows(world, 1.0, 4 << 20, seed, 16)
                s = comm.schedule(m, unit_bytes=1, kind=kind, chunk_bytes=256 << 10)
                ind = np.concatenate([[0], np.cumsum(m[rank])])
                inp = np.concatenate([((rank << 24) | (d << 16) | (np.arange(int(m[rank, d]) // 4) & 0xFFFF)).astype(np.int32) for d in range(world)])
                d_in = torch.from_numpy(inp).cuda()
                out.zero_()
                torch.cuda.synchronize()
                dist.barrier()
                want = np.concatenate([((src << 24) | (rank << 16) | (np.arange(int(m[src, rank]) // 4) & 0xFFFF)).astype(np.int32) for src in range(world)])
                for bulk in ((False, True) if seed == 0 else (False,)):   # also with the bulk-copy engine doing the transfers
                    comm.bulk_copy = bulk
                    out.zero_()
                    torch.cuda.synchronize()
                    dist.barrier()
                    for _ in range(2):
                        comm.all_to_all_v(out, d_in, s)
                    comm.check()
                    got = out[: want.size * 4].view(torch.int32).cpu().numpy()
                    assert np.array_equal(got, want), f"rank {rank} kind {kind} seed {seed} topo {topo} bulk {bulk}"
                comm.bulk_copy = False
        # torch.distributed-style entry point with uneven row splits
        rows = [(rank + d) % 3 + 1 for d in range(world)]
        x = torch.full((sum(rows), 8), float(rank), device="cuda", dtype=torch.bfloat16)
        recv_rows = [(s + rank) % 3 + 1 for s in range(world)]
        y = torch.empty((sum(recv_rows), 8), device="cuda", dtype=torch.bfloat16)
        comm.all_to_all_single(y, x, recv_rows, rows)
        comm.check()
        ref = torch.cat([torch.full((recv_rows[s], 8), float(s), dtype=torch.bfloat16) for s in range(world)])
        assert torch.equal(y.cpu(), ref)
        comm.free(out)
        dist.barrier()
    compat_on_real_peers(rank, world)
    if rank == 0:
        print("A2A_MP_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
