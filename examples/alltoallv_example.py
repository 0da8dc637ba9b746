"""Skewed all-to-all(v) through the Communicator, checked against torch.distributed.

    torchrun --nproc-per-node 4 examples/alltoallv_example.py
"""
import os

import numpy as np
import torch
import torch.distributed as dist

from fast_b200.parallel import Communicator
from fast_b200.sched import TrafficMatrix


def main():
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    tm = TrafficMatrix.zipf(world, skew=1.0, row_bytes=64 << 20, seed=3)      # the same matrix on every rank
    with Communicator(heap_bytes=1 << 30) as comm:
        s = comm.schedule(tm.units, unit_bytes=tm.unit_bytes, kind="auto", verify=True)
        x = torch.randint(0, 255, (s.input_bytes,), dtype=torch.uint8, device="cuda")
        out = comm.alloc(max(s.max_bytes["output"], 1), torch.uint8)          # peers write here directly
        comm.all_to_all_v(out, x, s)
        comm.check()                                                          # raises if a device wait gave up
        ref = torch.empty(s.output_bytes, dtype=torch.uint8, device="cuda")
        dist.all_to_all_single(ref, x, tm.output_splits(rank), tm.input_splits(rank))
        assert torch.equal(out[: s.output_bytes], ref)
        if rank == 0:
            print(f"{world} ranks, {np.asarray(tm.bytes).sum() >> 20} MiB moved, busiest port {tm.port_bound_bytes() >> 20} MiB, "
                  f"bound {tm.lower_bound_us():.0f} us: output equals all_to_all_single")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
