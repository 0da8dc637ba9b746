"""Launcher for the reference's own NVIDIA library (baseline/_ref/nv_build/libflash.so, built from
the unmodified sources by baseline/build_ref_nvshmem.sh) on one box: one process per GPU, each GPU
a "server" of its own, because the reference's scheduler does nothing for a single server
(nvidia/alltoall_nvshmem.cpp:549-561) and its class binds rank r to device ``r % dev_n``
(:411), so every process is given a device list that starts with its own GPU (the others stay
visible behind it, so that peer mappings between processes remain possible).

    python baseline/run_ref_flash.py --gpus 2 [--test flash|basic]

Status: the library builds and loads on a B200 box; this launcher has NOT been run yet. It is a
manual tool: nothing in the package, the tests or bench.py calls it. The reference's device waits
are unbounded, so its first run belongs in a call of its own, on 2 GPUs, under the launcher's
timeout, with NVLS switched off.

What it does: the parent starts N children with CUDA_VISIBLE_DEVICES=<i>,<the others>, a gloo process group for
the NVSHMEM unique id (as nvidia/flash_tester.py:11-22 does), then each child constructs
``flash_comm_t(rank, 1, world, uid)`` and calls ``test_flash_alltoall()`` or
``test_basic_alltoall()``; rank 0 of the reference prints its own "algbw ... GBps / total time"
lines, which the parent echoes.
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_ref", "nv_build", "libflash.so")


def child(rank: int, world: int, test: str) -> int:
    import torch
    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.ops.load_library(LIB)
    torch.classes.load_library(LIB)
    uid = torch.ops.flash_nvshmem.get_nvshmem_init_id() if rank == 0 else torch.zeros(128, dtype=torch.uint8)
    dist.broadcast(uid, src=0)
    torch.cuda.set_device(0)                                   # this rank's GPU is first in its device list
    comm = torch.classes.my_classes.flash_comm_t(rank, 1, world, uid)
    if test == "basic":
        comm.test_basic_alltoall()
    else:
        comm.test_flash_alltoall()
    dist.barrier()
    dist.destroy_process_group()
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--test", default="flash", choices=["flash", "basic"])
    ap.add_argument("--timeout", type=float, default=240.0, help="seconds before the children are stopped")
    ap.add_argument("--child", type=int, default=-1)
    a = ap.parse_args()
    if a.child >= 0:
        return child(a.child, a.gpus, a.test)
    if not os.path.exists(LIB):
        print(f"{LIB} is missing: run baseline/build_ref_nvshmem.sh first", file=sys.stderr)
        return 2
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=os.environ.get("MASTER_PORT", "29741"), NCCL_NVLS_ENABLE="0",
               NVSHMEM_DISABLE_NVLS="1", NVSHMEM_BOOTSTRAP="UID", NVSHMEM_IB_ENABLE_IBGDA="0", NVSHMEM_REMOTE_TRANSPORT="none")
    procs = []
    for r in range(a.gpus):
        order = [r] + [g for g in range(a.gpus) if g != r]
        e = dict(env, CUDA_VISIBLE_DEVICES=",".join(str(g) for g in order), RANK=str(r), WORLD_SIZE=str(a.gpus), LOCAL_RANK="0")
        procs.append(subprocess.Popen([sys.executable, os.path.abspath(__file__), "--gpus", str(a.gpus), "--test", a.test, "--child", str(r)], env=e))
    rc = 0
    for p in procs:
        try:
            rc |= p.wait(timeout=a.timeout)
        except subprocess.TimeoutExpired:
            rc |= 124
            for q in procs:              # exactly the children started above
                if q.poll() is None:
                    q.kill()
    return rc


if __name__ == "__main__":
    sys.exit(main())
