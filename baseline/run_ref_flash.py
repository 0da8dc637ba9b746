"""Launcher for the reference's own NVIDIA library (baseline/_ref/nv_build/libflash.so, built from
the unmodified sources by baseline/build_ref_nvshmem.sh) on one box: one process per GPU, each GPU
a "server" of its own, because the reference's scheduler does nothing for a single server
(nvidia/alltoall_nvshmem.cpp:549-561) and its class binds rank r to device ``r % dev_n``
(:411), so every process is given a device list that starts with its own GPU (the others stay
visible behind it, so that peer mappings between processes remain possible).

    python baseline/run_ref_flash.py --gpus 2 [--test flash|basic]

The parent starts N children; each child joins a gloo process group for the NVSHMEM unique id (as
nvidia/flash_tester.py:11-22 does), constructs ``flash_comm_t(rank, 1, world, uid)`` and calls
``test_flash_alltoall()`` or ``test_basic_alltoall()`` - the reference's stock path on its own
self-generated workload (``rand() % 2**23`` units of 8 bytes per pair, 50 warm-up and 50 timed
iterations). Rank 0 of the reference prints "algbw ... GBps / total time ... ms"; ``parse`` reads
those lines. The reference's device waits are unbounded, so every child runs under a timeout and
NVLS is switched off in NVSHMEM and NCCL. ``bench.py --impl reference`` uses ``spawn_rank`` and
``parse`` from here, one call per rank that its launcher started.
"""
import argparse
import os
import re
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
    sys.stdout.flush()
    dist.barrier()
    dist.destroy_process_group()
    return 0


def rank_env(rank: int, world: int, port: int, base_env=None) -> dict:
    """Environment of one rank's child: its own GPU first in the device list, NVLS off, no remote transport."""
    env = dict(base_env if base_env is not None else os.environ)
    visible = [d for d in env.get("CUDA_VISIBLE_DEVICES", "").split(",") if d] or [str(g) for g in range(world)]
    mine = visible[rank % len(visible)]
    order = [mine] + [d for d in visible if d != mine]
    env.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK="0",
               CUDA_VISIBLE_DEVICES=",".join(order), NCCL_NVLS_ENABLE="0", NVSHMEM_DISABLE_NVLS="1", NVSHMEM_BOOTSTRAP="UID",
               NVSHMEM_IB_ENABLE_IBGDA="0", NVSHMEM_REMOTE_TRANSPORT="none", NVSHMEM_SYMMETRIC_SIZE="8G")
    for k in ("TORCHELASTIC_RUN_ID", "GROUP_RANK", "ROLE_RANK", "LOCAL_WORLD_SIZE", "TORCHELASTIC_USE_AGENT_STORE"):
        env.pop(k, None)
    return env


def spawn_rank(rank: int, world: int, test: str, port: int, timeout: float):
    """Run one rank of the reference's tester as a child process. Returns (rc, output); rc 124 = stopped at the timeout."""
    p = subprocess.Popen([sys.executable, os.path.abspath(__file__), "--gpus", str(world), "--test", test, "--child", str(rank)],
                         env=rank_env(rank, world, port), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        out, _ = p.communicate(timeout=timeout)
        return p.returncode, out
    except subprocess.TimeoutExpired:
        p.kill()                                                # exactly the child started above
        out, _ = p.communicate()
        return 124, out


def parse(output: str) -> dict:
    """The reference's own result lines -> {"algbw_GBps", "time_ms", "per_gpu_MB", "verified"} (missing keys are absent)."""
    res = {}
    m = re.search(r"(flash|fanout) algbw: ([0-9.eE+-]+) GBps", output)
    if m:
        res["algbw_GBps"] = float(m.group(2))
    m = re.search(r"total time: ([0-9.eE+-]+) ms", output)
    if m:
        res["time_ms"] = float(m.group(1))
    m = re.search(r"per-GPU size:([0-9.eE+-]+) MB", output)
    if m:
        res["per_gpu_MB"] = float(m.group(1))
    checks = re.findall(r"verifying out buffer - correct: (\d)", output)
    if checks:
        res["verified"] = all(c == "1" for c in checks)
    return res


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
    from concurrent.futures import ThreadPoolExecutor

    port = int(os.environ.get("MASTER_PORT", "29741"))
    with ThreadPoolExecutor(max_workers=a.gpus) as ex:
        results = list(ex.map(lambda r: spawn_rank(r, a.gpus, a.test, port, a.timeout), range(a.gpus)))
    rc = 0
    for r, (code, out) in enumerate(results):
        rc |= code
        print(f"---- rank {r} rc={code}\n{out}")
    print("PARSED", parse("".join(o for _, o in results)))
    return rc


if __name__ == "__main__":
    sys.exit(main())
