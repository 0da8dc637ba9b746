"""Child of test_p2p_executor_gloo: CPU ranks over gloo run hierarchical and flat plans bit-exactly."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from fast_b200 import sched  # noqa: E402
from fast_b200.parallel.host_executor import check_same_plan_inputs  # noqa: E402
from fast_b200.parallel.p2p_executor import P2PExecutor  # noqa: E402
from fast_b200.sched import PlanKind, Topology  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    ex = P2PExecutor()
    ub = 4
    topos = [Topology.flat(world)] + ([Topology(2, world // 2)] if world % 2 == 0 and world >= 4 else [])
    for topo in topos:
        for kind in (PlanKind.STAGED, PlanKind.SINGLE_BURST, PlanKind.FANOUT, PlanKind.SPREAD_OUT):
            for seed in range(2):
                m = sched.workload_zipf_rows(world, 1.0, 4000, seed, 1)
                m[0, 0] = 17  # some self traffic too
                check_same_plan_inputs(m)
                plan = sched.build_plan(m, topo, kind=kind)
                assert plan.validate() == ""
                rng = np.random.default_rng(1000 + seed)
                ins = [rng.integers(0, 256, int(plan.buffers[r, 0]) * ub, dtype=np.uint8) for r in range(world)]
                want = [np.zeros(int(plan.buffers[r, 1]) * ub, dtype=np.uint8) for r in range(world)]
                plan.execute_on_host(ub, ins, want)
                out = torch.zeros(int(plan.buffers[rank, 1]) * ub, dtype=torch.uint8)
                prepared = ex.prepare(plan, ub, torch.from_numpy(ins[rank]), out)
                for _ in range(2):  # a prepared plan can be issued again (descriptors are bound to the buffers)
                    out.zero_()
                    prepared.run()
                    assert np.array_equal(out.numpy(), want[rank]), f"rank {rank} {kind} {topo}"
                # transposed plan = the reverse collective
                back = sched.build_plan(m, topo, kind=kind, transpose=True)
                ret = torch.zeros(int(back.buffers[rank, 1]) * ub, dtype=torch.uint8)
                ex.run(back, ub, out, ret)
                assert np.array_equal(ret.numpy(), ins[rank]), f"round trip rank {rank} {kind}"
    dist.barrier()
    if rank == 0:
        print("P2P_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
