"""Plan executor over ``torch.distributed`` point-to-point operations (gloo on CPU, NCCL on GPU).

It runs the same plans as the device executor, phase by phase, with one batch of isend/irecv per
phase: [balance] -> [stage 0 rails + intra-server traffic] -> [stage k rails + redistribution of
stage k-1] ... -> [last redistribution]. This is how the reference's RCCL/NCCL executor works
(amd/flash.cpp:71-273: one ncclGroup per phase, host synchronisation between phases); here it is
the portable fallback, the baseline arm "FAST over library send/recv", and the multi-process
executor that runs on CPU-only machines.
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np
import torch
import torch.distributed as dist

from .. import sched


class P2PExecutor:
    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def _slots(self, plan) -> List[np.ndarray]:
        """Ops grouped by execution slot, each slot keeping the plan's global op order."""
        ops = plan.ops
        K = plan.num_stages
        slot = np.zeros(len(ops), dtype=np.int64)
        phase, stage = ops[:, 0], ops[:, 1]
        slot[phase == sched.PHASE_BALANCE] = 0
        m = phase == sched.PHASE_INTRINSIC
        slot[m] = np.where(stage[m] < 0, 1, 1 + stage[m])
        m = phase == sched.PHASE_RAIL
        slot[m] = 1 + stage[m]
        m = phase == sched.PHASE_REDISTRIBUTE
        slot[m] = 2 + stage[m]
        return [np.nonzero(slot == s)[0] for s in range(K + 3)]

    def prepare(self, plan, unit_bytes: int, input: torch.Tensor, output: torch.Tensor) -> "PreparedP2P":
        """Resolves the plan against this rank's buffers once: per phase, the local copies and the
        send / receive descriptors. ``PreparedP2P.run()`` then only issues them, so that a timed
        loop measures the transport and not this bookkeeping (the reference lowers its schedule
        ahead of the run as well, nvidia/src/fast_alltoall/alltoall_global_scheduler.cc:1512-1821)."""
        if plan.matrix.shape[0] != self.world:
            raise ValueError("plan was built for a different world size")
        me, ub = self.rank, unit_bytes
        b = plan.buffers[me]
        dev = input.device
        bufs: Dict[int, torch.Tensor] = {
            sched.BUF_INPUT: input.view(torch.uint8).reshape(-1),
            sched.BUF_OUTPUT: output.view(torch.uint8).reshape(-1),
            sched.BUF_BALANCE: torch.empty(int(b[2]) * ub, dtype=torch.uint8, device=dev),
            sched.BUF_RAIL: torch.empty(int(b[3]) * ub, dtype=torch.uint8, device=dev),
        }
        if bufs[sched.BUF_INPUT].numel() < int(b[0]) * ub or bufs[sched.BUF_OUTPUT].numel() < int(b[1]) * ub:
            raise ValueError("buffer smaller than the plan needs")
        ops = plan.ops
        phases = []
        for idxs in self._slots(plan):
            copies, batch = [], []
            for k in idxs:
                _, _, src, dst, sbuf, dbuf, soff, doff, ln, _, _, _ = (int(v) for v in ops[k])
                if src == me and dst == me:
                    copies.append((bufs[dbuf][doff * ub:(doff + ln) * ub], bufs[sbuf][soff * ub:(soff + ln) * ub]))
                elif src == me:
                    batch.append(dist.P2POp(dist.isend, bufs[sbuf][soff * ub:(soff + ln) * ub], dst, self.group))
                elif dst == me:
                    batch.append(dist.P2POp(dist.irecv, bufs[dbuf][doff * ub:(doff + ln) * ub], src, self.group))
            if copies or batch:
                phases.append((copies, batch))
        return PreparedP2P(phases, output)

    def run(self, plan, unit_bytes: int, input: torch.Tensor, output: torch.Tensor) -> torch.Tensor:
        """``input`` / ``output``: flat uint8 tensors holding this rank's send / receive segments."""
        return self.prepare(plan, unit_bytes, input, output).run()


class PreparedP2P:
    """A plan bound to buffers: ``run()`` issues one batch of sends / receives per phase, waiting
    for each phase before the next (its forwards read what the phase delivered)."""

    def __init__(self, phases, output: torch.Tensor):
        self.phases, self.output = phases, output

    def run(self) -> torch.Tensor:
        for copies, batch in self.phases:
            for dst, src in copies:
                dst.copy_(src)
            if batch:
                for w in dist.batch_isend_irecv(batch):
                    w.wait()
        return self.output
