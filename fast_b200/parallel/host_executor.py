"""CPU model of the device executor: one thread per rank runs the lowered work list of a plan over
host byte buffers, with the same counters, waits and give-up behaviour as the a2a_push kernel.

It is the oracle for multi-rank logic that cannot run on a single GPU (ranks wait on one another)
and the target of host-side fault injection: a rank that never enters, a signal that is withheld,
a mismatched plan. Waits are bounded and report where they gave up, like the device status block.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np

from .. import sched

SITE_ENTRY, SITE_BALANCE, SITE_RAIL, SITE_OUTPUT = 1, 2, 3, 4


class HostTimeout(RuntimeError):
    def __init__(self, rank, site, detail, seen, want):
        self.rank, self.site, self.detail, self.seen, self.want = rank, site, detail, seen, want
        super().__init__(f"rank {rank}: wait gave up at site {site} (detail {detail}): saw {seen}, wanted {want}")


@dataclass
class _RankState:
    ready: np.ndarray            # epoch published by each peer
    counters: Dict[int, int] = field(default_factory=dict)  # 0 balance, 1 output, 2+k rail stage k
    cv: threading.Condition = field(default_factory=threading.Condition)
    buffers: Dict[int, np.ndarray] = field(default_factory=dict)


class HostExecutor:
    """Runs ``plan`` for all ranks. ``faults`` may contain ``{"absent_rank": r}`` (rank r never
    enters the collective) or ``{"drop_signal": (src_rank, item_index)}`` (the copy happens but its
    arrival is never counted)."""

    def __init__(self, plan: "sched.Plan", unit_bytes: int = 1, chunk_bytes: int = 4096, timeout_s: float = 1.0, faults: Optional[dict] = None,
                 rail_segment_bytes: int = 0):
        self.plan, self.unit_bytes, self.timeout_s = plan, unit_bytes, timeout_s
        self.n = plan.matrix.shape[0]
        self.programs = [plan.lower(r, unit_bytes, chunk_bytes, rail_segment_bytes) for r in range(self.n)]
        self.faults = faults or {}
        self.errors: List[Optional[HostTimeout]] = [None] * self.n

    def _wait(self, st: _RankState, read, want, rank, site, detail):
        deadline = time.monotonic() + self.timeout_s
        with st.cv:
            while read() < want:
                left = deadline - time.monotonic()
                if left <= 0 or self._abort.is_set():
                    raise HostTimeout(rank, site, detail, read(), want)
                st.cv.wait(min(left, 0.05))

    def _run_rank(self, r: int, epoch: int):
        prog, me = self.programs[r], self.states[r]
        try:
            for p in range(self.n):  # publish readiness to every peer
                with self.states[p].cv:
                    self.states[p].ready[r] = epoch
                    self.states[p].cv.notify_all()
            for idx, it in enumerate(prog["items"]):
                src_off, dst_off, nbytes, dst, src_buf, dst_buf, wait_kind, signal_kind, stage, wait_stage = (int(x) for x in it)
                self._wait(me, lambda: me.ready[dst], epoch, r, SITE_ENTRY, dst)
                if wait_kind == 1:
                    self._wait(me, lambda: me.counters.get(0, 0), int(prog["expect_balance_bytes"]), r, SITE_BALANCE, idx)
                elif wait_kind == 2:
                    self._wait(me, lambda: me.counters.get(2 + wait_stage, 0), int(prog["expect_rail_bytes"][wait_stage]), r, SITE_RAIL, wait_stage)
                peer = self.states[dst]
                peer.buffers[dst_buf][dst_off:dst_off + nbytes] = me.buffers[src_buf][src_off:src_off + nbytes]
                if self.faults.get("drop_signal") == (r, idx):
                    continue
                slot = 0 if signal_kind == 1 else (2 + stage if signal_kind == 2 else 1)
                with peer.cv:
                    peer.counters[slot] = peer.counters.get(slot, 0) + nbytes
                    peer.cv.notify_all()
            self._wait(me, lambda: me.counters.get(1, 0), int(prog["expect_output_bytes"]), r, SITE_OUTPUT, 0)
        except HostTimeout as e:
            self.errors[r] = e
            self._abort.set()

    def run(self, inputs: Sequence[np.ndarray], epoch: int = 1) -> List[np.ndarray]:
        """Returns the output byte arrays; raises the first ``HostTimeout`` if any rank gave up."""
        self._abort = threading.Event()
        self.errors = [None] * self.n
        self.states = []
        for r in range(self.n):
            g = self.programs[r]
            st = _RankState(ready=np.zeros(self.n, dtype=np.int64))
            st.buffers = {sched.BUF_INPUT: np.frombuffer(np.ascontiguousarray(inputs[r]).tobytes(), dtype=np.uint8).copy(),
                          sched.BUF_OUTPUT: np.zeros(int(g["output_bytes"]), dtype=np.uint8),
                          sched.BUF_BALANCE: np.zeros(int(g["balance_bytes"]), dtype=np.uint8),
                          sched.BUF_RAIL: np.zeros(int(g["rail_bytes"]), dtype=np.uint8)}
            self.states.append(st)
        threads = [threading.Thread(target=self._run_rank, args=(r, epoch)) for r in range(self.n) if r != self.faults.get("absent_rank")]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        for e in self.errors:
            if e is not None:
                raise e
        return [st.buffers[sched.BUF_OUTPUT] for st in self.states]


def check_same_plan_inputs(matrix, group=None) -> None:
    """Collective: raises if the ranks of ``group`` do not hold the same traffic matrix (compares
    64-bit hashes with an all-gather). Every rank must plan the same collective or the byte
    counters can never match."""
    import torch
    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    h = sched.matrix_hash(np.ascontiguousarray(matrix, dtype=np.int64))
    mine = torch.tensor([h & 0x7FFFFFFFFFFFFFFF], dtype=torch.int64)
    dev = torch.device("cuda") if dist.get_backend(group) == "nccl" else torch.device("cpu")
    allh = [torch.zeros(1, dtype=torch.int64, device=dev) for _ in range(dist.get_world_size(group))]
    dist.all_gather(allh, mine.to(dev), group=group)
    vals = [int(t.item()) for t in allh]
    if len(set(vals)) != 1:
        raise RuntimeError(f"ranks disagree on the traffic matrix (hashes {vals}); the collective would never complete")
