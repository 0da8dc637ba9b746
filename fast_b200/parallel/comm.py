"""Communicator: symmetric memory, traffic-matrix scheduling and the all-to-all(v) entry points.

API parity with the reference's framework-facing class (amd/flash.cpp:337-648): construct from
(rank, world, topology); ``schedule(matrix, transpose)``; ``buffer_sizes()``; caller-owned or
library-owned staging; ``all_to_all_v`` / ``all_to_all_single``; element-unit matrices with an
element size; bf16 / fp8 payloads are just bytes here. The NVIDIA class of the reference only
exposes self-tests (nvidia/alltoall_nvshmem.cpp:508-601); this one is a general collective.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import runtime, sched
from ..sched import PlanKind, Topology
from ..utils.config import CONFIG


MAX_RAIL_COUNTERS = 4096  # rail arrival counters in the device signal block (kSigMaxStages)
# Above this many ranks a communicator plans one-rank views instead of full plans. It equals the
# number of peers the device signal block has room for (kSigMaxWorld in csrc/kernels/api.h): planning
# (and the host executors) scale past it, a launch on more ranks than that is refused by a2a_launch.
VIEW_WORLD = 64


@dataclass
class Schedule:
    """A plan lowered for one rank, with its device-resident work list."""

    plan: "sched.Plan"
    unit_bytes: int
    program: object  # _C.A2AProgram
    lowered: dict
    rank: int

    @property
    def input_bytes(self) -> int:
        return int(self.lowered["input_bytes"])

    @property
    def output_bytes(self) -> int:
        return int(self.lowered["output_bytes"])

    @property
    def balance_bytes(self) -> int:
        return int(self.lowered["balance_bytes"])

    @property
    def rail_bytes(self) -> int:
        return int(self.lowered["rail_bytes"])

    @property
    def max_bytes(self) -> dict:
        """Largest need of any rank per buffer: symmetric staging is sized by these so that every
        rank allocates the same amounts in the same order.

        Staging is never reused inside one collective: every stage of a two-tier plan lands in a rail
        region of its own, so ``rail`` grows with the bytes a rank relays (about twice its payload for
        a 1 GiB-per-rank two-tier exchange, zero for single-server plans) and ``balance`` with the
        bytes it takes over from busier neighbours. That trades memory (180 GB per GPU) for the
        absence of buffer credits and their waits; a caller short of memory can split the exchange
        into several ``all_to_all_v`` calls over slices of the matrix, which reuse the same staging."""
        mb = self.__dict__.get("_max_bytes")
        if mb is None:  # computed once: this sits on the launch path of every collective
            b = self.plan.buffers.max(axis=0) * self.unit_bytes
            mb = self.__dict__["_max_bytes"] = {"input": int(b[0]), "output": int(b[1]), "balance": int(b[2]), "rail": int(b[3])}
        return mb

    def buffer_sizes(self) -> dict:
        """Bytes of each buffer this rank needs (the reference's get_buffer_szs, amd/flash.cpp:385-397)."""
        return {"input": self.input_bytes, "output": self.output_bytes, "balance": self.balance_bytes, "rail": self.rail_bytes}


class Communicator:
    """One rank of an all-to-all domain. Use ``Communicator(group)`` with one process per GPU, or
    ``LocalGroup`` for several virtual ranks on a single GPU (tests, single-GPU runs). With ``store``
    (any ``torch.distributed`` store shared by the ranks) the IPC handles are exchanged through it
    with a deadline of ``bootstrap_timeout_s``; every rank must then construct its communicators
    in the same order."""

    _bootstraps = 0  # generation counter of store-based bootstraps in this process

    def __init__(self, group=None, heap_bytes: int = 1 << 30, topo: Optional[Topology] = None, device=None,
                 timeout_s: Optional[float] = None, ctas: Optional[int] = None, threads: int = 512, store=None,
                 bootstrap_timeout_s: float = 60.0, _heap=None, _rank=None, _world=None):
        import torch.distributed as dist

        self._C = runtime.ext()
        self._virtual = _heap is not None  # one of several ranks of a LocalGroup inside this process
        if _heap is not None:
            self.rank, self.world, self.heap = _rank, _world, _heap
            self.device = torch.device("cuda", device if device is not None else torch.cuda.current_device())
            self.group = None
        else:
            self.group = group
            self.rank = dist.get_rank(group) if dist.is_initialized() else 0
            self.world = dist.get_world_size(group) if dist.is_initialized() else 1
            self.device = torch.device("cuda", device if device is not None else torch.cuda.current_device())
            self.heap = self._C.SymmHeap(self.rank, self.world, int(heap_bytes), self.device.index)
            if self.world > 1:
                if store is not None:
                    # Exchange through a key-value store with a deadline: a rank that never shows up is
                    # named in the error instead of blocking everyone in a collective.
                    from .liveness import bounded_exchange

                    Communicator._bootstraps += 1
                    handles = bounded_exchange(store, self.rank, self.world, f"fastb/ipc/{Communicator._bootstraps}", self.heap.ipc_handle(),
                                               timeout_s=bootstrap_timeout_s)
                else:
                    handles: List[Optional[bytes]] = [None] * self.world
                    dist.all_gather_object(handles, self.heap.ipc_handle(), group=group)
                self.heap.open_peers(handles)
                dist.barrier(group=group)
        self.topo = topo or Topology.flat(self.world)
        if self.topo.ranks != self.world:
            raise ValueError("topology does not match the world size")
        self.timeout_ns = int((CONFIG.timeout_s if timeout_s is None else timeout_s) * 1e9)
        # one CTA per SM: the collective runs alone on its stream (measured best at 8 GPUs)
        self.ctas = ctas or torch.cuda.get_device_properties(self.device).multi_processor_count
        self.threads = threads
        self.status = self._C.StatusBlock()
        self.sig_off = self.heap.alloc(self._C.SIG_WORDS * 8)
        self.epoch = 0
        self.broken = False
        self.plan_cache = sched.PlanCache()
        self._staging = {}  # name -> (offset, bytes)
        self._sched_cache = {}
        # Optional liveness.Heartbeat: consulted before every launch so that a lost peer raises
        # PeerLost on the host instead of making a kernel wait for its timeout.
        self.liveness = None
        self.liveness_max_age_s = 2.0
        # True: 16-byte aligned pieces are moved by the bulk-copy engine (one thread per CTA, shared-memory ring)
        # instead of by load/store loops of every thread.
        self.bulk_copy = bool(CONFIG.a2a_bulk)

    # ---- symmetric memory ---------------------------------------------------------------------
    def alloc(self, shape, dtype=torch.uint8, verify: Optional[bool] = None) -> torch.Tensor:
        """A tensor inside the symmetric heap. Every rank must make the same allocations (sizes and
        order): an offset then names the same buffer on every rank, which is what peers rely on when
        they write into it. Size receive buffers by ``Schedule.max_bytes``, not by a rank's own need.
        ``verify=True`` (default: the FASTB_CHECK_SYMM=1 switch) compares offset and size across the
        ranks with one small host collective and raises on a mismatch."""
        shape = (shape,) if isinstance(shape, int) else tuple(shape)
        nbytes = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        off = self.heap.alloc(max(nbytes, 1))
        if (CONFIG.check_symm if verify is None else verify) and self.world > 1 and not self._virtual:
            import torch.distributed as dist

            if dist.is_initialized():
                seen: List[Optional[tuple]] = [None] * self.world
                dist.all_gather_object(seen, (int(off), int(nbytes)), group=self.group)
                if any(x != seen[0] for x in seen):
                    raise RuntimeError(f"symmetric allocation differs across ranks (offset, bytes per rank): {seen}")
        t = self.heap.tensor(off, list(shape), dtype)
        t._symm_off = off
        return t

    def free(self, t: torch.Tensor) -> None:
        self.heap.free(t._symm_off)

    def offset_of(self, t: torch.Tensor) -> Optional[int]:
        base = self.heap.base_ptr(self.rank)
        p = t.data_ptr()
        return p - base if base <= p and p + t.numel() * t.element_size() <= base + self.heap.bytes else None

    def _stage(self, name: str, nbytes: int) -> int:
        cur = self._staging.get(name)
        if cur is None or cur[1] < nbytes:
            if cur is not None:
                self.heap.free(cur[0])
            grown = max(nbytes, 256)
            self._staging[name] = (self.heap.alloc(grown), grown)
        return self._staging[name][0]

    # ---- scheduling -----------------------------------------------------------------------------
    def schedule(self, matrix, unit_bytes: int = 1, transpose: bool = False, kind=PlanKind.STAGED, chunk_bytes: Optional[int] = None,
                 verify: bool = False, rail_segment_bytes: int = 0, **plan_opts) -> Schedule:
        """Plan the collective for ``matrix`` (units; ``matrix[i, j]`` = rank i -> rank j).

        Every rank must pass the same matrix. Staged plans are built with pieces cut on 16-byte
        boundaries whenever the unit size allows it. ``verify=True`` first compares the matrix hash
        across the ranks (one small all-gather) and raises if they differ - ranks that plan different
        collectives would wait for bytes that never come. ``kind="auto"`` lets the cost model choose
        between the fan-out and the staged plan (and the single-burst plan on a two-tier topology)
        for this matrix and unit size, under the link model fitted to this fabric.
        ``rail_segment_bytes > 0`` (two-tier plans) gives every such piece of a stage's rail staging its
        own arrival counter, so that redistribution starts piece by piece instead of stage by stage.
        """
        m = np.ascontiguousarray(matrix, dtype=np.int64)
        if verify and self.world > 1:
            from .host_executor import check_same_plan_inputs

            check_same_plan_inputs(m, self.group)
        if chunk_bytes is None:
            # Work items: about 8 per CTA for the busiest rank (an uneven last round of 1 MiB items costs
            # up to half the bandwidth at 148 CTAs), between 64 KiB and 1 MiB, a power of two.
            busiest = int(max(m.sum(1).max(), m.sum(0).max())) * unit_bytes
            chunk_bytes = 1 << 16
            while chunk_bytes < (1 << 20) and chunk_bytes * 2 * self.ctas * 8 <= busiest:
                chunk_bytes *= 2
        if "split_align" not in plan_opts:
            plan_opts["split_align"] = max(1, 16 // np.gcd(16, unit_bytes))
        key = (sched.matrix_hash(m), unit_bytes, transpose, str(kind), chunk_bytes, rail_segment_bytes, tuple(sorted((k, str(v)) for k, v in plan_opts.items())))
        s = self._sched_cache.get(key)
        if s is None:
            if kind == "auto":
                plan_opts.setdefault("mb_per_unit", unit_bytes * 1e-6)
            elif self.world > VIEW_WORLD:
                # Large jobs: keep only this rank's ops (same sizes, offsets and work list); the op list
                # of a full plan grows with the cube of the server count.
                plan_opts.setdefault("only_rank", self.rank)
            plan = self.plan_cache.get(m, self.topo, kind=kind, transpose=transpose, **plan_opts)
            err = plan.validate()
            if err:
                raise RuntimeError(f"scheduler produced an invalid plan: {err}")
            low = plan.lower(self.rank, unit_bytes, chunk_bytes, rail_segment_bytes, MAX_RAIL_COUNTERS)
            prog = self._C.A2AProgram(torch.from_numpy(low["items"]), [int(x) for x in low["expect_rail_bytes"]],
                                      int(low["expect_output_bytes"]), int(low["expect_balance_bytes"]), self.device.index)
            s = Schedule(plan, unit_bytes, prog, low, self.rank)
            if CONFIG.log and self.rank == 0 and plan.only_rank < 0:
                nv = sched.nvlink_model(900.0, 2.0)
                c = plan.cost(nv, nv, unit_bytes * 1e-6)
                print(f"[fast_b200] scheduled {kind}: {plan.num_stages} stages, {plan.num_ops} ops, {prog.n_items} work items on rank 0, "
                      f"modeled {c['total_us']:.1f} us, port bound {c['lower_bound_us']:.1f} us", flush=True)
            if len(self._sched_cache) > 512:
                self._sched_cache.pop(next(iter(self._sched_cache)))
            self._sched_cache[key] = s
        return s

    # ---- execution --------------------------------------------------------------------------------
    def _launch_args(self, s: Schedule, output: torch.Tensor, input: torch.Tensor, staging: Optional[dict] = None):
        if self.heap is None:
            raise RuntimeError("communicator is closed")
        if self.broken:
            raise RuntimeError("communicator saw a failed collective; call reset() on every rank first")
        if self.liveness is not None:
            self.liveness.require_alive(self.liveness_max_age_s)
        if input.numel() * input.element_size() < s.input_bytes:
            raise ValueError("input smaller than the schedule needs")
        if output.numel() * output.element_size() < s.output_bytes:
            raise ValueError("output smaller than the schedule needs")
        out_off = self.offset_of(output)
        copy_back = None
        if out_off is None:  # library-owned receive staging, copied out afterwards
            out_off = self._stage("recv", s.max_bytes["output"])
            copy_back = self.heap.tensor(out_off, [s.output_bytes], torch.uint8)
        def staged(name):
            t = (staging or {}).get(name)
            if t is None:
                return self._stage(name, s.max_bytes[name])
            off = self.offset_of(t)
            if off is None or t.numel() * t.element_size() < s.max_bytes[name]:
                raise ValueError(f"caller-owned {name} staging must be a symmetric-heap tensor of at least {s.max_bytes[name]} bytes")
            return off

        bal_off, rail_off = staged("balance"), staged("rail")
        base = self.heap.base_ptr(self.rank)
        src = [input.data_ptr(), 0, base + bal_off, base + rail_off]
        dst = [0, out_off, bal_off, rail_off]
        return src, dst, copy_back

    def init_buffers(self, s: Schedule):
        """Library-owned buffers for a schedule: ``(send, recv)`` byte tensors, ``recv`` in the
        symmetric heap (peers write it directly). Every rank must call this for the same schedule
        (the reference's init_buffers / free_buffers pair, amd/flash.cpp:447-519)."""
        send = torch.empty(max(s.max_bytes["input"], 1), dtype=torch.uint8, device=self.device)
        recv = self.alloc(max(s.max_bytes["output"], 1), torch.uint8)
        return send, recv

    def free_buffers(self, recv: torch.Tensor) -> None:
        self.free(recv)

    def new_phase_stamps(self) -> torch.Tensor:
        """A device buffer for ``all_to_all_v(..., phase_stamps=...)``, cleared for one collective."""
        t = torch.zeros(self._C.PHASE_STAMP_WORDS, dtype=torch.int64, device=self.device)
        return self.clear_phase_stamps(t)

    @staticmethod
    def clear_phase_stamps(t: torch.Tensor) -> torch.Tensor:
        t.zero_()
        t[[0, 1, 3, 5, 7]] = -1          # start slots hold a minimum: all ones as unsigned
        return t

    @staticmethod
    def read_phase_stamps(t: torch.Tensor) -> dict:
        """Stamps of one collective as microseconds since this rank's kernel start, per phase
        ``(first start, last end)``; phases the plan does not have are absent. The reference records
        the same breakdown with four event stamps per iteration (load balance / cross node /
        restore, amd/test_alltoall.cpp:903-1106, reported at :1432-1438)."""
        v = [int(x) for x in t.cpu().tolist()]
        t0 = v[0]
        out = {}
        for p, name in enumerate(("balance", "rail", "redistribute", "direct")):
            start, end = v[1 + 2 * p], v[2 + 2 * p]
            if start != -1 and end != 0:
                out[name] = ((start - t0) / 1e3, (end - t0) / 1e3)
        out["total"] = (0.0, (v[9] - t0) / 1e3)
        return out

    def all_to_all_v(self, output: torch.Tensor, input: torch.Tensor, s: Schedule, staging: Optional[dict] = None,
                     phase_stamps: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run a scheduled all-to-all(v) on the current stream. ``input`` holds the segments for
        rank 0..n-1 back to back; ``output`` receives the segments from rank 0..n-1 back to back.
        ``output`` in the symmetric heap (``alloc``) is written in place by the peers; any other
        tensor goes through a library-owned receive buffer and one extra local copy. ``staging``
        may name caller-owned symmetric tensors for the two-tier plans' ``"balance"`` and ``"rail"``
        areas (sizes from ``Schedule.max_bytes``; same allocation order on every rank), as the
        reference's all_to_all_2 takes them (amd/flash.cpp:570-629); by default the library keeps its own.
        ``phase_stamps`` (``new_phase_stamps()``) makes the kernel record when each phase of the plan
        (balance, rail, redistribute, direct) started and ended on this rank; read them with
        ``read_phase_stamps`` after the stream is idle."""
        src, dst, copy_back = self._launch_args(s, output, input, staging)
        self.epoch += 1
        ctas = max(1, min(self.ctas, s.program.n_items))  # a handful of work items needs a handful of CTAs
        self._C.a2a_launch(s.program, self.heap, src, dst, self.sig_off, self.epoch, self.status, self.timeout_ns, ctas, self.threads,
                           0 if phase_stamps is None else phase_stamps.data_ptr(), self.bulk_copy and not self._virtual)
        if copy_back is not None:
            output.view(torch.uint8).reshape(-1)[: s.output_bytes].copy_(copy_back[: s.output_bytes])
        return output

    def all_to_all_single(self, output: torch.Tensor, input: torch.Tensor, output_split_sizes: Optional[Sequence[int]] = None,
                          input_split_sizes: Optional[Sequence[int]] = None, matrix=None, kind=PlanKind.FANOUT) -> torch.Tensor:
        """``torch.distributed.all_to_all_single`` semantics (splits count rows of dim 0)."""
        import torch.distributed as dist

        row_bytes = input.element_size() * int(np.prod(input.shape[1:])) if input.dim() > 1 else input.element_size()
        if matrix is None:
            if input_split_sizes is None:
                per = input.shape[0] // self.world
                matrix = np.full((self.world, self.world), per, dtype=np.int64)
            else:
                mine = torch.tensor(list(input_split_sizes), dtype=torch.int64)
                rows = [torch.empty_like(mine) for _ in range(self.world)]
                if self.world > 1:
                    backend_dev = self.device if dist.get_backend(self.group) == "nccl" else torch.device("cpu")
                    g = [r.to(backend_dev) for r in rows]
                    dist.all_gather(g, mine.to(backend_dev), group=self.group)
                    rows = [r.cpu() for r in g]
                else:
                    rows = [mine]
                matrix = torch.stack(rows).numpy()
        s = self.schedule(matrix, unit_bytes=row_bytes, kind=kind)
        return self.all_to_all_v(output, input, s)

    # ---- health -------------------------------------------------------------------------------------
    def check(self) -> None:
        """Synchronise the stream and raise ``CollectiveTimeout`` if a device wait gave up."""
        code, site, detail, seen, want = self.status.read()
        if code != 0:
            self.broken = True
            raise runtime.CollectiveTimeout(code, site, detail, seen, want)

    def reset(self) -> None:
        """After a failed collective: clear status and signal words (collective over the group)."""
        import torch.distributed as dist

        torch.cuda.synchronize(self.device)
        if self.group is not None or (dist.is_initialized() and self.world > 1):
            dist.barrier(group=self.group)
        self.heap.tensor(self.sig_off, [self._C.SIG_WORDS], torch.int64).zero_()
        self.status.clear()
        self.epoch = 0
        torch.cuda.synchronize(self.device)
        if self.group is not None or (dist.is_initialized() and self.world > 1):
            dist.barrier(group=self.group)
        self.broken = False

    def close(self) -> None:
        """Collective: every rank calls it after its last collective. Teardown has two phases, because
        freeing a slab that a peer still has mapped is undefined in CUDA: (1) synchronise the device,
        meet the peers (nobody unmaps memory a peer may still write), unmap every peer's slab;
        (2) meet again, then let go of the local heap - its slab is freed once the last tensor
        carved from it is gone, which by then no peer can see. Stops an attached heartbeat. The
        communicator is unusable afterwards."""
        import torch.distributed as dist

        if self.heap is None:
            return
        multi = self.group is not None or (dist.is_initialized() and self.world > 1 and not self._virtual)
        torch.cuda.synchronize(self.device)
        if multi:
            dist.barrier(group=self.group)
        if not self._virtual:
            self.heap.close_peers()
        if multi:
            dist.barrier(group=self.group)
        if self.liveness is not None:
            self.liveness.leave()
            self.liveness = None
        self._staging.clear()
        self._sched_cache.clear()
        self.heap = None
        self.broken = True  # any further launch is refused

    def __enter__(self) -> "Communicator":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


class LocalGroup:
    """``world`` virtual ranks on one GPU, executed by ONE cooperative launch per collective.

    Kernels of different ranks wait on one another, so they may never run as separate launches on
    one device; the group launch puts every rank's CTAs in the same grid. Used by the single-GPU
    tests and by single-GPU runs of multi-rank plans.
    """

    def __init__(self, world: int, heap_bytes: int = 256 << 20, topo: Optional[Topology] = None, device: int = 0,
                 timeout_s: float = 5.0, ctas: int = 8, threads: int = 256):
        C = runtime.ext()
        self._C = C
        heaps = C.SymmHeap.create_local_group(world, int(heap_bytes), device)
        self.comms = [Communicator(heap_bytes=heap_bytes, topo=topo, device=device, timeout_s=timeout_s, ctas=ctas, threads=threads,
                                   _heap=h, _rank=r, _world=world) for r, h in enumerate(heaps)]
        self.world, self.ctas, self.threads = world, ctas, threads

    def schedule(self, matrix, **kw) -> List[Schedule]:
        return [c.schedule(matrix, **kw) for c in self.comms]

    def all_to_all_v(self, outputs, inputs, scheds) -> None:
        srcs, cbs = [], []
        dst0 = None
        for c, o, i, s in zip(self.comms, outputs, inputs, scheds):
            src, dst, cb = c._launch_args(s, o, i)
            if dst0 is None:
                dst0 = dst
            elif dst != dst0:
                raise RuntimeError("virtual ranks disagree on symmetric offsets; allocate in the same order on every rank")
            srcs.append(src)
            cbs.append(cb)
        c0 = self.comms[0]
        for c in self.comms:
            c.epoch += 1
        self._C.a2a_launch_group([s.program for s in scheds], [c.heap for c in self.comms], srcs, dst0, c0.sig_off, c0.epoch,
                                 [c.status for c in self.comms], c0.timeout_ns, self.ctas, self.threads)
        for o, cb, s in zip(outputs, cbs, scheds):
            if cb is not None:
                o.view(torch.uint8).reshape(-1)[: s.output_bytes].copy_(cb[: s.output_bytes])

    def check(self) -> None:
        for c in self.comms:
            c.check()
