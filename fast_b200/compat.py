"""Drop-in shape of the reference's framework-facing class for code written against it.

The reference's pybind module exposes ``flash_t(this_rank, total_rank, server_n, gpu_n, hidden_sz,
dtype_code, nccl_unique_id)`` with ``schedule(workload_tokens, backward)``, ``get_buffer_szs()``,
``init_buffers / free_buffers / all_to_all``, ``all_to_all_2`` (caller-owned staging),
``all_to_all_v`` (plain fan-out baseline) and a few getters (amd/flash.cpp:337-666; dtype codes
amd/flash.cpp:318-334). :class:`FlashAllToAll` offers the same calls on top of
:class:`fast_b200.parallel.Communicator`, so a training framework that called the reference can
switch by changing the import. What differs, by design:

* no NCCL unique id is needed (the argument is accepted and ignored): ranks meet through the
  default ``torch.distributed`` group and exchange CUDA IPC handles of the symmetric heap;
* the traffic matrix is in tokens, as in the reference; bytes = tokens x hidden_sz x dtype size;
* ``get_buffer_szs()`` keeps the reference's six slots ``[send, lbsend, lbrecv, cros, cros, rstr]``
  in tokens, but this runtime sends balance traffic straight from the input and lands
  redistributed data straight in the output, so ``lbsend`` and ``rstr`` are 0, ``lbrecv`` is the
  balance staging and the first ``cros`` is the rail staging of all stages (the second is 0: there
  is no ping-pong pair because staging is never reused inside a collective);
* ``all_to_all_2`` uses ``lbrecv`` and ``cros1`` as staging when they are symmetric-heap tensors
  (``alloc``) that are large enough, and the library's own staging otherwise; the other staging
  arguments are accepted and left untouched.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from .sched import PlanKind, Topology

# dtype codes of the reference (amd/flash.cpp:318-334); unknown codes fall back to int8 there too.
DTYPE_CODES = {
    0: torch.int8, 1: torch.uint8, 2: torch.int32, 3: torch.uint32, 4: torch.int64, 5: torch.uint64,
    6: torch.float16, 7: torch.float32, 8: torch.float64, 9: torch.bfloat16,
    10: torch.float8_e4m3fn, 11: torch.float8_e5m2,
}


def dtype_of(code: int) -> torch.dtype:
    return DTYPE_CODES.get(int(code), torch.int8)


def code_of(dtype: torch.dtype) -> int:
    for c, d in DTYPE_CODES.items():
        if d == dtype:
            return c
    raise ValueError(f"no dtype code for {dtype}")


class FlashAllToAll:
    """The reference's ``flash_t`` on this runtime. ``comm`` may be passed in (an existing
    :class:`Communicator`, or a stand-in with the same methods); otherwise one is created on the
    current CUDA device over the default process group."""

    def __init__(self, this_rank: int, total_rank: int, server_n: int, gpu_n: int, hidden_sz: int, dtype_code: int,
                 nccl_unique_id: Optional[bytes] = None, *, comm=None, heap_bytes: int = 4 << 30, flat: bool = False):
        if server_n * gpu_n != total_rank:
            raise ValueError("server_n * gpu_n must equal total_rank")
        self.rank, self.world, self.server_n, self.gpu_n = int(this_rank), int(total_rank), int(server_n), int(gpu_n)
        self.hidden_sz, self.dtype = int(hidden_sz), dtype_of(dtype_code)
        self.token_bytes = self.hidden_sz * torch.empty((), dtype=self.dtype).element_size()
        # One NVSwitch domain has no slow tier: ``flat=True`` plans every GPU as its own server
        # (fewer hops); the default keeps the two-tier plan the caller described.
        self.topo = Topology.flat(self.world) if flat else Topology(self.server_n, self.gpu_n)
        if comm is None:
            from .parallel import Communicator

            comm = Communicator(heap_bytes=heap_bytes, topo=self.topo)
        if comm.rank != self.rank or comm.world != self.world:
            raise ValueError("communicator rank / world do not match the arguments")
        self.comm = comm
        self.sched = None
        self._input = self._output = self._recv = None

    # ---- planning -----------------------------------------------------------------------------
    def schedule(self, workload, backward: int = 0) -> None:
        """``workload``: int array of ``total_rank * total_rank`` token counts, row = sender.
        ``backward == 1`` plans the transposed matrix (combine / backward pass)."""
        m = np.asarray(workload, dtype=np.int64).reshape(self.world, self.world)
        self.sched = self.comm.schedule(m, unit_bytes=self.token_bytes, transpose=bool(backward), kind=PlanKind.STAGED)

    def _need(self):
        if self.sched is None:
            raise RuntimeError("call schedule() first")
        return self.sched

    def get_buffer_szs(self) -> np.ndarray:
        s = self._need()
        tok = lambda b: int(b // self.token_bytes)
        mb = s.max_bytes
        return np.array([tok(s.input_bytes), 0, tok(mb["balance"]), tok(mb["rail"]), 0, 0], dtype=np.int64)

    # ---- library-owned buffers ------------------------------------------------------------------
    def init_buffers(self, input: torch.Tensor, output: torch.Tensor) -> None:
        s = self._need()
        self._input, self._output = input, output
        self._recv = None if self.comm.offset_of(output) is not None else self.comm.init_buffers(s)[1]

    def free_buffers(self) -> None:
        if self._recv is not None:
            self.comm.free_buffers(self._recv)
        self._input = self._output = self._recv = None

    def all_to_all(self) -> torch.Tensor:
        s = self._need()
        if self._input is None:
            raise RuntimeError("call init_buffers() first")
        if self._recv is None:
            return self.comm.all_to_all_v(self._output, self._input, s)
        self.comm.all_to_all_v(self._recv, self._input, s)
        self._output.view(torch.uint8).reshape(-1)[: s.output_bytes].copy_(self._recv[: s.output_bytes])
        return self._output

    # ---- caller-owned staging -------------------------------------------------------------------
    def all_to_all_2(self, input: torch.Tensor, output: torch.Tensor, send=None, lbsend=None, lbrecv=None, cros1=None,
                     cros2=None, rstr=None) -> torch.Tensor:
        s = self._need()
        staging = {}
        for name, t in (("balance", lbrecv), ("rail", cros1)):
            if t is not None and self.comm.offset_of(t) is not None and t.numel() * t.element_size() >= s.max_bytes[name]:
                staging[name] = t
        return self.comm.all_to_all_v(output, input, s, staging=staging or None)

    # ---- plain fan-out baseline -------------------------------------------------------------------
    def all_to_all_v(self, input: torch.Tensor, output: torch.Tensor, input_splits: Sequence[int], output_splits: Sequence[int]) -> torch.Tensor:
        """Every pair at once, no staging (the reference's baseline entry point). Splits in tokens."""
        if len(input_splits) != self.world or len(output_splits) != self.world:
            raise ValueError("one split per rank")
        return self.comm.all_to_all_single(output.view(-1, self.hidden_sz), input.view(-1, self.hidden_sz), list(output_splits),
                                           list(input_splits), kind=PlanKind.FANOUT)

    # ---- getters ------------------------------------------------------------------------------------
    def get_world_size(self) -> int:
        return self.world

    def get_rank(self) -> int:
        return self.rank

    def get_server_n(self) -> int:
        return self.server_n

    def get_hidden_sz(self) -> int:
        return self.hidden_sz

    @staticmethod
    def print_tensor(t: torch.Tensor) -> None:
        print(t.detach().cpu())


def get_nvshmem_init_id() -> torch.Tensor:
    """Shape-compatible stand-in for the reference's ``torch.ops.flash_nvshmem.get_nvshmem_init_id``
    (nvidia/alltoall_nvshmem.cpp:384-388): a CPU uint8 tensor of 128 bytes that callers may
    broadcast and pass to :class:`FlashComm` as before. Its content is unused: this runtime has no
    NVSHMEM bootstrap, ranks meet through ``torch.distributed``."""
    return torch.zeros(128, dtype=torch.uint8)


def pattern_words(src: int, dst: int, count: int, device) -> torch.Tensor:
    """Verification words of one (src, dst) segment: ``src << 24 | dst << 16 | index & 0xffff``, the
    scheme of the reference's buffer checks (nvidia/src/fast_alltoall/flash_alltoall_nvshmem.cu:1445-1473)."""
    idx = torch.arange(count, device=device, dtype=torch.int32) & 0xFFFF
    return idx | ((src << 24) | (dst << 16))


def reference_uniform_workload(world: int, bound: int = 1 << 23) -> np.ndarray:
    """The matrix the reference's tester runs on: ``uniform_distribution(workload, n, 2**23)``
    (nvidia/alltoall_nvshmem.cpp:111-123, called at :510 and :565) draws ``rand() % bound`` for
    every (i, j) in row-major order from the C library's generator, which the reference never
    seeds (so it starts from seed 1), rounds each entry up to a multiple of 512 and clears the
    diagonal. Reproduced here through the same C library so that both runtimes can be timed on
    the identical workload."""
    import ctypes

    libc = ctypes.CDLL("libc.so.6")
    libc.rand.restype = ctypes.c_int
    libc.srand(1)
    m = np.zeros((world, world), dtype=np.int64)
    for i in range(world):
        for j in range(world):
            m[i, j] = ((libc.rand() % bound) + 0x1FF) & ~0x1FF
    np.fill_diagonal(m, 0)
    return m


class FlashComm:
    """The reference's NVIDIA tester class (``flash_comm_t(rank, dev_n, world_size, uid)`` with
    ``test_basic_alltoall()`` and ``test_flash_alltoall()``, nvidia/alltoall_nvshmem.cpp:390-601) on
    this runtime: rank 0 draws a uniform random workload, every rank gets it, the collective is
    timed on the device after warm-up and the output is checked word for word. ``uid`` is accepted
    and ignored (no NVSHMEM bootstrap exists here). Both tests return
    ``{"time_ms", "algbw_GBps", "per_gpu_MB", "verified"}``; rank 0 also prints them."""

    def __init__(self, rank: int, dev_n: int, world_size: int, uid=None, *, comm=None, mean_units: int = 1 << 23,
                 heap_bytes: Optional[int] = None, seed: int = 1, generator: str = "seeded", quiet: bool = False):
        self.rank, self.dev_n, self.world = int(rank), int(dev_n), int(world_size)
        self.mean_units, self.seed = int(mean_units), int(seed)
        self.quiet = quiet
        assert generator in ("seeded", "glibc")
        # "glibc": the very matrix the reference's tester draws (reference_uniform_workload with bound = mean_units,
        # 2**23 by default as in the reference); "seeded": this library's generator with mean mean_units.
        self.generator = generator
        if comm is None:
            from .parallel import Communicator

            torch.cuda.set_device(self.rank % self.dev_n)
            need = 3 * 8 * self.mean_units * self.world * 2 + (64 << 20)   # output + staging, worst column twice the mean
            comm = Communicator(heap_bytes=heap_bytes or need)
        self.comm = comm

    def _workload(self) -> np.ndarray:
        import torch.distributed as dist

        from . import sched

        if self.generator == "glibc":
            m = torch.from_numpy(reference_uniform_workload(self.world, self.mean_units))  # the reference's bound: entries in [0, mean_units)
        else:
            m = torch.from_numpy(np.ascontiguousarray(sched.workload_uniform(self.world, 2 * self.mean_units, self.seed, False)))
        if self.world > 1:
            dev = self.comm.device if dist.get_backend() == "nccl" else torch.device("cpu")
            t = m.to(dev)
            dist.broadcast(t, 0)
            m = t.cpu()
        return m.numpy()

    def _run(self, kind, data_size: int, warmup: int, iters: int, name: str) -> dict:
        m = self._workload()
        r, dev, wpu = self.rank, self.comm.device, data_size // 4
        s = self.comm.schedule(m, unit_bytes=data_size, kind=kind)
        inp = torch.cat([pattern_words(r, d, int(m[r, d]) * wpu, dev) for d in range(self.world)] + [torch.zeros(4, dtype=torch.int32, device=dev)])
        want = torch.cat([pattern_words(src, r, int(m[src, r]) * wpu, dev) for src in range(self.world)])
        out = self.comm.alloc(max(s.max_bytes["output"], 16) // 4, torch.int32)
        out.zero_()
        for _ in range(warmup):
            self.comm.all_to_all_v(out, inp, s)
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            self.comm.all_to_all_v(out, inp, s)
        e1.record()
        torch.cuda.synchronize(dev)
        self.comm.check()
        ms = torch.tensor([e0.elapsed_time(e1) / max(iters, 1)], device=dev)
        ok = torch.tensor([1 if torch.equal(out[: want.numel()], want) else 0], device=dev)
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        self.comm.free(out)
        total = int(m.sum()) * data_size
        res = {"time_ms": float(ms.item()), "algbw_GBps": total / self.world / (float(ms.item()) * 1e-3) / 1e9 if ms.item() > 0 else 0.0,
               "per_gpu_MB": total / self.world / 1e6, "verified": bool(ok.item())}
        if self.rank == 0 and not self.quiet:
            print(f"per-GPU size: {res['per_gpu_MB']:.1f} MB, {name} algbw: {res['algbw_GBps']:.1f} GBps, total time: {res['time_ms']:.3f} ms, "
                  f"verified: {res['verified']}", flush=True)
        return res

    def test_basic_alltoall(self, warmup: int = 20, iters: int = 20) -> dict:
        """Every pair at once (the reference's spread-out / fan-out baseline run), 4-byte units."""
        return self._run(PlanKind.FANOUT, 4, warmup, iters, "fanout")

    def test_flash_alltoall(self, warmup: int = 50, iters: int = 50) -> dict:
        """The scheduled collective (balance, BvN stages, redistribute), 8-byte units as in the reference."""
        return self._run(PlanKind.STAGED, 8, warmup, iters, "flash")
