"""The reference-shaped adapter (FlashAllToAll) on a stand-in communicator: planning, buffer sizes,
staging choice and dtype codes, all on the CPU."""
import numpy as np
import pytest
import torch

from fast_b200 import sched
from fast_b200.compat import DTYPE_CODES, FlashAllToAll, code_of, dtype_of
from fast_b200.parallel.comm import Schedule
from fast_b200.sched import PlanKind, Topology


class _Comm:
    """Plans for real (host scheduler + lowering), records launches instead of running them."""

    def __init__(self, rank, world, topo):
        self.rank, self.world, self.topo = rank, world, topo
        self.calls = []
        self.symmetric = set()

    def schedule(self, m, unit_bytes=1, transpose=False, kind=PlanKind.STAGED):
        plan = sched.build_plan(m, self.topo, kind=kind, transpose=transpose, split_align=1)
        assert plan.validate() == ""
        return Schedule(plan, unit_bytes, None, plan.lower(self.rank, unit_bytes, 1 << 16), self.rank)

    def offset_of(self, t):
        return 0 if id(t) in self.symmetric else None

    def alloc(self, n, dtype=torch.uint8):
        t = torch.zeros(n, dtype=dtype)
        self.symmetric.add(id(t))
        return t

    def init_buffers(self, s):
        return torch.zeros(max(s.max_bytes["input"], 1), dtype=torch.uint8), self.alloc(max(s.max_bytes["output"], 1))

    def free_buffers(self, recv):
        self.symmetric.discard(id(recv))

    def all_to_all_v(self, output, input, s, staging=None):
        self.calls.append(("v", output, input, s, staging))
        return output

    def all_to_all_single(self, output, input, out_splits, in_splits, kind=None):
        self.calls.append(("single", output, input, out_splits, in_splits, kind))
        return output


def _matrix(world, seed=0):
    rng = np.random.default_rng(seed)
    m = rng.integers(0, 50, size=(world, world))
    np.fill_diagonal(m, 0)
    return m


def test_dtype_codes_follow_the_reference_table():
    assert dtype_of(9) == torch.bfloat16 and dtype_of(10) == torch.float8_e4m3fn and dtype_of(11) == torch.float8_e5m2
    assert dtype_of(6) == torch.float16 and dtype_of(7) == torch.float32 and dtype_of(99) == torch.int8
    for c, d in DTYPE_CODES.items():
        assert code_of(d) == c


def test_schedule_and_buffer_sizes_in_tokens():
    world, S, G, hidden = 8, 2, 4, 64
    m = _matrix(world)
    for rank in (0, 5):
        f = FlashAllToAll(rank, world, S, G, hidden, 9, b"ignored", comm=_Comm(rank, world, Topology(S, G)))
        assert (f.get_world_size(), f.get_rank(), f.get_server_n(), f.get_hidden_sz()) == (world, rank, S, hidden)
        with pytest.raises(RuntimeError):
            f.get_buffer_szs()
        f.schedule(m.reshape(-1), 0)
        szs = f.get_buffer_szs()
        assert len(szs) == 6 and szs[0] == m[rank].sum() and szs[1] == 0 and szs[4] == 0 and szs[5] == 0
        assert szs[2] > 0 and szs[3] > 0                        # two-tier plan: balance and rail staging exist
        assert f.sched.unit_bytes == hidden * 2 and f.sched.output_bytes == m[:, rank].sum() * hidden * 2
        f.schedule(m.reshape(-1), 1)                            # backward: the transposed collective
        assert f.get_buffer_szs()[0] == m[:, rank].sum() and f.sched.output_bytes == m[rank].sum() * hidden * 2
    flat = FlashAllToAll(0, world, S, G, hidden, 9, comm=_Comm(0, world, Topology.flat(world)), flat=True)
    flat.schedule(m, 0)
    assert list(flat.get_buffer_szs()[1:]) == [0, 0, 0, 0, 0]   # flat: data lands in place, no staging at all
    with pytest.raises(ValueError):
        FlashAllToAll(0, world, 3, 4, hidden, 9, comm=_Comm(0, world, Topology(S, G)))


def test_all_to_all_paths_choose_buffers_like_the_reference_calls():
    world, S, G, hidden = 4, 2, 2, 32
    comm = _Comm(1, world, Topology(S, G))
    f = FlashAllToAll(1, world, S, G, hidden, 7, comm=comm)
    m = _matrix(world, 3)
    f.schedule(m, 0)
    s = f.sched
    inp = torch.zeros(max(s.input_bytes, 1), dtype=torch.uint8)
    out = torch.zeros(max(s.output_bytes, 1), dtype=torch.uint8)
    with pytest.raises(RuntimeError):
        f.all_to_all()
    f.init_buffers(inp, out)                                    # plain output: goes through a symmetric receive buffer
    assert f.all_to_all() is out and comm.calls[-1][1] is f._recv
    f.free_buffers()
    sym_out = comm.alloc(max(s.output_bytes, 1))
    f.init_buffers(inp, sym_out)                                # symmetric output: written in place
    assert f.all_to_all() is sym_out and comm.calls[-1][1] is sym_out
    f.free_buffers()
    # caller-owned staging: used when symmetric and large enough, else the library's own
    lbrecv, cros = comm.alloc(s.max_bytes["balance"]), comm.alloc(s.max_bytes["rail"])
    f.all_to_all_2(inp, sym_out, None, None, lbrecv, cros, None, None)
    assert comm.calls[-1][4] == {"balance": lbrecv, "rail": cros}
    f.all_to_all_2(inp, sym_out, None, None, torch.zeros(8, dtype=torch.uint8), comm.alloc(1), None, None)
    assert comm.calls[-1][4] is None
    # fan-out baseline: splits in tokens, rows of hidden_sz elements
    x = torch.zeros(int(m[1].sum()) * hidden, dtype=torch.float32)
    y = torch.zeros(int(m[:, 1].sum()) * hidden, dtype=torch.float32)
    f.all_to_all_v(x, y, list(m[1]), list(m[:, 1]))
    kind, o, i, osz, isz, k = comm.calls[-1]
    assert kind == "single" and i.shape == (int(m[1].sum()), hidden) and o.shape == (int(m[:, 1].sum()), hidden) and k == PlanKind.FANOUT
    with pytest.raises(ValueError):
        f.all_to_all_v(x, y, [1], [1])


def test_pattern_words_match_the_reference_scheme():
    from fast_b200.compat import pattern_words

    w = pattern_words(3, 5, 70000, "cpu")
    assert w.dtype == torch.int32 and w.numel() == 70000
    assert int(w[0]) == (3 << 24) | (5 << 16) and int(w[65535]) == (3 << 24) | (5 << 16) | 0xFFFF and int(w[65536]) == int(w[0])
    assert pattern_words(0, 0, 0, "cpu").numel() == 0


def test_named_configs_and_memory_plan():
    from fast_b200.models.configs import (CONFIGS, DEEPSEEK_V3_MOE_LAYER, HBM_BYTES, MIXTRAL_8X7B_BLOCK, flops_per_step, max_tokens_per_rank,
                                          memory_plan)

    assert set(CONFIGS) == {"mixtral-8x7b-block", "deepseek-v3-moe-layer"}
    mx, ds = MIXTRAL_8X7B_BLOCK, DEEPSEEK_V3_MOE_LAYER
    assert (mx.hidden, mx.inter, mx.num_experts, mx.top_k, mx.tokens_per_rank, mx.vocab) == (4096, 14336, 8, 2, 32768, 32000)
    assert (ds.hidden, ds.inter, ds.num_experts, ds.top_k, ds.tokens_per_rank, ds.fp8_dispatch) == (7168, 2048, 256, 8, 4096, True)
    # capacity: the engine's formula (worst case, padded to 256 rows)
    assert mx.capacity_rows(1) == 67584 and mx.capacity_rows(8) == (8 * 32768 * 1 + 256 + 255) // 256 * 256
    assert mx.capacity_rows(8, capacity_factor=1.0) == (32768 * 2 + 256 + 255) // 256 * 256
    with pytest.raises(ValueError):
        mx.experts_per_rank(3)
    for cfg in (mx, ds):
        for world in (1, 2, 4, 8):
            p = memory_plan(cfg, world)
            assert p["total"] == sum(p[k] for k in ("symmetric_heap", "workspace", "weights", "grads", "optimizer", "tokens"))
            assert p["fits_b200"] and p["total"] < HBM_BYTES
    # expert weights shard over ranks, AdamW state is 6x the bf16 weights, forward-only layers carry none
    p1, p8 = memory_plan(mx, 1), memory_plan(mx, 8)
    assert p1["optimizer"] == 6 * p1["weights"] and p8["weights"] < p1["weights"] / 4 and memory_plan(ds, 8)["optimizer"] == 0
    assert memory_plan(mx, 8, capacity_factor=1.0)["total"] < p8["total"] / 2
    # the largest batch that fits is far above the benchmark's, and one step more does not fit
    t = max_tokens_per_rank(mx, 8)
    assert t > mx.tokens_per_rank and memory_plan(mx.with_(tokens_per_rank=t), 8)["fits_b200"]
    assert not memory_plan(mx.with_(tokens_per_rank=t + 1024), 8)["fits_b200"]
    f = flops_per_step(mx, 8)
    assert f["expert_gemm_total"] == 3 * f["expert_gemm_fwd"] == 3 * 2.0 * 65536 * 4096 * 14336 * 3


def test_init_id_stand_in_has_the_reference_shape():
    from fast_b200.compat import get_nvshmem_init_id

    uid = get_nvshmem_init_id()
    assert uid.dtype == torch.uint8 and uid.numel() == 128 and uid.device.type == "cpu"


def test_torch_custom_ops_are_registered_with_schemas_and_trace_with_fake_tensors():
    from torch._subclasses.fake_tensor import FakeTensorMode

    from fast_b200.ops import registry  # noqa: F401  (registers torch.ops.fast_b200.*)

    schema = str(torch.ops.fast_b200.grouped_gemm_fwd.default._schema)
    assert "Tensor(a3!) out" in schema and "Tensor(a5!)? gate_up_out" in schema      # outputs are declared as mutated
    assert "-> (Tensor, Tensor)" in str(torch.ops.fast_b200.route_topk.default._schema)
    for name in ("grouped_gemm_dgrad", "grouped_gemm_wgrad"):
        assert hasattr(torch.ops.fast_b200, name)
    with FakeTensorMode():                                                               # shapes propagate, no kernel runs
        logits = torch.empty(100, 8, dtype=torch.float32, device="cuda")
        idx, w = torch.ops.fast_b200.route_topk(logits, None, 2)
        assert idx.shape == (100, 2) and idx.dtype == torch.int32 and w.dtype == torch.float32 and w.device.type == "cuda"
        a = torch.empty(512, 256, dtype=torch.bfloat16, device="cuda")
        wt = torch.empty(2, 512, 256, dtype=torch.bfloat16, device="cuda")
        off = torch.empty(3, dtype=torch.int32, device="cuda")
        out = torch.empty(512, 512, dtype=torch.bfloat16, device="cuda")
        assert torch.ops.fast_b200.grouped_gemm_fwd(a, wt, off, out, False, None) is None
        assert torch.ops.fast_b200.grouped_gemm_dgrad(out, wt, off, a, None) is None
        assert torch.ops.fast_b200.grouped_gemm_wgrad(out, a, off, torch.empty_like(wt)) is None


def test_step_roofline_adds_up():
    from fast_b200.models.configs import DEEPSEEK_V3_MOE_LAYER, MIXTRAL_8X7B_BLOCK, step_roofline

    r1 = step_roofline(MIXTRAL_8X7B_BLOCK, 1, 1395.2, 6546.6)
    r8 = step_roofline(MIXTRAL_8X7B_BLOCK, 8, 1395.2, 6546.6)
    assert r1["gemm_ms"] == pytest.approx(69.27e12 / 1395.2e12 * 1e3, rel=1e-3) and r1["a2a_ms"] == 0.0
    assert r1["adamw_ms"] == pytest.approx(8 * 3 * 4096 * 14336 * 28 / 6546.6e9 * 1e3, rel=1e-6)
    assert r8["adamw_ms"] == pytest.approx(r1["adamw_ms"] / 8) and r8["a2a_ms"] > 0 and r8["gemm_ms"] == r1["gemm_ms"]
    assert all(abs(r["total_ms"] - (r["gemm_ms"] + r["adamw_ms"] + r["a2a_ms"])) < 1e-9 for r in (r1, r8))
    d = step_roofline(DEEPSEEK_V3_MOE_LAYER, 8, 1395.2, 6546.6)
    assert d["adamw_ms"] == 0.0 and d["a2a_ms"] == pytest.approx(4096 * 8 * 7 / 8 * (7168 + 14336) / 770e9 * 1e3)


def test_differentiable_all_to_all_wrapper_logic_on_a_stand_in():
    """The autograd wrapper with a stand-in communicator (identity exchange on one rank): output
    shape from the plan's sizes, gradient routed through the transposed schedule."""
    from types import SimpleNamespace

    from fast_b200.parallel import autograd as ag

    class _Comm:
        def __init__(self):
            self.calls = []

        def schedule(self, matrix, unit_bytes=1, kind=None, transpose=False):
            rows = int(np.asarray(matrix).sum())
            return SimpleNamespace(unit_bytes=unit_bytes, output_bytes=rows * unit_bytes, transpose=transpose)

        def all_to_all_v(self, out, inp, s):
            self.calls.append(s.transpose)
            out.view(-1).copy_(inp.reshape(-1))
            return out

    comm = _Comm()
    x = torch.randn(30, 8, requires_grad=True)
    y = ag.all_to_all_v(x, comm, np.array([[30]]), kind="auto")
    assert y.shape == (30, 8) and torch.equal(y.detach(), x.detach())
    w = torch.randn(30, 8)
    (y * w).sum().backward()
    assert torch.equal(x.grad, w) and comm.calls == [False, True]


def _bare_communicator(rank, world, topo):
    """A Communicator without a device: enough state for ``schedule`` (planning, validation,
    lowering, caching); the device program is replaced by a recorder."""
    from types import SimpleNamespace

    from fast_b200.parallel.comm import Communicator

    c = object.__new__(Communicator)
    c.rank, c.world, c.topo, c.ctas, c.group = rank, world, topo, 148, None
    c.plan_cache, c._sched_cache = sched.PlanCache(), {}
    c.device = SimpleNamespace(index=0)
    c._C = SimpleNamespace(A2AProgram=lambda items, rail, out, bal, dev: SimpleNamespace(n_items=int(items.shape[0]), rail=list(rail)))
    return c


def test_communicator_schedule_paths_without_a_device():
    m = sched.workload_uniform(8, 4000, 3, False)
    c = _bare_communicator(2, 8, Topology(2, 4))
    s = c.schedule(m, unit_bytes=16, kind=PlanKind.STAGED)
    assert s.plan.only_rank == -1 and s.program.n_items > 0 and len(s.program.rail) == s.plan.num_stages
    assert c.schedule(m, unit_bytes=16, kind=PlanKind.STAGED) is s                       # cached
    seg = c.schedule(m, unit_bytes=16, kind=PlanKind.STAGED, rail_segment_bytes=512)
    assert seg is not s and len(seg.program.rail) > s.plan.num_stages and sum(seg.program.rail) == sum(s.program.rail)
    auto = c.schedule(m, unit_bytes=16, kind="auto")
    assert auto.plan.kind in (PlanKind.FANOUT, PlanKind.STAGED, PlanKind.SINGLE_BURST) and auto.plan.validate() == ""
    back = c.schedule(m, unit_bytes=16, kind=PlanKind.STAGED, transpose=True)
    assert back.input_bytes == int(m[:, 2].sum()) * 16 and back.output_bytes == int(m[2].sum()) * 16
    # beyond 64 ranks a communicator plans a one-rank view, with the same work list as the full plan
    big = sched.workload_uniform(72, 300, 5, False)
    c72 = _bare_communicator(7, 72, Topology(9, 8))
    v = c72.schedule(big, unit_bytes=4, kind=PlanKind.STAGED)
    full = sched.build_plan(big, Topology(9, 8), split_align=4)
    assert v.plan.only_rank == 7 and v.plan.num_ops < full.num_ops / 10
    ref = full.lower(7, 4, 65536)                                                          # 64 KiB work items are what schedule() picks here
    assert v.lowered["items"].shape == ref["items"].shape and (v.lowered["items"] == ref["items"]).all()
    assert v.lowered["expect_output_bytes"] == ref["expect_output_bytes"] and v.max_bytes["rail"] == int(full.buffers[:, 3].max()) * 4


def test_communicator_launch_arguments_and_close_without_a_device():
    from types import SimpleNamespace

    from fast_b200.parallel.liveness import PeerLost

    class _Heap:
        bytes = 1 << 30

        def __init__(self):
            self.next, self.freed = 256, []

        def alloc(self, n):
            off, self.next = self.next, self.next + (n + 255) // 256 * 256
            return off

        def free(self, off):
            self.freed.append(off)

        def base_ptr(self, rank):
            return 1 << 40                                   # no CPU tensor lies inside this "slab"

        def tensor(self, off, shape, dtype):
            return torch.zeros(shape, dtype=dtype)

    c = _bare_communicator(0, 4, Topology(2, 2))
    c.heap, c.broken, c.liveness, c.liveness_max_age_s, c._staging = _Heap(), False, None, 2.0, {}
    s = c.schedule(sched.workload_uniform(4, 100, 1, False), unit_bytes=4, kind=PlanKind.STAGED)
    inp, out = torch.zeros(s.input_bytes, dtype=torch.uint8), torch.zeros(s.output_bytes, dtype=torch.uint8)
    src, dst, copy_back = c._launch_args(s, out, inp)
    assert copy_back is not None and src[0] == inp.data_ptr() and dst[0] == 0 and dst[1] == c._staging["recv"][0]
    assert dst[2] == c._staging["balance"][0] and dst[3] == c._staging["rail"][0] and src[2] == (1 << 40) + dst[2]
    again = c._launch_args(s, out, inp)
    assert again[1] == dst and c.heap.freed == []                          # staging is reused, not re-allocated
    with pytest.raises(ValueError):
        c._launch_args(s, out[:-1], inp)
    with pytest.raises(ValueError):
        c._launch_args(s, out, inp, staging={"rail": torch.zeros(8, dtype=torch.uint8)})   # not symmetric memory
    c.liveness = SimpleNamespace(require_alive=lambda age: (_ for _ in ()).throw(PeerLost([3], "no heartbeat")), leave=lambda: None)
    with pytest.raises(PeerLost):
        c._launch_args(s, out, inp)                                          # a lost peer stops the launch on the host
    c.liveness = None
    c.broken = True
    with pytest.raises(RuntimeError, match="reset"):
        c._launch_args(s, out, inp)
    c.broken, c.heap = False, None
    with pytest.raises(RuntimeError, match="closed"):
        c._launch_args(s, out, inp)


def test_close_unmaps_peers_between_two_barriers_before_the_slab_goes(monkeypatch):
    """Teardown order across ranks: sync, barrier, unmap peers, barrier, and only then drop the heap
    (whose destructor frees the local slab). A peer that still had the slab mapped when its owner
    freed it would be undefined behaviour in CUDA."""
    import torch.distributed as dist

    log = []

    class _Heap:
        def close_peers(self):
            log.append("close_peers")

        def __del__(self):
            log.append("free_local")

    c = _bare_communicator(1, 4, Topology.flat(4))
    c.heap, c.group, c._virtual, c.liveness, c._staging, c.broken = _Heap(), object(), False, None, {}, False
    monkeypatch.setattr(torch.cuda, "synchronize", lambda dev=None: log.append("sync"))
    monkeypatch.setattr(dist, "barrier", lambda group=None: log.append("barrier"))
    c.close()
    import gc

    gc.collect()
    assert log == ["sync", "barrier", "close_peers", "barrier", "free_local"]
    c.close()                                                   # idempotent: nothing more happens
    assert log[-1] == "free_local" and len(log) == 5
    # virtual ranks of an in-process group share one address space: no mappings to close, no barrier
    v = _bare_communicator(0, 2, Topology.flat(2))
    v.heap, v.group, v._virtual, v.liveness, v._staging, v.broken = _Heap(), None, True, None, {}, False
    del log[:]
    v.close()
    gc.collect()
    assert log == ["sync", "free_local"]
