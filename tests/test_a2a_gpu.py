"""GPU tests of the all-to-all(v) executor: bit-exact against the host replay of the same plan.

Pattern words follow the reference's verification scheme (src << 24 | dst << 16 | index,
nvidia/src/fast_alltoall/flash_alltoall_nvshmem.cu:1445-1473).
"""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from fast_b200 import sched
from fast_b200.sched import PlanKind, Topology

pytestmark = pytest.mark.gpu


def _pattern_inputs(m, unit_words):
    n = m.shape[0]
    ins = []
    for r in range(n):
        segs = []
        for d in range(n):
            k = int(m[r, d]) * unit_words
            segs.append(((r << 24) | (d << 16) | (np.arange(k) & 0xFFFF)).astype(np.int32))
        ins.append(np.concatenate(segs) if segs else np.zeros(0, np.int32))
    return ins


def _expected_outputs(m, ins, unit_words):
    n = m.shape[0]
    ind = np.concatenate([np.zeros((n, 1), np.int64), np.cumsum(m, 1)], 1) * unit_words
    outs = []
    for d in range(n):
        outs.append(np.concatenate([ins[s][ind[s, d]:ind[s, d + 1]] for s in range(n)]))
    return outs


@pytest.mark.parametrize("servers,gpus", [(1, 1), (2, 1), (4, 1), (8, 1), (2, 2), (2, 4), (1, 4)])
@pytest.mark.parametrize("kind", [PlanKind.STAGED, PlanKind.FANOUT, PlanKind.SPREAD_OUT, PlanKind.SINGLE_BURST, "auto"])
def test_local_group_bit_exact(servers, gpus, kind):
    from fast_b200.parallel import LocalGroup

    n = servers * gpus
    grp = LocalGroup(n, heap_bytes=64 << 20, topo=Topology(servers, gpus), ctas=4, threads=256)
    for seed, unit_words in [(1, 4), (2, 1), (3, 64)]:
        m = sched.workload_uniform(n, 300, seed + n, zero_diag=False)
        ss = grp.schedule(m, unit_bytes=4 * unit_words, kind=kind, chunk_bytes=8192)
        ins = _pattern_inputs(m, unit_words)
        want = _expected_outputs(m, ins, unit_words)
        d_in = [torch.from_numpy(x).cuda() for x in ins]
        mx = max(s.max_bytes["output"] for s in ss) // 4
        d_out = [c.alloc(mx, torch.int32) for c in grp.comms]
        for o in d_out:
            o.fill_(-1)
        for _ in range(2):  # twice: counters must be clean for the next epoch
            grp.all_to_all_v(d_out, d_in, ss)
            grp.check()
            for r in range(n):
                got = d_out[r][: want[r].size].cpu().numpy()
                assert np.array_equal(got, want[r]), f"rank {r} differs"
        for c, o in zip(grp.comms, d_out):
            c.free(o)


def test_unaligned_byte_units():
    from fast_b200.parallel import LocalGroup

    n = 4
    grp = LocalGroup(n, heap_bytes=16 << 20, ctas=2, threads=128)
    rng = np.random.default_rng(0)
    m = np.array([[0, 1, 15, 17], [33, 0, 16, 5], [7, 1000, 3, 0], [129, 2, 0, 31]], dtype=np.int64)
    ss = grp.schedule(m, unit_bytes=1, kind=PlanKind.STAGED, chunk_bytes=64)
    ins = [rng.integers(0, 256, int(m[r].sum()), dtype=np.uint8) for r in range(n)]
    d_in = [torch.from_numpy(x).cuda() for x in ins]
    d_out = [torch.zeros(int(m[:, r].sum()) + 16, dtype=torch.uint8, device="cuda") for r in range(n)]  # library-owned staging path
    grp.all_to_all_v(d_out, d_in, ss)
    grp.check()
    host_out = [np.zeros(int(m[:, r].sum()), np.uint8) for r in range(n)]
    ss[0].plan.execute_on_host(1, ins, host_out)
    for r in range(n):
        assert np.array_equal(d_out[r][: host_out[r].size].cpu().numpy(), host_out[r])


def test_bounded_wait_reports_timeout():
    """A wait on a flag nobody sets must end by itself and leave a readable status."""
    from fast_b200 import runtime

    C = runtime.ext()
    st = C.StatusBlock()
    flag = torch.zeros(1, dtype=torch.int64, device="cuda")
    C.wait_probe(flag.data_ptr(), 1, st, 50_000_000)  # 50 ms
    code, site, detail, seen, want = st.read()
    assert (code, site, seen, want) == (1, 9, 0, 1)
    # the context stays usable
    assert int((torch.ones(4, device="cuda") * 2).sum().item()) == 8
    st.clear()
    flag.fill_(1)
    C.wait_probe(flag.data_ptr(), 1, st, 50_000_000)
    assert st.read()[0] == 0


def test_missing_peer_times_out_cleanly():
    """Rank 1 of a 2-rank group never publishes its epoch: rank 0's push must give up, not hang."""
    from fast_b200 import runtime
    from fast_b200.parallel import LocalGroup

    grp = LocalGroup(2, heap_bytes=8 << 20, timeout_s=0.05, ctas=1, threads=64)
    m = np.array([[0, 64], [64, 0]], dtype=np.int64)
    c0 = grp.comms[0]
    s0 = c0.schedule(m, unit_bytes=16, kind=PlanKind.FANOUT)
    out = c0.alloc(64 * 16, torch.uint8)
    grp.comms[1].alloc(64 * 16, torch.uint8)
    inp = torch.zeros(64 * 16, dtype=torch.uint8, device="cuda")
    c0.all_to_all_v(out, inp, s0)  # alone: the peer never enters
    with pytest.raises(runtime.CollectiveTimeout) as e:
        c0.check()
    assert e.value.site == 1 and e.value.detail == 1
    assert c0.broken


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_multi_process_bit_exact():
    n = min(torch.cuda.device_count(), 8)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
                        "--master-port", "29533", os.path.join(os.path.dirname(__file__), "mp_a2a_worker.py")], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "A2A_MP_OK" in r.stdout


def test_reference_shaped_adapter_on_one_rank():
    """FlashAllToAll (the reference's flash_t calls) end to end on a world of one: library-owned
    and caller-owned paths both deliver the self segment."""
    from fast_b200.compat import FlashAllToAll
    from fast_b200.parallel import Communicator

    comm = Communicator(heap_bytes=64 << 20, device=0)
    f = FlashAllToAll(0, 1, 1, 1, 128, 9, comm=comm)
    tokens = 1000
    f.schedule(np.array([tokens], dtype=np.int32), 0)
    assert list(f.get_buffer_szs()) == [tokens, 0, 0, 0, 0, 0]
    x = torch.randn(tokens, 128, device="cuda").to(torch.bfloat16)
    y = torch.zeros_like(x)
    f.init_buffers(x, y)
    f.all_to_all()
    comm.check()
    assert torch.equal(x, y)
    f.free_buffers()
    z = comm.alloc((tokens, 128), torch.bfloat16)
    z.zero_()
    f.all_to_all_2(x, z, None, None, None, None, None, None)
    comm.check()
    assert torch.equal(x, z)
    w = torch.zeros_like(x)
    f.all_to_all_v(x.view(-1), w.view(-1), [tokens], [tokens])
    comm.check()
    assert torch.equal(x, w)


def test_reference_tester_class_on_one_rank():
    """FlashComm (the reference's NVIDIA tester class): both self-tests verify their buffers."""
    from fast_b200.compat import FlashComm
    from fast_b200.parallel import Communicator

    t = FlashComm(0, 1, 1, None, comm=Communicator(heap_bytes=64 << 20, device=0), mean_units=1 << 16)
    for res in (t.test_basic_alltoall(warmup=2, iters=2), t.test_flash_alltoall(warmup=2, iters=2)):
        assert res["verified"] and res["time_ms"] > 0 and res["per_gpu_MB"] > 0


def test_close_refuses_further_launches_and_keeps_live_tensors_valid():
    from fast_b200.parallel import Communicator

    with Communicator(heap_bytes=16 << 20, device=0) as comm:
        s = comm.schedule(np.array([[256]], dtype=np.int64), unit_bytes=4)
        out = comm.alloc(256, torch.int32)
        x = torch.arange(256, dtype=torch.int32, device="cuda")
        comm.all_to_all_v(out, x, s)
        comm.check()
        assert torch.equal(out, x)
    with pytest.raises(RuntimeError, match="closed"):
        comm.all_to_all_v(out, x, s)
    out.add_(1)                      # the slab lives as long as a tensor carved from it
    torch.cuda.synchronize()
    assert torch.equal(out, x + 1)
    comm.close()                     # idempotent


@pytest.mark.parametrize("servers,gpus", [(2, 2), (2, 4)])
@pytest.mark.parametrize("kind", [PlanKind.STAGED, PlanKind.SINGLE_BURST])
def test_rail_segments_bit_exact(servers, gpus, kind):
    """Two-tier plans with one arrival counter per 512 bytes of rail staging (chunk-level readiness
    inside a stage): same kernel, more counters; outputs equal the expected pattern, twice in a row."""
    from fast_b200.parallel import LocalGroup

    n = servers * gpus
    grp = LocalGroup(n, heap_bytes=64 << 20, topo=Topology(servers, gpus), ctas=4, threads=256)
    m = sched.workload_uniform(n, 300, 41 + n, zero_diag=False)
    unit_words = 4
    ss = grp.schedule(m, unit_bytes=4 * unit_words, kind=kind, chunk_bytes=8192, rail_segment_bytes=512)
    assert max(len(s.lowered["expect_rail_bytes"]) for s in ss) > ss[0].plan.num_stages
    ins = _pattern_inputs(m, unit_words)
    want = _expected_outputs(m, ins, unit_words)
    d_in = [torch.from_numpy(x).cuda() for x in ins]
    mx = max(s.max_bytes["output"] for s in ss) // 4
    d_out = [c.alloc(mx, torch.int32) for c in grp.comms]
    for _ in range(2):
        for o in d_out:
            o.fill_(-1)
        grp.all_to_all_v(d_out, d_in, ss)
        grp.check()
        for r in range(n):
            assert np.array_equal(d_out[r][: want[r].size].cpu().numpy(), want[r]), f"rank {r} differs"


def test_differentiable_all_to_all_on_one_rank():
    """The autograd wrapper: forward through the plan, gradients back through the transposed plan."""
    from fast_b200.parallel import Communicator, all_to_all_v

    with Communicator(heap_bytes=32 << 20, device=0) as comm:
        x = torch.randn(300, 64, device="cuda", dtype=torch.float32, requires_grad=True)
        y = all_to_all_v(x, comm, np.array([[300]], dtype=np.int64), kind=PlanKind.FANOUT)
        comm.check()
        assert y.shape == x.shape and torch.equal(y.detach(), x.detach())
        w = torch.randn_like(y)
        (y * w).sum().backward()
        comm.check()
        assert torch.equal(x.grad, w)
