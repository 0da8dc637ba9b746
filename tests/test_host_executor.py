"""CPU rank model of the executor: correctness of the multi-rank wait/signal logic and host-made
failures (absent rank, withheld signal, mismatched matrices over gloo)."""
import os
import subprocess
import sys
import time

import numpy as np
import pytest

from fast_b200 import sched
from fast_b200.parallel.host_executor import HostExecutor, HostTimeout
from fast_b200.sched import PlanKind, Topology


def _inputs(plan, ub, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, 256, int(plan.buffers[r, 0]) * ub, dtype=np.uint8) for r in range(plan.matrix.shape[0])]


@pytest.mark.parametrize("servers,gpus", [(4, 1), (2, 2), (2, 3), (1, 4)])
@pytest.mark.parametrize("kind", [PlanKind.STAGED, PlanKind.SINGLE_BURST, PlanKind.FANOUT, PlanKind.SPREAD_OUT])
def test_threads_match_sequential_replay(servers, gpus, kind):
    n = servers * gpus
    m = sched.workload_uniform(n, 200, 5 + n)
    plan = sched.build_plan(m, Topology(servers, gpus), kind=kind)
    ub = 3
    ins = _inputs(plan, ub)
    want = [np.zeros(int(plan.buffers[r, 1]) * ub, dtype=np.uint8) for r in range(n)]
    plan.execute_on_host(ub, ins, want)
    got = HostExecutor(plan, unit_bytes=ub, chunk_bytes=64).run(ins)
    for r in range(n):
        assert np.array_equal(got[r], want[r])


def test_absent_rank_is_reported_not_hung():
    m = sched.workload_uniform(4, 50, 1, zero_diag=True)
    plan = sched.build_plan(m, Topology.flat(4))
    ex = HostExecutor(plan, timeout_s=0.2, faults={"absent_rank": 2})
    with pytest.raises(HostTimeout) as e:
        ex.run(_inputs(plan, 1))
    assert e.value.site in (1, 4) and (e.value.site != 1 or e.value.detail == 2)


def test_withheld_signal_times_out_at_the_receiver():
    m = np.array([[0, 100], [100, 0]], dtype=np.int64)
    plan = sched.build_plan(m, Topology.flat(2), kind=PlanKind.FANOUT)
    ex = HostExecutor(plan, chunk_bytes=32, timeout_s=0.2, faults={"drop_signal": (0, 1)})
    with pytest.raises(HostTimeout) as e:
        ex.run(_inputs(plan, 1))
    assert e.value.rank == 1 and e.value.site == 4 and e.value.seen == 100 - 32 and e.value.want == 100


def test_hierarchical_withheld_rail_signal_blocks_redistribution():
    m = np.zeros((4, 4), dtype=np.int64)
    m[0, 3] = 64  # server 0 gpu 0 -> server 1 gpu 1: rail to (1,0) then redistribute
    plan = sched.build_plan(m, Topology(2, 2))
    rail_src = int(plan.ops[plan.ops[:, 0] == sched.PHASE_RAIL][0, 2])
    ex = HostExecutor(plan, chunk_bytes=1 << 20, timeout_s=0.2, faults={"drop_signal": (rail_src, 0)})
    with pytest.raises(HostTimeout) as e:
        ex.run(_inputs(plan, 1))
    assert e.value.site in (2, 3, 4)


def test_mismatched_matrices_detected_over_gloo(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(
        "import os, sys, numpy as np, torch.distributed as dist\n"
        f"sys.path.insert(0, {os.path.dirname(os.path.dirname(os.path.abspath(__file__)))!r})\n"
        "from fast_b200.parallel.host_executor import check_same_plan_inputs\n"
        "dist.init_process_group('gloo')\n"
        "r = dist.get_rank()\n"
        "m = np.full((2, 2), 7, dtype=np.int64)\n"
        "check_same_plan_inputs(m)\n"
        "m[0, 1] += r\n"
        "try:\n"
        "    check_same_plan_inputs(m)\n"
        "    print('MISSED')\n"
        "except RuntimeError as e:\n"
        "    print('DETECTED')\n"
        "dist.destroy_process_group()\n")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29571", str(script)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.count("DETECTED") == 2 and "MISSED" not in r.stdout


@pytest.mark.parametrize("world", [2, 4])
def test_p2p_executor_gloo(world):
    """Multi-process CPU ranks (gloo) execute flat and two-tier plans, forward and transposed."""
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mp_p2p_worker.py")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", str(29580 + world), worker], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-2500:]
    assert "P2P_OK" in r.stdout


# ---- native threaded twin of the device executor (csrc/sched/host_threads.cc) -----------------------

def _byte_inputs(m, unit, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, 256, size=int(m[r].sum()) * unit, dtype=np.uint8) for r in range(m.shape[0])]


@pytest.mark.parametrize("servers,gpus", [(4, 1), (2, 2), (2, 4), (3, 2)])
@pytest.mark.parametrize("kind", [PlanKind.STAGED, PlanKind.FANOUT, PlanKind.SINGLE_BURST, PlanKind.SPREAD_OUT])
def test_native_twin_matches_sequential_replay(servers, gpus, kind):
    """Several worker threads per rank, three collectives in a row over the same signal words:
    the outputs equal the sequential replay of the plan, bit for bit."""
    n = servers * gpus
    m = sched.workload_uniform(n, 200, 3 + n, False)
    p = sched.build_plan(m, Topology(servers, gpus), kind=kind)
    ins = _byte_inputs(m, 3, seed=n)
    want = [np.zeros(int(m[:, r].sum()) * 3, np.uint8) for r in range(n)]
    p.execute_on_host(3, ins, want)
    res = p.run_threads(ins, unit_bytes=3, chunk_bytes=128, workers=4, epochs=3, timeout_s=20.0)
    assert res["ok"], res["failure"]
    for r in range(n):
        assert np.array_equal(res["outputs"][r], want[r]), f"rank {r}"


def test_native_twin_reports_host_made_failures():
    m = sched.workload_uniform(4, 100, 1, True)
    p = sched.build_plan(m, Topology(2, 2))
    ins = _byte_inputs(m, 1)
    t0 = time.monotonic()
    res = p.run_threads(ins, timeout_s=0.3, absent_rank=2)           # a rank that never enters
    rank, site, detail, seen, want = res["failure"]                   # whichever wait ran out first is the one reported
    assert not res["ok"] and rank != 2 and site in (1, 2, 3, 4) and seen < want and (site != 1 or detail == 2)
    res = p.run_threads(ins, timeout_s=0.3, withhold_rank=0, withhold_item=0)    # a copy whose arrival is never counted
    assert not res["ok"] and res["failure"][1] in (2, 3, 4) and res["failure"][3] < res["failure"][4]
    assert time.monotonic() - t0 < 10.0
    with pytest.raises(Exception):
        p.tampered(0, "len", 0).run_threads(ins)                       # invalid plans are refused before anything runs


def test_protocol_is_race_free_under_thread_sanitizer():
    """The twin built with ThreadSanitizer is the protocol's race detector: clean as written,
    and reported as soon as the arrival signals lose their release / acquire order."""
    from fast_b200 import _build

    try:
        good = _build.build_twin_check(tsan=True)
        broken = _build.build_twin_check(tsan=True, relaxed=True)
    except Exception as e:  # no sanitizer runtime on this host
        pytest.skip(f"ThreadSanitizer build unavailable: {e}")
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=1 exitcode=66")
    r = subprocess.run([str(good), "1"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and '"failures":0' in r.stdout, r.stdout[-500:] + r.stderr[-2000:]
    r = subprocess.run([str(broken), "1"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 66 and "data race" in r.stderr


def test_moe_step_protocol_is_race_free_under_thread_sanitizer():
    """The expert-parallel step's flags and counters order every reuse of the receive buffers
    across steps (forward-only and forward + backward, 1 to 4 ranks); dropping the wait for the
    owners' ready flags before combine is reported."""
    from fast_b200 import _build

    try:
        good = _build.build_moe_twin(tsan=True)
        broken = _build.build_moe_twin(tsan=True, broken=True)
    except Exception as e:
        pytest.skip(f"ThreadSanitizer build unavailable: {e}")
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=1 exitcode=66")
    r = subprocess.run([str(good), "4"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and '"failures":0' in r.stdout, r.stdout[-500:] + r.stderr[-2000:]
    # the backward pass' entry handshake is belt and braces: the count exchange already orders the reuse
    r = subprocess.run([str(good), "4", "0"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and '"failures":0' in r.stdout, r.stdout[-500:] + r.stderr[-2000:]
    r = subprocess.run([str(broken), "3"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 66 and "data race" in r.stderr


@pytest.mark.parametrize("servers,gpus", [(2, 2), (2, 4), (3, 2)])
def test_rail_segments_run_bit_exact_in_both_host_models(servers, gpus):
    n = servers * gpus
    m = sched.workload_uniform(n, 300, 9 + n, False)
    p = sched.build_plan(m, Topology(servers, gpus))
    ins = _byte_inputs(m, 3, seed=n)
    want = [np.zeros(int(m[:, r].sum()) * 3, np.uint8) for r in range(n)]
    p.execute_on_host(3, ins, want)
    res = p.run_threads(ins, unit_bytes=3, chunk_bytes=128, workers=4, epochs=3, timeout_s=20.0, rail_segment_bytes=192)
    assert res["ok"], res["failure"]
    outs = HostExecutor(p, unit_bytes=3, chunk_bytes=128, timeout_s=10.0, rail_segment_bytes=192).run(ins)
    for r in range(n):
        assert np.array_equal(res["outputs"][r], want[r]) and np.array_equal(outs[r], want[r]), f"rank {r}"


def test_random_plans_and_lowering_options_through_the_native_twin():
    """Random topologies, sparse / skewed / single-entry matrices, plan kinds, alignments, unit and
    chunk sizes, rail segments and worker counts: the threaded twin always equals the replay."""
    from fast_b200.sched import MatchPolicy

    rng = np.random.default_rng(2024)
    kinds = [PlanKind.STAGED, PlanKind.SINGLE_BURST, PlanKind.FANOUT, PlanKind.SPREAD_OUT]
    for trial in range(240):
        S, G = int(rng.integers(1, 6)), int(rng.integers(1, 5))  # five servers and aligned cuts: remainders staged out of stage order
        n = S * G
        if trial % 3 == 0:
            m = sched.workload_uniform(n, int(rng.integers(1, 500)), trial, bool(trial % 2))
        elif trial % 3 == 1:
            m = rng.integers(0, 50, size=(n, n))
            m[rng.random((n, n)) < 0.6] = 0
        else:
            m = np.zeros((n, n), dtype=np.int64)
            m[rng.integers(0, n), rng.integers(0, n)] = int(rng.integers(1, 1000))
        p = sched.build_plan(np.ascontiguousarray(m, dtype=np.int64), Topology(S, G), kind=kinds[int(rng.integers(0, 4))],
                             split_align=int(rng.choice([1, 2, 4, 16])), transpose=bool(rng.integers(0, 2)),
                             match=MatchPolicy.BOTTLENECK if trial % 5 == 0 else MatchPolicy.FIRST_FIT)
        assert p.validate() == ""
        ub, pm = int(rng.choice([1, 3, 8, 16])), p.matrix
        ins = [rng.integers(0, 256, size=int(pm[r].sum()) * ub, dtype=np.uint8) for r in range(n)]
        want = [np.zeros(int(pm[:, r].sum()) * ub, np.uint8) for r in range(n)]
        p.execute_on_host(ub, ins, want)
        res = p.run_threads(ins, unit_bytes=ub, chunk_bytes=int(rng.choice([16, 64, 256, 4096])), workers=int(rng.integers(1, 5)), epochs=2,
                            timeout_s=20.0, rail_segment_bytes=int(rng.choice([0, 16, 48, 256, 1000])))
        assert res["ok"], (trial, res["failure"])
        for r in range(n):
            assert np.array_equal(res["outputs"][r], want[r]), (trial, r)
