"""Host-side failure detection: all failures are made on the host (a rank that never joins, one
that leaves between steps, one whose process exits); no GPU is involved."""
import os
import subprocess
import sys
import threading
import time

import pytest
import torch.distributed as dist

from fast_b200.parallel.liveness import BootstrapTimeout, Heartbeat, PeerLost, bounded_exchange


def test_bounded_exchange_gathers_every_rank():
    store = dist.HashStore()
    out = [None] * 3

    def run(r):
        out[r] = bounded_exchange(store, r, 3, "handles/0", {"rank": r, "blob": bytes([r]) * 64}, timeout_s=5.0)

    ts = [threading.Thread(target=run, args=(r,)) for r in range(3)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    for r in range(3):
        assert [o["rank"] for o in out[r]] == [0, 1, 2]
        assert out[r][2]["blob"] == b"\x02" * 64


def test_bounded_exchange_names_the_rank_that_never_posted():
    store = dist.HashStore()
    errs = {}

    def run(r):
        try:
            bounded_exchange(store, r, 3, "handles/1", r, timeout_s=0.3)
        except BootstrapTimeout as e:
            errs[r] = e

    ts = [threading.Thread(target=run, args=(r,)) for r in (0, 2)]  # rank 1 never starts
    t0 = time.monotonic()
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert time.monotonic() - t0 < 3.0
    assert set(errs) == {0, 2} and errs[0].missing == [1] and errs[2].missing == [1]


def test_heartbeat_sees_silence_and_goodbye():
    store = dist.HashStore()
    hbs = [Heartbeat(store, r, 3, interval_s=0.02) for r in range(3)]
    [h.start() for h in hbs]
    hbs[0].wait_all_started(timeout_s=2.0)
    time.sleep(0.1)
    hbs[0].require_alive(max_age_s=5.0)            # everyone beats
    hbs[1].stop()                                  # rank 1 goes silent (as if its process died)
    hbs[0].poll()
    time.sleep(1.2)
    assert hbs[0].dead_peers(max_age_s=0.8) == [1]  # rank 2 beats every 20 ms: far inside the window even on a loaded host
    with pytest.raises(PeerLost) as e:
        hbs[0].require_alive(max_age_s=0.8)
    assert e.value.ranks == [1] and "no heartbeat" in str(e.value)
    hbs[2].leave()                                 # orderly exit is seen at once, without waiting
    with pytest.raises(PeerLost) as e:
        hbs[0].require_alive(max_age_s=60.0)
    assert e.value.ranks == [2] and "left the job" in str(e.value)
    hbs[0].stop()


def test_wait_all_started_has_a_deadline():
    store = dist.HashStore()
    hb = Heartbeat(store, 0, 2, interval_s=0.05)
    with pytest.raises(BootstrapTimeout) as e:
        hb.wait_all_started(timeout_s=0.2)
    assert e.value.missing == [1]


_WORKER = r"""
import os, sys, time, datetime
import torch.distributed as dist
from fast_b200.parallel.liveness import Heartbeat, PeerLost
rank, world, port, mode = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=datetime.timedelta(seconds=20))
hb = Heartbeat(store, rank, world, interval_s=0.05).start()
hb.wait_all_started(10.0)
steps = 0
try:
    for step in range(200):
        hb.require_alive(max_age_s=1.5)   # the check a rank makes before it launches a collective
        steps += 1
        if rank == world - 1 and step == 3:
            if mode == "leave":
                hb.leave()
            os._exit(0)                  # between steps, nothing in flight ("crash": no goodbye)
        time.sleep(0.02)
    print(f"rank {rank} NOT-DETECTED", flush=True)
except PeerLost as e:
    print(f"rank {rank} detected {e.ranks} after {steps} steps", flush=True)
    if rank == 0:
        time.sleep(2.5)                  # keep the store up until the other survivors have reported
"""


@pytest.mark.parametrize("mode", ["leave", "crash"])
def test_processes_learn_of_a_lost_rank_before_their_next_launch(tmp_path, mode):
    world, port = 3, 29611 if mode == "leave" else 29612
    script = tmp_path / "w.py"
    script.write_text(_WORKER)
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([os.path.dirname(os.path.dirname(os.path.abspath(__file__))), os.environ.get("PYTHONPATH", "")]))
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(world), str(port), mode], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True, env=env) for r in range(world)]
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=60)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append(o)
    for r in range(world - 1):
        assert f"rank {r} detected [{world - 1}]" in outs[r], outs
    assert procs[-1].returncode == 0
