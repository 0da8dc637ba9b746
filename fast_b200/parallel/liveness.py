"""Host-side failure detection: heartbeats and a bounded bootstrap exchange over a key-value store.

The reference has no failure detection: its error macros exit the process and every device wait
is unbounded (nvidia/src/include/fast_alltoall/alltoall_nvshmem.h:18-42,
nvidia/src/fast_alltoall/flash_alltoall_nvshmem.cu:1669-1676), so a lost peer is a hung GPU. Here
the device waits are bounded (a timed-out collective returns a status word), and this module is the
host half: ranks learn that a peer is gone BEFORE they launch the next collective, so that no
kernel is ever started that would have to time out.

Both classes work on any ``torch.distributed`` store (``TCPStore``, ``FileStore``, ``HashStore``,
``PrefixStore``), need no process group and never touch a GPU.
"""
from __future__ import annotations

import pickle
import threading
import time
from typing import Any, Dict, List, Optional


class PeerLost(RuntimeError):
    """Raised when one or more peers stopped beating (or said goodbye)."""

    def __init__(self, ranks: List[int], reason: str):
        self.ranks = list(ranks)
        self.reason = reason
        super().__init__(f"peer(s) {self.ranks} lost: {reason}")


class BootstrapTimeout(RuntimeError):
    """Raised when some ranks did not post their part of a bootstrap exchange in time."""

    def __init__(self, missing: List[int], what: str, timeout_s: float):
        self.missing = list(missing)
        super().__init__(f"bootstrap exchange '{what}': rank(s) {self.missing} posted nothing within {timeout_s:.1f} s")


def _try_get(store, key: str) -> Optional[bytes]:
    """Non-blocking read: ``None`` while the key does not exist."""
    if not store.check([key]):
        return None
    return store.get(key)


def bounded_exchange(store, rank: int, world: int, what: str, payload: Any, timeout_s: float = 30.0,
                     poll_s: float = 0.01) -> List[Any]:
    """All-gather of one picklable object per rank through the store, with a deadline.

    Every rank posts ``payload`` under ``what/<rank>`` and collects the others'. A rank that never
    posts (crashed before bootstrap, wrong world size, never started) makes the others raise
    :class:`BootstrapTimeout` naming it, instead of blocking in a collective for the process-group
    timeout. ``what`` must be unique per exchange (include a generation number when repeating)."""
    store.set(f"{what}/{rank}", pickle.dumps(payload))
    out: Dict[int, Any] = {rank: payload}
    deadline = time.monotonic() + timeout_s
    while len(out) < world:
        for r in range(world):
            if r not in out:
                raw = _try_get(store, f"{what}/{r}")
                if raw is not None:
                    out[r] = pickle.loads(raw)
        if len(out) == world:
            break
        if time.monotonic() > deadline:
            raise BootstrapTimeout([r for r in range(world) if r not in out], what, timeout_s)
        time.sleep(poll_s)
    return [out[r] for r in range(world)]


class Heartbeat:
    """Per-rank heartbeat counters in a store.

    Each rank increments its own counter every ``interval_s`` from a daemon thread (or by calling
    :meth:`beat` from its step loop). Observers never compare clocks between hosts: a peer is
    alive while its counter keeps changing, judged against the observer's own monotonic clock. A
    rank that leaves on purpose calls :meth:`leave`, which peers see at once.

    Typical use, between steps and before any launch::

        hb = Heartbeat(store, rank, world).start()
        for step in ...:
            hb.require_alive(max_age_s=2.0)     # raises PeerLost before a kernel could hang
            comm.all_to_all_v(...)
        hb.leave()
    """

    GONE = -1

    def __init__(self, store, rank: int, world: int, prefix: str = "fastb/hb", interval_s: float = 0.2):
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.prefix, self.interval_s = prefix, float(interval_s)
        self._count = 0
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        now = time.monotonic()
        self._seen: Dict[int, int] = {r: -2 for r in range(world)}       # last counter value read
        self._changed: Dict[int, float] = {r: now for r in range(world)}  # when it last changed, local clock
        self._left: set = set()
        self.beat()

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self) -> None:
        self._count += 1
        self.store.set(self._key(self.rank), str(self._count))

    def start(self) -> "Heartbeat":
        if self._thread is None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, name="fastb-heartbeat", daemon=True)
            self._thread.start()
        return self

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            try:
                self.beat()
            except Exception:  # the store went away with the job: nothing left to tell
                return

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5 * self.interval_s + 1.0)
            self._thread = None

    def leave(self) -> None:
        """Announce an orderly exit (between steps, nothing in flight) and stop beating."""
        self.stop()
        self.store.set(self._key(self.rank), str(self.GONE))

    def poll(self) -> None:
        now = time.monotonic()
        for r in range(self.world):
            if r == self.rank:
                continue
            raw = _try_get(self.store, self._key(r))
            if raw is None:
                continue
            v = int(raw)
            if v == self.GONE:
                self._left.add(r)
            elif v != self._seen[r]:
                self._seen[r], self._changed[r] = v, now

    def dead_peers(self, max_age_s: float) -> List[int]:
        """Ranks that left, or whose counter has not moved for ``max_age_s`` seconds."""
        self.poll()
        now = time.monotonic()
        return sorted(r for r in range(self.world)
                      if r != self.rank and (r in self._left or now - self._changed[r] > max_age_s))

    def require_alive(self, max_age_s: float = 2.0) -> None:
        dead = self.dead_peers(max_age_s)
        if dead:
            left = [r for r in dead if r in self._left]
            raise PeerLost(dead, f"left the job: {left}" if left == dead else f"no heartbeat for {max_age_s:.1f} s")

    def wait_all_started(self, timeout_s: float = 30.0) -> None:
        """Block until every peer has beaten at least once (start-up rendezvous with a deadline)."""
        deadline = time.monotonic() + timeout_s
        while True:
            self.poll()
            missing = [r for r in range(self.world) if r != self.rank and self._seen[r] == -2 and r not in self._left]
            if not missing:
                return
            if time.monotonic() > deadline:
                raise BootstrapTimeout(missing, self.prefix, timeout_s)
            time.sleep(0.01)
