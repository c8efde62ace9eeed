"""Host-side failure detection for multi-process training.

The reference has none (it restarts from a checkpoint by hand, omegalax/trainers/text.py:115-120).
Two pieces, both pure host code so that nothing ever waits on a GPU for a peer that is gone:

``StepWatchdog``   a daemon thread with a per-step deadline.  The training loop calls ``beat(step)``
                   once per step; if no beat arrives in time the watchdog dumps every Python stack
                   to stderr (it never touches the device, which may be the thing that is stuck)
                   and runs ``on_timeout`` (default: leave the process with exit code 124 so
                   that a launcher can restart from the last checkpoint).
``PeerHeartbeat``  liveness over the rendezvous key-value store (``torch.distributed`` TCPStore /
                   FileStore / HashStore): every rank publishes a counter from a daemon thread and
                   ``check()`` -- called between steps, before the next collective or kernel that
                   would wait for the peers is launched -- raises ``PeerFailure`` naming the ranks
                   whose counter has not moved for ``max_age_s``.  A rank that leaves on purpose
                   calls ``leave()`` first, which the others report as ``PeerLeft``.
"""
from __future__ import annotations

import faulthandler
import os
import sys
import threading
import time


class PeerFailure(RuntimeError):
    def __init__(self, ranks, reason: str = "no heartbeat"):
        self.ranks = list(ranks)
        super().__init__(f"ranks {self.ranks}: {reason}")


class PeerLeft(PeerFailure):
    def __init__(self, ranks):
        super().__init__(ranks, "left the job")


class StepWatchdog:
    def __init__(self, deadline_s: float, on_timeout=None, poll_s: float | None = None, stream=None):
        self.deadline_s = float(deadline_s)
        self.on_timeout = on_timeout
        self.poll_s = poll_s if poll_s is not None else max(0.05, min(1.0, self.deadline_s / 4))
        self.stream = stream or sys.stderr
        self._last = time.monotonic()
        self._step = -1
        self._stop = threading.Event()
        self._paused = False
        self.fired = False
        self._thread = threading.Thread(target=self._run, name="step-watchdog", daemon=True)

    def start(self):
        self._last = time.monotonic()
        self._thread.start()
        return self

    def beat(self, step: int | None = None):
        self._last = time.monotonic()
        if step is not None:
            self._step = step

    def pause(self):
        """Suspend the deadline (checkpoint writes, evaluation)."""
        self._paused = True

    def resume(self):
        self._last = time.monotonic()
        self._paused = False

    def stop(self):
        self._stop.set()
        if self._thread.is_alive():
            self._thread.join(timeout=2 * self.poll_s + 1.0)

    def __enter__(self):
        return self.start()

    def __exit__(self, *a):
        self.stop()

    def _run(self):
        while not self._stop.wait(self.poll_s):
            if self._paused:
                continue
            late = time.monotonic() - self._last
            if late > self.deadline_s:
                self.fired = True
                self._dump(late)
                if self.on_timeout is not None:
                    self.on_timeout(self._step, late)
                else:  # pragma: no cover - ends the process
                    os._exit(124)
                return

    def _dump(self, late: float):
        try:
            print(f"[watchdog] step {self._step} exceeded its deadline: {late:.1f}s > {self.deadline_s:.1f}s "
                  f"(pid {os.getpid()}, rank {os.environ.get('RANK', '0')})", file=self.stream, flush=True)
            faulthandler.dump_traceback(file=self.stream, all_threads=True)
        except Exception:
            pass


class PeerHeartbeat:
    """Counters in the key-value store, one per rank.  ``store`` is any ``torch.distributed.Store``;
    by default the one the default process group was created with."""

    def __init__(self, rank: int, world: int, store=None, *, interval_s: float = 0.5, max_age_s: float = 5.0,
                 prefix: str = "hb"):
        if store is None:
            import torch.distributed as dist
            from torch.distributed import distributed_c10d as c10d

            store = c10d._get_default_store() if dist.is_initialized() else None
        if store is None:
            raise ValueError("PeerHeartbeat needs a torch.distributed store")
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.interval_s, self.max_age_s, self.prefix = interval_s, max_age_s, prefix
        self._stop = threading.Event()
        self._lock = threading.Lock()
        self._left = False
        self._seen: dict[int, tuple[int, float]] = {}
        self._count = 0
        self._thread = threading.Thread(target=self._run, name="peer-heartbeat", daemon=True)

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def start(self):
        self._publish()
        now = time.monotonic()
        self._seen = {r: (-1, now) for r in range(self.world) if r != self.rank}
        self._thread.start()
        return self

    def _publish(self):
        with self._lock:
            if self._left:       # "left" stays the last word of this rank
                return
            self._count += 1
            self.store.set(self._key(self.rank), str(self._count))

    def _run(self):
        while not self._stop.wait(self.interval_s):
            try:
                self._publish()
            except Exception:
                return

    def leave(self):
        """Announce an orderly exit (between steps, nothing in flight), then stop beating."""
        self._stop.set()
        with self._lock:         # a beat that is being written finishes first and none follows
            self._left = True
            try:
                self.store.set(self._key(self.rank), "left")
            except Exception:
                pass

    def stop(self):
        self._stop.set()
        if self._thread.is_alive():
            self._thread.join(timeout=2 * self.interval_s + 1.0)

    def _read(self, r: int):
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            return self.store.get(self._key(r)).decode()
        except Exception:
            return None

    def check(self):
        """Raise ``PeerLeft`` / ``PeerFailure`` for peers that left or stopped beating."""
        now = time.monotonic()
        left, dead = [], []
        for r in list(self._seen):
            v = self._read(r)
            if v == "left":
                left.append(r)
                continue
            last_v, last_t = self._seen[r]
            cur = int(v) if v is not None else -1
            if cur != last_v:
                self._seen[r] = (cur, now)
            elif now - last_t > self.max_age_s:
                dead.append(r)
        if left:
            raise PeerLeft(left)
        if dead:
            raise PeerFailure(dead, f"no heartbeat for more than {self.max_age_s:.1f}s")

    def wait_all_alive(self, timeout_s: float = 30.0):
        """Block until every peer has published at least once (start-up rendezvous)."""
        t0 = time.monotonic()
        while time.monotonic() - t0 < timeout_s:
            if all(self._read(r) is not None for r in self._seen):
                now = time.monotonic()
                self._seen = {r: (-1, now) for r in self._seen}
                return
            time.sleep(min(0.05, self.interval_s))
        raise PeerFailure([r for r in self._seen if self._read(r) is None], "never joined")
