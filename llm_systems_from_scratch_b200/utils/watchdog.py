"""Host-side failure detection: store-based heartbeats, a per-rank watchdog thread and a
step-boundary health check.

The reference has no failure handling (a crashed child only surfaces through ``mp.spawn(join=True)``,
train.py:337-342, and collectives wait for the NCCL default timeout).  Here every rank publishes a
heartbeat (monotonic counter + wall time) in a ``torch.distributed`` key-value store from a daemon
thread.  ``check()`` is called between steps, when no kernel or collective of this rank is in
flight: it raises ``RankFailure`` naming the silent ranks *before* the next launch, so the caller
can stop cleanly and restart from the last checkpoint (restart-from-checkpoint on any world size
is the recovery story).  Device-side waits are bounded separately: a kernel that gives up writes a
status word which ``ops.native.check_status`` turns into an exception.

Failures are injected on the host only (a rank that exits, raises or stops beating); nothing here
faults, traps or hangs a GPU.
"""
from __future__ import annotations

import threading
import time


class RankFailure(RuntimeError):
    def __init__(self, dead: list[int], detail: str = ""):
        super().__init__(f"ranks {dead} stopped responding{': ' + detail if detail else ''}")
        self.dead = dead


class Heartbeat:
    """Publishes ``hb/{rank}`` = "<counter>:<unix time>" every ``interval`` seconds."""

    def __init__(self, store, rank: int, world_size: int, interval: float = 0.5, timeout: float = 5.0,
                 clock=time.time):
        self.store, self.rank, self.world_size = store, rank, world_size
        self.interval, self.timeout, self.clock = interval, timeout, clock
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._count = 0
        self._paused = False
        self._seen: set[int] = set()      # peers whose heartbeat key has been read at least once
        self.beat()

    def beat(self):
        self._count += 1
        self.store.set(f"hb/{self.rank}", f"{self._count}:{self.clock():.3f}")

    def start(self):
        if self._thread is None:
            self._thread = threading.Thread(target=self._run, daemon=True, name=f"heartbeat-{self.rank}")
            self._thread.start()
        return self

    def _run(self):
        while not self._stop.wait(self.interval):
            if not self._paused:
                try:
                    self.beat()
                except Exception:
                    return   # store gone: the job is shutting down

    def pause(self, flag: bool = True):
        """Fault injection on the host: a paused rank looks dead to its peers."""
        self._paused = flag

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)

    def mark_done(self):
        """A rank that finished normally is not a failure."""
        self.store.set(f"hb/{self.rank}", f"done:{self.clock():.3f}")

    def silent_ranks(self) -> list[int]:
        now = self.clock()
        dead = []
        for r in range(self.world_size):
            if r == self.rank:
                continue
            key = f"hb/{r}"
            try:
                # A peer seen before whose key is gone (dropped from the store) is reported at once: `get` on a torch
                # store would wait for the key up to the store's own timeout, `check` answers immediately.  A peer
                # not seen yet is still starting up; for it the wait inside `get` is the start-up rendezvous.
                probe = getattr(self.store, "check", None)
                if r in self._seen and probe is not None and not probe([key]):
                    dead.append(r)
                    continue
                raw = self.store.get(key).decode()
                self._seen.add(r)
            except Exception:
                dead.append(r)
                continue
            tag, stamp = raw.split(":")
            if tag != "done" and now - float(stamp) > self.timeout:
                dead.append(r)
        return dead

    def check(self):
        """Raise ``RankFailure`` if a peer's heartbeat is older than ``timeout``.  Call between steps."""
        dead = self.silent_ranks()
        if dead:
            raise RankFailure(dead, f"no heartbeat for more than {self.timeout}s")


class StepWatchdog:
    """Flags a step that runs longer than ``limit`` seconds (a stuck collective, a hung peer).

    ``arm()`` at step start, ``disarm()`` at step end; ``on_timeout`` runs on the watchdog thread and
    defaults to recording the event, which ``expired`` exposes to the training loop.
    """

    def __init__(self, limit: float, on_timeout=None):
        self.limit = limit
        self.on_timeout = on_timeout
        self.expired = False
        self._deadline = None
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True, name="step-watchdog")
        self._thread.start()

    def arm(self):
        with self._lock:
            self._deadline = time.monotonic() + self.limit

    def disarm(self):
        with self._lock:
            self._deadline = None

    def _run(self):
        while not self._stop.wait(min(0.05, self.limit / 4)):
            with self._lock:
                hit = self._deadline is not None and time.monotonic() > self._deadline
                if hit:
                    self._deadline = None
            if hit:
                self.expired = True
                if self.on_timeout is not None:
                    self.on_timeout()

    def stop(self):
        self._stop.set()
        self._thread.join(timeout=1)
