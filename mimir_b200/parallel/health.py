"""Failure detection on the host (the reference has none: its collectives block for ever when a
rank is lost).  Three pieces:

* ``Heartbeat``: every rank publishes a counter in the job's key-value store from a daemon thread;
  ``dead_ranks()`` lists the ranks whose counter has not moved for ``timeout`` seconds.  A rank
  checks it BEFORE it launches a step, so a lost peer is learned on the host and no kernel is
  left waiting on a flag that nothing will set.
* ``Watchdog``: wraps a step; if the step (launch + synchronisation) does not return within the
  limit it records the stall and calls ``on_stall`` (by default it raises in the caller once
  control returns; it never kills a thread or resets a device).
* ``device_status()``: reads the device error word that every native kernel's bounded wait raises
  (wait timeout, peer timeout, index, shape) and turns it into an exception naming the bits.

The in-kernel side is in the kernels themselves: every spin on an mbarrier or on a peer's flag
has a time limit, after which the kernel sets its bit in the error word and returns.
"""
from __future__ import annotations

import threading
import time


class RankLost(RuntimeError):
    def __init__(self, ranks):
        super().__init__(f"ranks {sorted(ranks)} stopped sending heartbeats")
        self.ranks = sorted(ranks)


class StepStalled(RuntimeError):
    pass


class DeviceFault(RuntimeError):
    BITS = {1: "index out of range", 2: "integer division by zero", 4: "wait on a barrier timed out",
            8: "wait on another GPU's flag timed out", 16: "arguments refused"}

    def __init__(self, word: int):
        names = [n for b, n in self.BITS.items() if word & b] or [f"unknown bits {word:#x}"]
        super().__init__("device error word: " + ", ".join(names))
        self.word = word


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval: float = 0.2, timeout: float = 2.0, prefix: str = "hb"):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.prefix = interval, timeout, prefix
        self._stop = threading.Event()
        self._seen = {}      # rank -> (value, time it last changed)
        self._count = 0
        self._beat()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _beat(self):
        self._count += 1
        self.store.set(f"{self.prefix}/{self.rank}", str(self._count))

    def _run(self):
        while not self._stop.wait(self.interval):
            try:
                self._beat()
            except Exception:      # the store went away: nothing more to publish
                return

    def dead_ranks(self) -> list:
        now, dead = time.monotonic(), []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                v = self.store.get(f"{self.prefix}/{r}")
            except Exception:
                v = None
            last = self._seen.get(r)
            if last is None or last[0] != v:
                self._seen[r] = (v, now)
            elif v is None or now - last[1] > self.timeout:
                dead.append(r)
        return dead

    def check(self) -> None:
        """Raises ``RankLost`` if a peer has been silent for longer than the timeout."""
        dead = self.dead_ranks()
        if dead:
            raise RankLost(dead)

    def wait_all(self, limit: float = 30.0) -> None:
        """Blocks until every rank has published at least one beat (start of the job)."""
        t0 = time.monotonic()
        while time.monotonic() - t0 < limit:
            try:
                for r in range(self.world):
                    self.store.get(f"{self.prefix}/{r}")
                return
            except Exception:
                time.sleep(0.05)
        raise RankLost([r for r in range(self.world) if r != self.rank])

    def stop(self) -> None:
        self._stop.set()
        self._thread.join(2 * self.interval + 1)


class Watchdog:
    """``with Watchdog(5.0) as w: step()``; ``w.stalled`` tells whether the limit passed while the
    body ran; leaving the block then raises ``StepStalled`` (or calls ``on_stall`` at once)."""

    def __init__(self, limit: float, on_stall=None):
        self.limit, self.on_stall, self.stalled = limit, on_stall, False
        self._timer = None

    def _fire(self):
        self.stalled = True
        if self.on_stall is not None:
            self.on_stall()

    def __enter__(self):
        self.stalled = False
        self._timer = threading.Timer(self.limit, self._fire)
        self._timer.daemon = True
        self._timer.start()
        return self

    def __exit__(self, exc_type, exc, tb):
        self._timer.cancel()
        if self.stalled and exc_type is None and self.on_stall is None:
            raise StepStalled(f"step took longer than {self.limit} s")
        return False


def device_status(clear: bool = True) -> None:
    """Raises ``DeviceFault`` if a native kernel raised a bit in the device error word."""
    from .. import _native
    word = int(_native.lib().mimir_error_word(1 if clear else 0))
    if word:
        raise DeviceFault(word)


def guarded_step(step, heartbeat: Heartbeat | None = None, limit: float | None = None):
    """Runs ``step()`` the safe way: peers are checked on the host first, the step runs under a
    watchdog, and the device error word is read afterwards."""
    if heartbeat is not None:
        heartbeat.check()
    if limit is None:
        out = step()
    else:
        with Watchdog(limit):
            out = step()
    try:
        device_status()
    except (OSError, AttributeError):   # no native library on this host (CPU-only run)
        pass
    return out
