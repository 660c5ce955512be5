"""Failure detection on the host: a rank that stops, a step that stalls, a raised error word.
No GPU is involved: the lost rank is a process that exits between steps."""
import multiprocessing as mp
import time
from datetime import timedelta

import pytest
import torch.distributed as dist

from mimir_b200.parallel import health


def _rank(rank, world, port, quit_after, q):
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=20),
                          wait_for_workers=False)
    hb = health.Heartbeat(store, rank, world, interval=0.05, timeout=0.5)
    hb.wait_all(10)
    steps, lost = 0, None
    t0 = time.monotonic()
    while time.monotonic() - t0 < 6:
        if quit_after is not None and steps >= quit_after:
            hb.stop()                 # leaves between steps: nothing of it is in flight
            q.put((rank, "left", steps))
            return
        try:
            health.guarded_step(lambda: time.sleep(0.02), hb)
        except health.RankLost as e:
            lost = e.ranks
            break
        steps += 1
    hb.stop()
    q.put((rank, lost, steps))
    if rank == 0:
        time.sleep(1.0)               # the store's owner outlives the others' last reads


def test_lost_rank_is_learned_on_the_host_before_the_next_step():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 3, 29921, 5 if r == 2 else None, q)) for r in range(3)]
    for p in procs:
        p.start()
    out = dict((r, (what, steps)) for r, what, steps in (q.get(timeout=60) for _ in range(3)))
    for p in procs:
        p.join(20)
    assert out[2][0] == "left"
    assert out[0][0] == [2] and out[1][0] == [2]
    assert out[0][1] >= 5          # the survivors kept stepping until the heartbeat went quiet


def test_watchdog_and_error_word_decoding():
    with health.Watchdog(1.0) as w:
        time.sleep(0.01)
    assert not w.stalled
    with pytest.raises(health.StepStalled):
        with health.Watchdog(0.05):
            time.sleep(0.2)
    fired = []
    with health.Watchdog(0.05, on_stall=lambda: fired.append(1)):
        time.sleep(0.2)
    assert fired == [1]
    e = health.DeviceFault(8 | 4)
    assert "another GPU" in str(e) and "barrier" in str(e) and e.word == 12


def test_phase_timer_on_host():
    from mimir_b200.utils.phases import PhaseTimer
    t = PhaseTimer()
    for _ in range(3):
        with t.phase("forward"):
            time.sleep(0.01)
        with t.phase("backward"):
            time.sleep(0.02)
    rep = t.report()
    assert rep["forward"]["calls"] == 3 and 25 < rep["forward"]["ms"] < 200
    assert rep["backward"]["ms"] > rep["forward"]["ms"]
    off = PhaseTimer(enabled=False)
    with off.phase("x"):
        pass
    assert off.report() == {}
