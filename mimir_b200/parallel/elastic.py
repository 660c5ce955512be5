"""Recovery after a lost rank: the other half of failure detection (``parallel/health.py``).

The reference has no elastic path (a lost device blocks its collectives for ever).  Here a rank
learns on the HOST that a peer is gone (``Heartbeat.check`` raises ``RankLost`` before the next
launch, or a bounded in-kernel wait raised the device error word and ``guarded_step`` turned it
into ``DeviceFault``), and the survivors then:

1. drop what was shared with the old group: peer-memory mappings (``SymmetricBuffer`` and the
   objects built on it expose ``close``), captured CUDA graphs that point into them, the old
   process group (destroyed without a collective: nobody waits for the lost rank);
2. agree on the new, smaller group through the job's key-value store (the survivors keep their
   relative order; the store's host, rank 0 of the job, must be among them) and initialise a
   new process group under a fresh key prefix;
3. reload the last complete checkpoint (``checkpoint.mim`` is written atomically, so it is
   always a whole step) into model and optimizer, and go on from its step counter.

Nothing here touches a GPU's state beyond freeing this process's own mappings: no device
reset, no fault injection.  The test (``tests/test_elastic.py``) runs it on CPU ranks (gloo): a
rank leaves between two steps with nothing in flight, the others shrink the group, resume, and
end with the weights of an uninterrupted run.
"""
from __future__ import annotations

import torch.distributed as dist

from . import health


def detect(heartbeat, wait: float = 3.0, poll: float = 0.1) -> list:
    """Ranks whose heartbeat has gone quiet, polling for up to ``wait`` seconds: what to call when a
    collective ended with an error (a short process-group timeout, a closed connection) and the
    cause may be a peer that left."""
    import time
    t0 = time.monotonic()
    while True:
        dead = heartbeat.dead_ranks()
        if dead or time.monotonic() - t0 > wait:
            return dead
        time.sleep(poll)


def shrink_group(store, rank: int, world: int, dead, backend: str = "gloo", generation: int = 1, timeout=None):
    """Replaces the default process group by one of the surviving ranks.  Returns ``(new_rank,
    new_world)``; the survivors keep their order.  ``generation`` must increase with every shrink
    (it names the key prefix of the new rendezvous)."""
    dead = set(dead)
    if rank in dead:
        raise health.RankLost([rank])
    if 0 in dead:
        raise health.RankLost(sorted(dead))       # the store's host is gone: the job cannot regroup
    alive = [r for r in range(world) if r not in dead]
    if dist.is_initialized():
        # no barrier and no collective: the lost rank would never join it
        dist.destroy_process_group()
    prefix = dist.PrefixStore(f"gen{generation}", store)
    kw = {} if timeout is None else {"timeout": timeout}
    dist.init_process_group(backend, store=prefix, rank=alive.index(rank), world_size=len(alive), **kw)
    return alive.index(rank), len(alive)


def recover(store, rank: int, world: int, dead, model, opt, checkpoint_dir: str, backend: str = "gloo",
            generation: int = 1, shared=(), timeout=None):
    """The whole recovery: close ``shared`` (objects with a ``close`` method that hold peer
    mappings; their ``close`` must not wait for peers), shrink the group, reload the checkpoint.
    Returns ``(new_rank, new_world, training)`` where ``training`` is the checkpoint's Training
    section (``steps``, ``epochs``, ``lr``) or None when no checkpoint exists yet."""
    from ..train.fit import load_checkpoint
    for obj in shared:
        try:
            obj.close()
        except Exception:  # noqa: BLE001 - a mapping that is already gone is not an error here
            pass
    new_rank, new_world = shrink_group(store, rank, world, dead, backend, generation, timeout)
    opt.zero_grad()
    training = load_checkpoint(checkpoint_dir, model, opt)
    return new_rank, new_world, training
