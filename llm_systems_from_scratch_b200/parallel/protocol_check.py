"""Host-side model checker for the flag protocol of the peer-memory collectives.

The device kernels (``csrc/comm_kernels.cu``) synchronise ranks with epoch-numbered flags in peer memory:
a rank *signals* by storing the epoch into its slot of a flag row on every peer, and *waits* until every
slot of its own copy of the row holds at least that epoch.  Each logical staging buffer owns two rows:

* ``ready``  "my staging for this unit is complete"            (signalled at the start of the reduce-scatter)
* ``done``   "I no longer read anybody's staging for this unit" (signalled by the last CTA to finish)

and the producer of a staging buffer waits on ``done`` (``PeerComm.wait_readers``) before it overwrites it.

A GPU cannot be asked to exhibit a race on demand, so the protocol is replayed here on the host: every rank is
a coroutine that performs the same sequence of signal / wait / read / write events as the kernels, a scheduler
interleaves the ranks at random (any rank that is not blocked may take the next event), and the checker asserts
the two safety properties that the device code relies on

1. a rank reads peer p's staging of unit u in epoch e only after p wrote it for epoch e and before p writes it
   for epoch e+1;
2. every wait is eventually satisfied (no schedule deadlocks).

``tests/test_parallel_cpu.py`` runs many random schedules and also checks that the checker has teeth: with the
``wait_readers`` step removed it reports the write-while-read race.
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field


class ProtocolViolation(AssertionError):
    pass


@dataclass
class _World:
    world: int
    units: int
    # flags[rank][row][slot]: rank's local copy of a flag row; slot p is written by rank p
    flags: list = field(default_factory=list)
    # version[rank][unit]: epoch whose gradients the rank's staging buffer currently holds (0 = nothing yet)
    version: list = field(default_factory=list)
    # readers[rank][unit]: number of peers currently in the middle of reading this staging buffer
    readers: list = field(default_factory=list)

    def __post_init__(self):
        rows = 2 * self.units
        self.flags = [[[0] * self.world for _ in range(rows)] for _ in range(self.world)]
        self.version = [[0] * self.units for _ in range(self.world)]
        self.readers = [[0] * self.units for _ in range(self.world)]


def _rank_program(w: _World, rank: int, steps: int, use_wait_readers: bool):
    """Generator of one rank's events.  Yields ("wait", row, epoch) while blocked and ("step",) after an event."""
    for step in range(1, steps + 1):
        epoch = step
        for u in range(w.units):
            ready_row, done_row = 2 * u, 2 * u + 1
            # -- backward of unit u writes this rank's staging; before that, everybody must be done reading it
            if use_wait_readers and epoch > 1:
                while min(w.flags[rank][done_row]) < epoch - 1:
                    yield ("wait", done_row, epoch - 1)
            if w.readers[rank][u] != 0:
                raise ProtocolViolation(f"rank {rank} overwrites staging of unit {u} (epoch {epoch}) while "
                                        f"{w.readers[rank][u]} peer(s) still read it")
            w.version[rank][u] = epoch
            yield ("step",)
            # -- reduce-scatter kernel: signal ready, wait for all, read every peer's slice, signal done
            for p in range(w.world):
                w.flags[p][ready_row][rank] = epoch
            yield ("step",)
            while min(w.flags[rank][ready_row]) < epoch:
                yield ("wait", ready_row, epoch)
            for p in range(w.world):                      # begin reading: one event per peer, interleavable
                if w.version[p][u] != epoch:
                    raise ProtocolViolation(f"rank {rank} reads unit {u} of rank {p} in epoch {epoch} but the "
                                            f"buffer holds epoch {w.version[p][u]}")
                w.readers[p][u] += 1
                yield ("step",)
            for p in range(w.world):                      # finish reading
                if w.version[p][u] != epoch:
                    raise ProtocolViolation(f"staging of unit {u} on rank {p} changed to epoch {w.version[p][u]} "
                                            f"while rank {rank} was reading epoch {epoch}")
                w.readers[p][u] -= 1
                yield ("step",)
            for p in range(w.world):
                w.flags[p][done_row][rank] = epoch
            yield ("step",)


def check_reduce_scatter_protocol(world: int = 4, units: int = 3, steps: int = 3, seed: int = 0,
                                  use_wait_readers: bool = True, max_events: int = 1_000_000) -> int:
    """Run one random interleaving; returns the number of events.  Raises ``ProtocolViolation`` on a race or a
    deadlock."""
    rng = random.Random(seed)
    w = _World(world, units)
    programs = [_rank_program(w, r, steps, use_wait_readers) for r in range(world)]
    alive = list(range(world))
    blocked: dict[int, tuple] = {}
    events = 0
    while alive:
        # a blocked rank may run again only when its wait could pass; picking it earlier just re-yields the wait
        runnable = [r for r in alive if r not in blocked or min(w.flags[r][blocked[r][1]]) >= blocked[r][2]]
        if not runnable:
            raise ProtocolViolation(f"deadlock: ranks {sorted(blocked)} wait on {blocked}")
        r = rng.choice(runnable)
        try:
            ev = next(programs[r])
        except StopIteration:
            alive.remove(r)
            blocked.pop(r, None)
            continue
        if ev[0] == "wait":
            blocked[r] = ev
        else:
            blocked.pop(r, None)
        events += 1
        if events > max_events:
            raise ProtocolViolation("schedule did not terminate")
    return events
