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
``wait_readers`` step removed it reports the write-while-read race.  The two-shot all-reduce of the DDP buckets
(``check_allreduce_protocol``) and the weight shards / gather slots / "weights published" flag of FSDP
(``check_weight_gather_protocol``) are replayed the same way, each with a switch that removes one wait so that the
test can see the checker find the race that the wait prevents.
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
    return _run(programs, lambda r, row: w.flags[r][row], rng, max_events)


# ----------------------------------------------------------------------------------------------------------------
# The same replay for the two other flag protocols of the package.  `_run` is the scheduler shared by all three.

def _run(programs, flag_rows, rng, max_events: int) -> int:
    """Interleave the rank programs at random.  A program yields ("wait", row, epoch) while the minimum of its own
    copy of flag row ``row`` (``flag_rows(rank, row)``) is below ``epoch``, and ("step",) after any other event."""
    alive = list(range(len(programs)))
    blocked: dict[int, tuple] = {}
    events = 0
    while alive:
        runnable = [r for r in alive if r not in blocked or min(flag_rows(r, blocked[r][1])) >= blocked[r][2]]
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


def check_allreduce_protocol(world: int = 4, buckets: int = 2, steps: int = 3, seed: int = 0,
                             wait_for_pushes: bool = True, max_events: int = 1_000_000) -> int:
    """Two-shot in-place all-reduce of DDP gradient buckets (``peer_allreduce_kernel``).

    Every rank holds the whole bucket; rank r owns chunk r: it waits for every peer's ``ready`` flag, reads chunk r
    of every peer, and pushes the mean into chunk r of every peer, then signals ``done`` and waits for every peer's
    ``done`` before the kernel ends (``wait_for_pushes``), because only then are all chunks of its own buffer
    reduced.  Checked: a chunk is read only while it holds this epoch's local gradients, the optimizer (the next
    event on the stream) sees only reduced chunks, and the next backward never overwrites a chunk that a peer is
    still reading or has not pushed to yet."""
    rng = random.Random(seed)
    LOCAL, REDUCED = 0, 1
    # state[rank][bucket][chunk] = (epoch, LOCAL | REDUCED); readers[rank][bucket][chunk] = peers reading it now
    state = [[[(0, REDUCED)] * world for _ in range(buckets)] for _ in range(world)]
    readers = [[[0] * world for _ in range(buckets)] for _ in range(world)]
    flags = [[[0] * world for _ in range(2 * buckets)] for _ in range(world)]

    def program(rank):
        for epoch in range(1, steps + 1):
            for b in range(buckets):
                ready_row, done_row = 2 * b, 2 * b + 1
                # backward writes this rank's copy of the bucket (stream order after the previous kernel on it)
                for c in range(world):
                    if readers[rank][b][c]:
                        raise ProtocolViolation(f"rank {rank} overwrites chunk {c} of bucket {b} while it is being read")
                    if state[rank][b][c] != (epoch - 1, REDUCED):
                        raise ProtocolViolation(f"rank {rank} starts epoch {epoch} on bucket {b} before chunk {c} of the "
                                                f"previous all-reduce arrived ({state[rank][b][c]})")
                    state[rank][b][c] = (epoch, LOCAL)
                yield ("step",)
                for p in range(world):
                    flags[p][ready_row][rank] = epoch
                yield ("step",)
                while min(flags[rank][ready_row]) < epoch:
                    yield ("wait", ready_row, epoch)
                for p in range(world):                          # read my chunk everywhere
                    if state[p][b][rank] != (epoch, LOCAL):
                        raise ProtocolViolation(f"rank {rank} reads chunk {rank} of rank {p} holding {state[p][b][rank]}")
                    readers[p][b][rank] += 1
                    yield ("step",)
                for p in range(world):                          # push the mean everywhere
                    readers[p][b][rank] -= 1
                    state[p][b][rank] = (epoch, REDUCED)
                    yield ("step",)
                for p in range(world):
                    flags[p][done_row][rank] = epoch
                yield ("step",)
                if wait_for_pushes:
                    while min(flags[rank][done_row]) < epoch:
                        yield ("wait", done_row, epoch)
                # the optimizer consumes the bucket next
                for c in range(world):
                    if state[rank][b][c] != (epoch, REDUCED):
                        raise ProtocolViolation(f"rank {rank} consumes bucket {b} of epoch {epoch} but chunk {c} is "
                                                f"{state[rank][b][c]}")
                yield ("step",)

    return _run([program(r) for r in range(world)], lambda r, row: flags[r][row], rng, max_events)


def check_weight_gather_protocol(world: int = 4, units: int = 3, steps: int = 3, seed: int = 0,
                                 await_weights: bool = True, fused_update: bool = True, slots: int = 2,
                                 max_events: int = 1_000_000) -> int:
    """FSDP weight shards, their gathers and the gather-slot pool over whole training steps.

    Per step every rank pulls every unit's shards from all peers twice (forward in unit order, backward in reverse)
    into ``slots`` local buffers used in turn, then updates its own shard of each unit: inside the unit's
    reduce-scatter once every peer has signalled ``ready`` for it (``fused_update``), or after all reduce-scatters.
    After its last update a rank publishes the weights flag; the next step starts with ``await_weights``.
    Checked: a gather of step s reads shards of exactly version s - 1 and never overlaps an update of them; a
    gather slot is not refilled while its previous occupant is still the weights of the block being computed."""
    rng = random.Random(seed)
    version = [[0] * units for _ in range(world)]           # version[rank][unit] of the rank's own shard
    readers = [[0] * units for _ in range(world)]
    rows_ready = lambda u: 1 + u                              # row 0: weights published
    flags = [[[0] * world for _ in range(1 + units)] for _ in range(world)]
    slot_owner = [[None] * slots for _ in range(world)]      # (unit, in_use) per local gather buffer

    def gather(rank, u, step):
        s = u % slots
        if slot_owner[rank][s] is not None and slot_owner[rank][s][1]:
            raise ProtocolViolation(f"rank {rank} refills gather slot {s} while unit {slot_owner[rank][s][0]} computes from it")
        slot_owner[rank][s] = (u, True)
        for p in range(world):
            if version[p][u] != step - 1:
                raise ProtocolViolation(f"rank {rank} gathers unit {u} of rank {p} in step {step}: version {version[p][u]}")
            readers[p][u] += 1
            yield ("step",)
        for p in range(world):
            if version[p][u] != step - 1:
                raise ProtocolViolation(f"shard of unit {u} on rank {p} changed while rank {rank} gathered it")
            readers[p][u] -= 1
            yield ("step",)

    def update(rank, u, step):
        if readers[rank][u]:
            raise ProtocolViolation(f"rank {rank} updates its shard of unit {u} while {readers[rank][u]} peer(s) gather it")
        version[rank][u] = step

    def program(rank):
        for step in range(1, steps + 1):
            if await_weights and step > 1:
                while min(flags[rank][0]) < step - 1:
                    yield ("wait", 0, step - 1)
            for u in range(units):                                       # forward
                yield from gather(rank, u, step)
                slot_owner[rank][u % slots] = (u, False)                 # released after the block's forward
                yield ("step",)
            for u in reversed(range(units)):                             # backward
                yield from gather(rank, u, step)
                slot_owner[rank][u % slots] = (u, False)
                for p in range(world):                                   # reduce-scatter of unit u: ready handshake
                    flags[p][rows_ready(u)][rank] = step
                yield ("step",)
                while min(flags[rank][rows_ready(u)]) < step:
                    yield ("wait", rows_ready(u), step)
                if fused_update:
                    update(rank, u, step)
                    yield ("step",)
            if not fused_update:
                for u in range(units):
                    update(rank, u, step)
                    yield ("step",)
            for p in range(world):                                       # publish: my shards are final for step + 1
                flags[p][0][rank] = step
            yield ("step",)

    return _run([program(r) for r in range(world)], lambda r, row: flags[r][row], rng, max_events)
