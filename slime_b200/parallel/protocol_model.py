"""Executable model of the signal protocols of the peer-memory kernels, for checking them under arbitrary interleavings.

The kernels in ``csrc/dp_fused.cu``, ``csrc/tp_fused.cu`` and the collective modes of ``csrc/gemm_sm100.cu`` coordinate
GPUs with words in each other's memory: a writer stores data, then a flag with release semantics; a reader spins on the
flag with acquire semantics and then reads the data. Whether such a protocol is right does not depend on timing but on
the order of those few memory operations, so it can be replayed on the host: every rank is a Python generator that
yields before each shared-memory operation, a scheduler picks which rank moves next (at random, or exhaustively for
small cases), and every read checks that it sees the version of the data it is supposed to see. A protocol error shows
up as ``ProtocolViolation`` with the schedule that produced it; a mutant of the protocol (a barrier left out) must be
caught, which is how the tests show that the checker has teeth.

Modelled: the epoch barrier (``symm_barrier_kernel``: rank r stores ``epoch`` into word ``r`` of every peer's pad, then
waits until all words of its own pad have reached ``epoch``, compared as a signed 32-bit difference so that the counter
may wrap), its bounded wait with the sticky status word, the data-parallel step built on it (write gradients ->
barrier -> read every peer's gradients of my shard -> write my shard of the parameters into every peer -> barrier), and
the per-tile flags of the reduce-scatter GEMM (a tile is stored into its owner's slot, then its flag is raised to the
call's epoch; the owner reads a slot only after the flag; receive buffers and flag sets alternate between two copies, which
is what lets a slot be refilled without a barrier between calls).
"""

from __future__ import annotations

import random


class ProtocolViolation(AssertionError):
    pass


BLOCKED = "blocked"  # yielded by a rank whose last poll of a flag failed: it changes nothing until another rank moves


def _i32(x: int) -> int:
    x &= 0xFFFFFFFF
    return x - (1 << 32) if x & 0x80000000 else x


class Barrier:
    """State of the epoch barrier: ``pad[r][p]`` = last epoch rank p announced in rank r's pad."""

    def __init__(self, world: int, start_epoch: int = 0):
        self.world = world
        self.pad = [[start_epoch & 0xFFFFFFFF] * world for _ in range(world)]
        self.status = [0] * world  # sticky error word per rank
        self.entered = [start_epoch] * world  # bookkeeping for the safety check (not part of the protocol)

    def run(self, rank: int, epoch: int, limit: int | None = None):
        """Generator: one barrier of ``rank`` at ``epoch``. ``limit``: spins after which the wait gives up."""
        self.entered[rank] = epoch
        failed = self.status[rank] != 0
        for p in range(self.world):
            yield  # st.release.sys into peer p's pad
            self.pad[p][rank] = epoch & 0xFFFFFFFF
        if failed:
            return  # an earlier wait expired: announce, do not wait again
        for p in range(self.world):
            spins = 0
            while True:
                yield BLOCKED if spins else None  # ld.acquire.sys from my own pad
                if _i32(self.pad[rank][p] - epoch) >= 0:
                    break
                spins += 1
                if limit is not None and spins > limit:
                    if self.status[rank] == 0:
                        self.status[rank] = 1 | (p << 8)
                    break
        if self.status[rank] == 0:
            late = [q for q in range(self.world) if _i32(self.entered[q] - epoch) < 0]
            if late:
                raise ProtocolViolation(f"rank {rank} left barrier {epoch} before ranks {late} entered it")


def run_schedule(ranks: list, choose) -> list[int]:
    """Advance the rank generators until all are done; ``choose(alive) -> index`` picks who moves. Returns the schedule."""
    alive = list(range(len(ranks)))
    trace = []
    while alive:
        r = choose(alive)
        trace.append(r)
        try:
            next(ranks[r])
        except StopIteration:
            alive.remove(r)
    return trace


def random_schedules(make_ranks, n: int, seed: int = 0, bias: float = 0.0):
    """Run ``n`` random interleavings. ``bias`` > 0 makes one rank (rotating) that much likelier to be starved, which
    produces the lopsided arrival orders that expose ordering bugs."""
    rng = random.Random(seed)
    for k in range(n):
        ranks = make_ranks()
        slow = k % len(ranks)

        def choose(alive, slow=slow):
            if bias and len(alive) > 1 and slow in alive and rng.random() < bias:
                return rng.choice([a for a in alive if a != slow])
            return rng.choice(alive)

        try:
            run_schedule(ranks, choose)
        except ProtocolViolation as e:
            raise ProtocolViolation(f"schedule {k} (seed {seed}): {e}") from None


def exhaustive_schedules(make_ranks, max_schedules: int | None = None) -> int:
    """Every interleaving of a small case, depth-first over the choice at each step; returns how many were run (at most
    ``max_schedules``). A rank whose poll just failed is not offered again until another rank has moved (polling twice
    in a row sees the same memory), which keeps the tree finite; if every live rank is in that state the protocol has
    deadlocked. Waits must be unbounded (``limit=None``) here: an expiring wait makes progress by itself."""

    def replay(prefix):
        ranks = make_ranks()
        alive, blocked = list(range(len(ranks))), set()
        for r in prefix:
            step(ranks, alive, blocked, r)
        return ranks, alive, blocked

    def step(ranks, alive, blocked, r):
        try:
            tag = next(ranks[r])
        except StopIteration:
            alive.remove(r)
            tag = None
        if tag == BLOCKED:
            blocked.add(r)
        else:  # the rank performed an operation: the others may see something new
            blocked.clear()

    count = 0
    stack = [[]]  # prefixes of choices still to extend
    while stack:
        if max_schedules is not None and count >= max_schedules:
            break
        path = stack.pop()
        ranks, alive, blocked = replay(path)
        while alive:
            ready = [a for a in alive if a not in blocked]
            if not ready:
                raise ProtocolViolation(f"deadlock: ranks {alive} all wait on flags nobody will raise (schedule {path})")
            for alt in ready[1:]:
                stack.append(path + [alt])
            path = path + [ready[0]]
            step(ranks, alive, blocked, ready[0])
        count += 1
    return count


# ------------------------------------------------------------------------------------------- data-parallel step
class DataParallelStep:
    """Versions instead of values: ``grads[r]`` = step whose gradients rank r's buffer holds, ``params[r][s]`` = step
    whose update shard s of rank r's parameter buffer holds."""

    def __init__(self, world: int, trailing_barrier: bool = True, leading_barrier: bool = True):
        self.world, self.trailing, self.leading = world, trailing_barrier, leading_barrier
        self.bar = Barrier(world)
        self.grads = [-1] * world
        self.params = [[-1] * world for _ in range(world)]

    def rank(self, r: int, steps: int):
        epoch = 0
        for s in range(steps):
            if s > 0:  # forward / backward of step s read the parameters of step s - 1 ...
                for shard in range(self.world):
                    yield
                    if self.params[r][shard] != s - 1:
                        raise ProtocolViolation(f"rank {r} starts step {s} with shard {shard} of step {self.params[r][shard]}")
            yield  # ... and overwrite the gradient buffer
            self.grads[r] = s
            if self.leading:
                epoch += 1
                yield from self.bar.run(r, epoch)
            for p in range(self.world):  # reduce my shard: read it from every rank
                yield
                if self.grads[p] != s:
                    raise ProtocolViolation(f"rank {r} reduces step {s} but reads step {self.grads[p]} gradients of rank {p}")
            for p in range(self.world):  # Adam on my shard, stored into every rank's parameter buffer
                yield
                self.params[p][r] = s
            if self.trailing:
                epoch += 1
                yield from self.bar.run(r, epoch)


# ------------------------------------------------------------------------------------- reduce-scatter GEMM flags
class ScatterGemm:
    """The fused GEMM -> reduce-scatter of ``parallel/fused_tp.py``: writer w stores its partial tile t for owner o into
    o's receive buffer and then raises that tile's flag to the call's epoch; the owner waits for the flag and reads.
    There is no barrier between calls: receive buffers and flag sets alternate between two copies, and a writer that
    refills copy b in call c + 2 has waited, in call c + 1, for a flag every owner raises only after finishing call c.
    ``buffers=1`` is the mutant without that alternation."""

    def __init__(self, world: int, tiles_per_rank: int = 2, buffers: int = 2):
        self.world, self.tiles, self.buffers = world, tiles_per_rank, buffers
        mk = lambda v: [[[[v] * tiles_per_rank for _ in range(world)] for _ in range(world)] for _ in range(buffers)]  # noqa: E731
        self.slot, self.flag, self.consumed = mk(-1), mk(0), mk(-1)  # indexed [buffer][owner][writer][tile]

    def rank(self, r: int, calls: int):
        epochs = [0] * self.buffers
        for c in range(calls):
            b = c % self.buffers
            epochs[b] += 1
            epoch = epochs[b]
            for t in range(self.tiles):  # owners interleaved along the tile walk
                for o in range(self.world):
                    yield  # TMA store of the tile into the owner's slot (complete before the flag: wait_group + fence)
                    held = self.slot[b][o][r][t]
                    if held >= 0 and self.consumed[b][o][r][t] < held:
                        raise ProtocolViolation(f"writer {r} refills a slot of owner {o} in call {c} whose call-{held} tile was not read yet")
                    self.slot[b][o][r][t] = c
                    yield  # st.release.sys of the flag
                    self.flag[b][o][r][t] = epoch
            for t in range(self.tiles):  # phase 2: sum my tiles over the writers, in rank order
                for w in range(self.world):
                    polled = False
                    while True:
                        yield BLOCKED if polled else None  # ld.acquire.sys
                        if _i32(self.flag[b][r][w][t] - epoch) >= 0:
                            break
                        polled = True
                    yield
                    if self.slot[b][r][w][t] != c:
                        raise ProtocolViolation(f"owner {r} sums call {c} but the slot of writer {w} holds call {self.slot[b][r][w][t]}")
                    self.consumed[b][r][w][t] = c
