"""Signal protocols of the peer-memory kernels replayed on the host under random and exhaustive interleavings."""

import pytest

from slime_b200.parallel import protocol_model as pm


def test_barrier_is_safe_under_every_interleaving_of_two_ranks_and_many_of_four():
    def two():
        b = pm.Barrier(2)
        return [iter(_seq(b, r, [1, 2])) for r in range(2)]

    def _seq(b, r, epochs):
        for e in epochs:
            yield from b.run(r, e)

    n = pm.exhaustive_schedules(two, max_schedules=30000)
    assert n > 1000  # two barriers of two ranks: thousands of distinct interleavings, all fine

    def four():
        b = pm.Barrier(4)
        return [iter(_seq(b, r, range(1, 6))) for r in range(4)]

    pm.random_schedules(four, 300, seed=1)
    pm.random_schedules(four, 300, seed=2, bias=0.9)  # one rank starved: the others run up to a barrier ahead of it


def test_barrier_epoch_may_wrap_around():
    start = 0xFFFFFFFE

    def ranks():
        b = pm.Barrier(3, start_epoch=start)

        def seq(r):
            for e in range(start + 1, start + 6):  # crosses 2^32
                yield from b.run(r, e)

        return [iter(seq(r)) for r in range(3)]

    pm.random_schedules(ranks, 200, seed=3, bias=0.8)


def test_a_rank_that_never_arrives_expires_the_wait_and_later_barriers_do_not_wait_again():
    b = pm.Barrier(3)

    def present(r):
        yield from b.run(r, 1, limit=50)
        yield from b.run(r, 2, limit=50)  # status is sticky: announce and return

    ranks = [iter(present(0)), iter(present(1))]  # rank 2 never shows up
    turn = iter(range(10**6))
    trace = pm.run_schedule(ranks, lambda alive: alive[next(turn) % len(alive)])  # round robin
    assert b.status[0] == (1 | (2 << 8)) and b.status[1] == (1 | (2 << 8))  # "waited for peer 2"
    assert len(trace) < 400  # bounded: two expired waits, no further spinning in the second barrier
    assert b.pad[0][1] == 2 and b.pad[1][0] == 2  # the peers were still told about barrier 2


def test_data_parallel_step_needs_both_barriers():
    def make(**kw):
        def ranks():
            st = pm.DataParallelStep(3, **kw)
            return [iter(st.rank(r, 4)) for r in range(3)]

        return ranks

    pm.random_schedules(make(), 300, seed=4)
    pm.random_schedules(make(), 300, seed=5, bias=0.9)
    # mutants: without the leading barrier a rank reduces gradients a peer has not written yet; without the trailing one
    # a fast rank starts the next step on stale parameters or overwrites gradients a peer still reads
    with pytest.raises(pm.ProtocolViolation, match="reads step"):
        pm.random_schedules(make(leading_barrier=False), 300, seed=6, bias=0.9)
    with pytest.raises(pm.ProtocolViolation):
        pm.random_schedules(make(trailing_barrier=False), 300, seed=7, bias=0.9)


def test_scatter_gemm_flags_with_two_alternating_buffers_need_no_barrier():
    def make(**kw):
        def ranks():
            g = pm.ScatterGemm(3, tiles_per_rank=2, **kw)
            return [iter(g.rank(r, 6)) for r in range(3)]

        return ranks

    pm.random_schedules(make(), 300, seed=8)
    pm.random_schedules(make(), 300, seed=9, bias=0.95)
    with pytest.raises(pm.ProtocolViolation, match="was not read yet"):  # a single buffer is refilled under the reader
        pm.random_schedules(make(buffers=1), 300, seed=10, bias=0.95)

    def tiny():
        g = pm.ScatterGemm(2, tiles_per_rank=1)
        return [iter(g.rank(r, 1)) for r in range(2)]

    assert pm.exhaustive_schedules(tiny, max_schedules=30000) > 100


def test_exhaustive_exploration_reports_a_deadlock():
    def ranks():
        b = pm.Barrier(2)

        def only_one(r):
            if r == 0:
                yield from b.run(0, 1)  # rank 1 never announces epoch 1

        return [iter(only_one(r)) for r in range(2)]

    with pytest.raises(pm.ProtocolViolation, match="deadlock"):
        pm.exhaustive_schedules(ranks)
