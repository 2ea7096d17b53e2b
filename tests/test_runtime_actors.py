import time

import pytest

from slime_b200.runtime import actors, object_store
from slime_b200.runtime.testing import Counter, FailingInit


def test_remote_calls_errors_and_death():
    h = Counter.options(env={"SLIME_TEST_FLAG": "7"}).remote(5)
    try:
        assert actors.get([h.add.remote(1), h.add.remote(2)]) == [6, 8]
        assert actors.get(h.env.remote("SLIME_TEST_FLAG")) == "7"
        with pytest.raises(actors.RemoteError, match="nope"):
            actors.get(h.boom.remote())
        assert actors.get(h.add.remote(0)) == 8  # the actor survives an exception in a method
        other = Counter.remote(100)
        assert actors.get(h.call_other.remote(other, 5)) == 105  # handles are picklable: actor-to-actor calls
        ref = h.exit_now.remote()
        with pytest.raises(actors.ActorDiedError):
            actors.get(ref, timeout=10)
        deadline = time.time() + 5
        while h.is_alive() and time.time() < deadline:
            time.sleep(0.01)
        assert not h.is_alive()
        with pytest.raises(actors.ActorDiedError):
            actors.get(h.add.remote(1), timeout=5)
        actors.kill(other)
    finally:
        actors.kill(h)


def test_constructor_failure_and_concurrency_and_wait():
    with pytest.raises(actors.RemoteError, match="constructor failure"):
        FailingInit.remote()
    h = Counter.options(max_concurrency=4).remote(0)
    try:
        t0 = time.time()
        refs = [h.sleep.remote(0.3) for _ in range(4)]
        done, pending = actors.wait(refs, num_returns=4, timeout=5)
        assert len(done) == 4 and time.time() - t0 < 1.0  # ran concurrently
    finally:
        actors.kill(h)


def test_lock_actor_and_object_store():
    lock = actors.Lock.remote()
    try:
        assert actors.get(lock.acquire.remote()) is True
        assert actors.get(lock.acquire.remote()) is False
        actors.get(lock.release.remote())
        with actors.LockClient(lock):
            assert actors.get(lock.acquire.remote()) is False
        assert actors.get(lock.acquire.remote()) is True
    finally:
        actors.kill(lock)
    import torch

    ref = object_store.put({"tokens": [torch.arange(5)], "n": 3})
    back = object_store.get(ref)
    assert back["n"] == 3 and back["tokens"][0].tolist() == [0, 1, 2, 3, 4]
    object_store.free(ref)
