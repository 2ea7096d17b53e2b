"""Small actors used by the test-suite and by fault-injection runs (host-side failures only)."""

from __future__ import annotations

import os
import time

from slime_b200.runtime import actors


@actors.remote
class Counter:
    def __init__(self, start: int = 0):
        self.v = start

    def add(self, n: int) -> int:
        self.v += n
        return self.v

    def boom(self):
        raise ValueError("nope")

    def pid(self) -> int:
        return os.getpid()

    def env(self, key: str):
        return os.environ.get(key)

    def sleep(self, s: float) -> float:
        time.sleep(s)
        return s

    def exit_now(self, code: int = 3):
        os._exit(code)

    def call_other(self, other, n: int) -> int:
        return actors.get(other.add.remote(n))


@actors.remote
class FailingInit:
    def __init__(self):
        raise RuntimeError("constructor failure")
