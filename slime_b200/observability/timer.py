"""Named wall-clock timers.

``Timer()`` is a process singleton; ``with timer("name")`` / ``@timer`` accumulate seconds under
``name``; ``inverse_timer("x")`` measures the time *outside* its body (idle time between two
phases, e.g. ``train_wait``). ``log_dict()`` feeds ``perf/*_time`` metrics.
Parity: slime/observability/timer.py:15-100.
"""

from __future__ import annotations

import time
from contextlib import contextmanager
from functools import wraps

from slime_b200.utils.misc import SingletonMeta


class Timer(metaclass=SingletonMeta):
    def __init__(self):
        self.timers: dict[str, float] = {}
        self.start_time: dict[str, float] = {}
        self.seq_lens = None

    def start(self, name):
        assert name not in self.start_time, f"Timer {name} already started."
        self.start_time[name] = time.time()

    def end(self, name):
        assert name in self.start_time, f"Timer {name} not started."
        self.add(name, time.time() - self.start_time.pop(name))

    def add(self, name, elapsed):
        self.timers[name] = self.timers.get(name, 0.0) + elapsed

    def reset(self, name=None):
        if name is None:
            self.timers = {}
        else:
            self.timers.pop(name, None)

    def log_dict(self):
        return dict(self.timers)

    @contextmanager
    def context(self, name):
        self.start(name)
        try:
            yield
        finally:
            self.end(name)


def timer(name_or_func):
    """``with timer("x"):`` or ``@timer`` (uses the function name)."""
    if isinstance(name_or_func, str):
        return Timer().context(name_or_func)
    func = name_or_func

    @wraps(func)
    def wrapper(*a, **k):
        with Timer().context(func.__name__):
            return func(*a, **k)

    return wrapper


@contextmanager
def inverse_timer(name):
    """Stop ``name`` while the body runs; restart it on exit (accumulates time spent elsewhere)."""
    t = Timer()
    if name in t.start_time:
        t.end(name)
    try:
        yield
    finally:
        t.start(name)


def with_defer(deferred):
    """Decorator: always run ``deferred()`` after the wrapped function."""

    def deco(fn):
        @wraps(fn)
        def wrapper(*a, **k):
            try:
                return fn(*a, **k)
            finally:
                deferred()

        return wrapper

    return deco
