"""A background asyncio loop shared by synchronous callers (``run(coro)`` blocks for the result).

Parity: slime/utils/async_utils.py:34 — rollout functions are sync entry points over async internals."""

from __future__ import annotations

import asyncio
import threading

_loop: asyncio.AbstractEventLoop | None = None
_lock = threading.Lock()


def get_async_loop() -> asyncio.AbstractEventLoop:
    global _loop
    with _lock:
        if _loop is None or _loop.is_closed():
            _loop = asyncio.new_event_loop()
            threading.Thread(target=_loop.run_forever, daemon=True, name="slime-async-loop").start()
    return _loop


def run(coro):
    """Run ``coro`` on the shared background loop and wait for its result."""
    return asyncio.run_coroutine_threadsafe(coro, get_async_loop()).result()
