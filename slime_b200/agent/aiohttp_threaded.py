"""Serve an ``aiohttp`` application from a background thread that owns its own event loop.

The adapters (chat-protocol front ends for agent harnesses) are started this way from inside a rollout function, whose
own event loop must stay free for generation requests. ``serve_in_thread`` returns once the socket is listening, with
the port the kernel picked when ``port=0``. Parity: slime/agent/aiohttp_threaded.py:14-98.
"""

from __future__ import annotations

import asyncio
import dataclasses
import threading
from typing import Any

from aiohttp import web
from aiohttp.web_log import AccessLogger


class QuietAccessLogger(AccessLogger):
    """Logs only what deserves attention: non-200 answers and requests slower than ``slow_sec``."""

    slow_sec = 120.0

    def log(self, request, response, time):
        if request.method != "HEAD" and (response.status != 200 or time > self.slow_sec):
            super().log(request, response, time)


@dataclasses.dataclass
class AppHandle:
    host: str
    port: int
    thread: threading.Thread
    loop: asyncio.AbstractEventLoop
    runner: web.AppRunner

    @property
    def url(self) -> str:
        return f"http://{'127.0.0.1' if self.host in ('0.0.0.0', '') else self.host}:{self.port}"

    def stop(self, timeout: float = 10.0) -> None:
        try:
            asyncio.run_coroutine_threadsafe(self.runner.cleanup(), self.loop).result(timeout)
        except Exception:  # noqa: BLE001
            pass
        self.loop.call_soon_threadsafe(self.loop.stop)
        self.thread.join(5)


def serve_in_thread(app: web.Application, *, host: str = "0.0.0.0", port: int = 0, thread_name: str = "aiohttp-app",
                    start_timeout_sec: float = 15.0, runner_kwargs: dict[str, Any] | None = None) -> AppHandle:  # fmt: skip
    """``runner_kwargs`` go to ``web.AppRunner`` (``{"handler_cancellation": True}`` makes a client disconnect cancel
    the handler, which the adapters use to abort generation nobody is waiting for)."""
    ready = threading.Event()
    out: dict[str, Any] = {}

    def body():
        loop = asyncio.new_event_loop()
        asyncio.set_event_loop(loop)
        try:
            runner = web.AppRunner(app, **(runner_kwargs or {}))
            loop.run_until_complete(runner.setup())
            site = web.TCPSite(runner, host, port)
            loop.run_until_complete(site.start())
            bound = runner.addresses[0][1] if runner.addresses else port
            out.update(loop=loop, runner=runner, port=int(bound))
        except BaseException as e:  # noqa: BLE001
            out["error"] = e
            ready.set()
            return
        ready.set()
        loop.run_forever()
        loop.close()

    t = threading.Thread(target=body, name=thread_name, daemon=True)
    t.start()
    if not ready.wait(start_timeout_sec):
        raise TimeoutError(f"{thread_name}: not listening after {start_timeout_sec}s")
    if "error" in out:
        raise out["error"]
    return AppHandle(host, out["port"], t, out["loop"], out["runner"])


run_app_in_thread = serve_in_thread  # the name slime.agent.aiohttp_threaded exports
FilteredAccessLogger = QuietAccessLogger
