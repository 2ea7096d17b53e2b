"""Abort-until-idle: keep sending ``/abort_request {abort_all}`` to every engine until its load endpoint
reports no running or queued requests. Parity: slime/backends/sglang_utils/server_control.py:12-67."""

from __future__ import annotations

import asyncio

from slime_b200.utils.http_utils import get, post


def num_requests_from_load(load) -> int:
    """Total requests an engine still holds, from a ``/v1/loads`` reply (list of per-DP-rank dicts)."""
    items = load if isinstance(load, list) else load.get("loads", [load]) if isinstance(load, dict) else []
    total = 0
    for it in items:
        if "num_reqs" in it:
            total += int(it["num_reqs"])
        else:
            total += int(it.get("num_running_reqs", 0)) + int(it.get("num_waiting_reqs", 0))
    return total


async def _abort_server_once(url: str):
    await post(f"{url}/abort_request", {"abort_all": True}, max_retries=3)


async def _get_server_num_requests(url: str) -> int:
    return num_requests_from_load(await get(f"{url}/v1/loads?include=core", max_retries=3))


async def abort_server_until_idle(url: str, interval: float = 0.2, max_rounds: int = 600) -> int:
    rounds = 0
    while rounds < max_rounds:
        await _abort_server_once(url)
        if await _get_server_num_requests(url) == 0:
            return rounds
        rounds += 1
        await asyncio.sleep(interval)
    raise TimeoutError(f"engine {url} still busy after {max_rounds} abort rounds")


async def abort_servers_until_idle(urls: list[str]):
    await asyncio.gather(*[abort_server_until_idle(u) for u in urls])
