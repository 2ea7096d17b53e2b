"""HTTP helpers: one shared async client sized for the rollout concurrency, retrying POST/GET,
host/port discovery. Parity: slime/utils/http_utils.py:165-317 (60 x 1 s retry budget)."""

from __future__ import annotations

import asyncio
import json
import logging
import os
import socket

logger = logging.getLogger(__name__)
_client = None
_client_limit = 0
MAX_RETRIES = 60


def is_port_available(port: int) -> bool:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            s.bind(("", port))
            return True
        except OSError:
            return False


def find_available_port(base_port: int) -> int:
    port = base_port
    while not is_port_available(port):
        port += 1
    return port


def get_host_info() -> tuple[str, str]:
    """(hostname, ip). ``SLIME_HOST_IP`` overrides; ``SLIME_PREFER_IPV6`` picks an IPv6 address when available."""
    host = socket.gethostname()
    if os.environ.get("SLIME_HOST_IP"):
        return host, os.environ["SLIME_HOST_IP"]
    fam = socket.AF_INET6 if os.environ.get("SLIME_PREFER_IPV6") else socket.AF_INET
    probe = ("2001:4860:4860::8888", 80) if fam == socket.AF_INET6 else ("10.255.255.255", 1)
    try:
        with socket.socket(fam, socket.SOCK_DGRAM) as s:
            s.connect(probe)
            return host, s.getsockname()[0]
    except OSError:
        return host, "127.0.0.1"


def init_http_client(args) -> None:
    """(Re)create the shared client with ``server_concurrency x engines`` connections."""
    global _client, _client_limit
    import httpx

    engines = max(1, (getattr(args, "rollout_num_gpus", None) or 1) // max(getattr(args, "rollout_num_gpus_per_engine", 1), 1))
    limit = max(16, getattr(args, "sglang_server_concurrency", 512) * engines)
    if _client is None or _client_limit != limit:
        _client = httpx.AsyncClient(limits=httpx.Limits(max_connections=limit), timeout=httpx.Timeout(None))
        _client_limit = limit


def _get_client():
    global _client
    if _client is None:
        import httpx

        _client = httpx.AsyncClient(limits=httpx.Limits(max_connections=1024), timeout=httpx.Timeout(None))
    return _client


async def post(url: str, payload: dict | None = None, max_retries: int = MAX_RETRIES, headers: dict | None = None, action: str = "post"):
    """JSON request with a fixed 1 s back-off; in-flight rollout requests survive an engine restart this way."""
    client = _get_client()
    last = None
    for attempt in range(max_retries):
        try:
            if action == "get":
                resp = await client.get(url, headers=headers)
            elif action == "delete":
                resp = await client.delete(url, headers=headers)
            else:
                resp = await client.post(url, json=payload or {}, headers=headers)
            resp.raise_for_status()
            try:
                return resp.json()
            except json.JSONDecodeError:
                return resp.text
        except Exception as e:  # noqa: BLE001
            last = e
            if attempt + 1 < max_retries:
                logger.debug("%s %s failed (%r), retry %d/%d", action, url, e, attempt + 1, max_retries)
                await asyncio.sleep(1.0)
    raise last


async def get(url: str, max_retries: int = MAX_RETRIES, headers: dict | None = None):
    return await post(url, None, max_retries=max_retries, headers=headers, action="get")


def sync_request(method: str, url: str, payload: dict | None = None, timeout: float | None = 60.0):
    import requests

    r = requests.request(method, url, json=payload, timeout=timeout)
    r.raise_for_status()
    try:
        return r.json()
    except ValueError:
        return r.text
