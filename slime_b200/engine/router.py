"""Request router in front of one model's rollout engines.

Replaces the ``sglang_router`` process the reference launches per model
(slime/ray/rollout.py:916-968). Surface: ``POST /workers {url, worker_type, bootstrap_port}``,
``GET /workers``, ``DELETE /workers/{id}``, proxied ``POST /generate`` (plus every other engine path,
fanned out or forwarded), ``GET /engine_metrics``, ``GET /health``.

Policies: ``cache_aware`` (default; requests whose prompts share a page-aligned prefix go to the worker
that served the prefix before unless it is overloaded), ``round_robin``, ``random``, ``power_of_two``
(least loaded of two random workers) and ``consistent_hashing`` keyed by the ``X-SMG-Routing-Key``
header (session affinity for multi-turn rollouts). Prefill/decode disaggregation: a request is sent to a
prefill worker first (``max_new_tokens=0`` with its KV exported) and then to a decode worker.
"""

from __future__ import annotations

import asyncio
import bisect
import hashlib
import itertools
import json
import random
import threading
import time
from dataclasses import dataclass, field


@dataclass
class Worker:
    id: str
    url: str
    worker_type: str = "regular"  # regular | prefill | decode | encoder
    bootstrap_port: int | None = None
    inflight: int = 0
    healthy: bool = True
    served: int = 0
    added: float = field(default_factory=time.time)


class Router:
    def __init__(self, host="127.0.0.1", port=30100, policy="cache_aware", balance_abs_threshold=32,
                 balance_rel_threshold=1.1, request_timeout_secs=14400, prefix_block=64):  # fmt: skip
        self.host, self.port, self.policy = host, port, policy
        self.abs_thr, self.rel_thr = balance_abs_threshold, balance_rel_threshold
        self.timeout = request_timeout_secs
        self.prefix_block = prefix_block
        self.workers: dict[str, Worker] = {}
        self._rr = itertools.count()
        self._ids = itertools.count()
        self._prefix_owner: dict[bytes, str] = {}
        self._ring: list[tuple[int, str]] = []
        self._session = None
        self._loop = None
        self._runner = None

    # ---------------------------------------------------------------------- membership
    def add_worker(self, url, worker_type="regular", bootstrap_port=None) -> Worker:
        for w in self.workers.values():
            if w.url == url:
                return w
        w = Worker(id=str(next(self._ids)), url=url.rstrip("/"), worker_type=worker_type, bootstrap_port=bootstrap_port)
        self.workers[w.id] = w
        self._rebuild_ring()
        return w

    def remove_worker(self, wid_or_url) -> bool:
        for wid, w in list(self.workers.items()):
            if wid == wid_or_url or w.url == str(wid_or_url).rstrip("/"):
                del self.workers[wid]
                self._prefix_owner = {k: v for k, v in self._prefix_owner.items() if v != wid}
                self._rebuild_ring()
                return True
        return False

    def _rebuild_ring(self, vnodes=64):
        self._ring = sorted(
            (int.from_bytes(hashlib.md5(f"{w.id}:{v}".encode()).digest()[:8], "big"), w.id)
            for w in self.workers.values() for v in range(vnodes)
        )  # fmt: skip

    # -------------------------------------------------------------------------- policies
    def _candidates(self, kind="regular"):
        ws = [w for w in self.workers.values() if w.healthy and w.worker_type == kind]
        if not ws and kind == "regular":
            ws = [w for w in self.workers.values() if w.healthy and w.worker_type == "decode"]
        return ws

    def pick(self, input_ids=None, routing_key: str | None = None, kind="regular") -> Worker:
        ws = self._candidates(kind)
        if not ws:
            raise RuntimeError(f"no healthy {kind} workers registered")
        policy = self.policy
        if routing_key is not None and (policy == "consistent_hashing" or policy == "cache_aware"):
            return self._by_ring(routing_key, ws)
        if policy == "round_robin":
            return ws[next(self._rr) % len(ws)]
        if policy == "random":
            return random.choice(ws)
        if policy == "power_of_two":
            a, b = random.choice(ws), random.choice(ws)
            return a if a.inflight <= b.inflight else b
        if policy == "consistent_hashing":
            return self._by_ring(json.dumps(input_ids[:64]) if input_ids else str(next(self._rr)), ws)
        return self._cache_aware(input_ids, ws)

    def _by_ring(self, key: str, ws) -> Worker:
        alive = {w.id for w in ws}
        h = int.from_bytes(hashlib.md5(key.encode()).digest()[:8], "big")
        i = bisect.bisect(self._ring, (h, ""))
        for j in range(len(self._ring)):
            wid = self._ring[(i + j) % len(self._ring)][1]
            if wid in alive:
                return self.workers[wid]
        return ws[0]

    def _cache_aware(self, input_ids, ws) -> Worker:
        least = min(ws, key=lambda w: w.inflight)
        most = max(ws, key=lambda w: w.inflight)
        imbalanced = most.inflight - least.inflight > self.abs_thr and most.inflight > self.rel_thr * max(least.inflight, 1)
        if not input_ids or imbalanced:
            return least
        # longest known page-aligned prefix wins
        keys, h = [], hashlib.blake2b(digest_size=8)
        for s in range(0, len(input_ids) - len(input_ids) % self.prefix_block, self.prefix_block):
            h.update(str(input_ids[s : s + self.prefix_block]).encode())
            keys.append(h.digest())
        owner = None
        for k in reversed(keys):
            wid = self._prefix_owner.get(k)
            if wid is not None and wid in self.workers and self.workers[wid].healthy and self.workers[wid] in ws:
                owner = self.workers[wid]
                break
        target = owner or least
        for k in keys:
            self._prefix_owner.setdefault(k, target.id)
        if len(self._prefix_owner) > 1_000_000:
            self._prefix_owner.clear()
        return target

    # -------------------------------------------------------------------------- HTTP app
    async def _client(self):
        import aiohttp

        if self._session is None or self._session.closed:
            self._session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.timeout),
                                                  connector=aiohttp.TCPConnector(limit=0))  # fmt: skip
        return self._session

    async def _h_add(self, request):
        from aiohttp import web

        body = await request.json()
        w = self.add_worker(body["url"], body.get("worker_type", "regular"), body.get("bootstrap_port"))
        return web.json_response({"id": w.id, "url": w.url, "worker_type": w.worker_type})

    async def _h_list(self, request):
        from aiohttp import web

        return web.json_response({"workers": [vars(w) for w in self.workers.values()]})

    async def _h_del(self, request):
        from aiohttp import web

        ok = self.remove_worker(request.match_info["wid"])
        return web.json_response({"success": ok}, status=200 if ok else 404)

    async def _h_generate(self, request):
        from aiohttp import web

        body = await request.json()
        ids = body.get("input_ids")
        key = request.headers.get("X-SMG-Routing-Key")
        has_pd = any(w.worker_type == "prefill" for w in self.workers.values())
        try:
            if has_pd and isinstance(ids, list) and ids and isinstance(ids[0], int):
                # prefill on one worker (it keeps the prompt's KV and samples the first token), decode on another,
                # which pulls the KV from the first and continues without a prefill pass of its own
                pre = self.pick(ids, key, "prefill")
                status, first = await self._forward(pre, "/generate", dict(body, disaggregation="prefill", stream=False, return_logprob=True))
                meta = first.get("meta_info", {}) if isinstance(first, dict) else {}
                if status != 200 or (meta.get("finish_reason") or {}).get("type") != "prefill_done":
                    return web.json_response(first, status=status)  # failed, or already finished with its first token
                lp = (meta.get("output_token_logprobs") or [[0.0]])[0][0]
                body = dict(body, bootstrap_host=pre.url, bootstrap_room=meta["kv_handle"], first_token=first["output_ids"][0],
                            first_logprob=lp)  # fmt: skip
                w = self.pick(None, key, "decode")
            elif has_pd:
                w = self.pick(None, key, "decode")  # batched prompts: the decode worker runs both phases
            else:
                w = self.pick(ids if isinstance(ids, list) and ids and isinstance(ids[0], int) else None, key)
        except RuntimeError as e:
            return web.json_response({"error": str(e)}, status=503)
        if body.get("stream"):
            return await self._forward_stream(request, w, body)
        status, payload = await self._forward(w, "/generate", body)
        return web.json_response(payload, status=status)

    async def _forward(self, w: Worker, path: str, body):
        s = await self._client()
        w.inflight += 1
        try:
            async with s.post(w.url + path, json=body) as resp:
                w.served += 1
                return resp.status, await resp.json(content_type=None)
        except Exception as e:  # noqa: BLE001
            w.healthy = False
            return 502, {"error": f"worker {w.url} failed: {e!r}"}
        finally:
            w.inflight -= 1

    async def _forward_stream(self, request, w: Worker, body):
        from aiohttp import web

        s = await self._client()
        out = web.StreamResponse(headers={"Content-Type": "text/event-stream"})
        await out.prepare(request)
        w.inflight += 1
        try:
            async with s.post(w.url + "/generate", json=body) as resp:
                async for chunk in resp.content.iter_any():
                    await out.write(chunk)
        finally:
            w.inflight -= 1
        return out

    async def _h_fanout(self, request):
        """Control endpoints are applied to every worker (flush_cache, abort_request, pause/continue...)."""
        from aiohttp import web

        s = await self._client()
        body = await request.read()
        results = []
        for w in list(self.workers.values()):
            try:
                async with s.request(request.method, w.url + request.path_qs, data=body or None,
                                     headers={"Content-Type": "application/json"}) as resp:  # fmt: skip
                    results.append({"worker": w.url, "status": resp.status, "body": await resp.text()})
            except Exception as e:  # noqa: BLE001
                results.append({"worker": w.url, "status": 502, "body": repr(e)})
        ok = all(r["status"] < 400 for r in results)
        return web.json_response({"results": results}, status=200 if ok else 502)

    async def _h_metrics(self, request):
        from aiohttp import web

        s = await self._client()
        parts = []
        for w in list(self.workers.values()):
            try:
                async with s.get(w.url + "/metrics") as resp:
                    parts.append(f"# worker {w.url}\n" + await resp.text())
            except Exception:  # noqa: BLE001
                parts.append(f"# worker {w.url} unreachable\n")
        return web.Response(text="\n".join(parts))

    async def _h_health(self, request):
        from aiohttp import web

        return web.json_response({"status": "ok", "workers": len(self.workers)})

    def build_app(self):
        from aiohttp import web

        app = web.Application(client_max_size=1 << 34)
        r = app.router
        r.add_post("/workers", self._h_add)
        r.add_get("/workers", self._h_list)
        r.add_delete("/workers/{wid}", self._h_del)
        r.add_post("/generate", self._h_generate)
        r.add_get("/engine_metrics", self._h_metrics)
        r.add_get("/health", self._h_health)
        for path in ("/flush_cache", "/abort_request", "/pause_generation", "/continue_generation", "/start_profile",
                     "/stop_profile", "/release_memory_occupation", "/resume_memory_occupation"):  # fmt: skip
            r.add_route("*", path, self._h_fanout)
        return app

    def start(self, block=False):
        from aiohttp import web

        ready = threading.Event()

        def serve():
            self._loop = asyncio.new_event_loop()
            asyncio.set_event_loop(self._loop)
            self._runner = web.AppRunner(self.build_app(), access_log=None)
            self._loop.run_until_complete(self._runner.setup())
            self._loop.run_until_complete(web.TCPSite(self._runner, self.host, self.port).start())
            ready.set()
            self._loop.run_forever()

        if block:
            serve()
        else:
            threading.Thread(target=serve, daemon=True, name="router-http").start()
            ready.wait(timeout=30)
        return self

    def shutdown(self):
        if self._loop is not None:
            self._loop.call_soon_threadsafe(self._loop.stop)


if __name__ == "__main__":
    import argparse

    p = argparse.ArgumentParser("slime_b200.engine.router")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=30100)
    p.add_argument("--policy", default="cache_aware")
    p.add_argument("--request-timeout-secs", type=int, default=14400)
    a = p.parse_args()
    Router(a.host, a.port, a.policy, request_timeout_secs=a.request_timeout_secs).start(block=True)
