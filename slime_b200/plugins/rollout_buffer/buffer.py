"""HTTP service that decouples trajectory *production* (agents, multi-turn generators) from the trainer.

    python -m slime_b200.plugins.rollout_buffer.buffer --port 8889

    POST /start_rollout     {"task_type", "num_repeat_per_sample", "input_file", "remote_engine_url", ...}
                            picks the generator registered for ``task_type`` and runs it in the background
    POST /buffer/write      one trajectory {"instance_id", "uid", "messages", "reward", "extra_info"}
    POST /get_rollout_data  every *complete* group (>= group_size trajectories of one instance_id, and whatever else
                            the generator's ``is_valid_group`` demands), after the generator's ``transform_group``
                            (e.g. reward normalisation); plus ``meta_info`` over everything written since the last read
    GET  /stats

Generators are modules in ``generator/`` (or any directory given with ``--generator-dir``) that define ``TASK_TYPE``
and ``run_rollout(payload)``; optional ``transform_group``, ``is_valid_group``, ``get_group_data_meta_info`` replace
the defaults. Replies have the shape ``{"success", "message", "data"}``.
Parity: slime_plugins/rollout_buffer/buffer.py:17-340.
"""

from __future__ import annotations

import argparse
import copy
import importlib.util
import logging
import pathlib
import threading
from typing import Any, Callable

logger = logging.getLogger(__name__)
Group = tuple[Any, list[dict]]


def default_is_valid_group(group: Group, min_valid_group_size: int, task_type: str) -> bool:
    return len(group[1]) >= min_valid_group_size


def default_group_meta(written: dict[Any, list[dict]]) -> dict[str, Any]:
    """Counts and mean reward over the trajectories written since the last read (kept or not)."""
    rewards = [s["reward"] for samples in written.values() for s in samples]
    n = len(rewards)
    return {"total_samples": n, "num_groups": len(written), "avg_group_size": n / len(written) if written else 0,
            "avg_reward": sum(rewards) / n if n else 0}  # fmt: skip


def discover_generators(*dirs: str | pathlib.Path) -> dict[str, dict[str, Any]]:
    """``task_type -> {"run_rollout", "transform_group", "is_valid_group", "get_group_data_meta_info", "file"}``."""
    found: dict[str, dict[str, Any]] = {}
    for d in dirs or (pathlib.Path(__file__).parent / "generator",):
        for path in sorted(pathlib.Path(d).glob("*.py")):
            if path.name == "__init__.py":
                continue
            try:
                spec = importlib.util.spec_from_file_location(f"_rollout_generator_{path.stem}", path)
                mod = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(mod)
            except Exception as e:  # noqa: BLE001
                logger.warning("generator %s failed to import: %r", path, e)
                continue
            if not hasattr(mod, "TASK_TYPE") or not hasattr(mod, "run_rollout"):
                logger.warning("generator %s lacks TASK_TYPE or run_rollout, ignored", path)
                continue
            found[mod.TASK_TYPE] = {"file": str(path), "run_rollout": mod.run_rollout,
                                    **{k: getattr(mod, k, None)
                                       for k in ("transform_group", "is_valid_group", "get_group_data_meta_info")}}  # fmt: skip
    return found


class RolloutBuffer:
    """Thread-safe store of trajectories grouped by ``instance_id``."""

    def __init__(self, group_size: int = 16, task_type: str = "math", transform_group_func: Callable | None = None,
                 is_valid_group_func: Callable | None = None, get_group_data_meta_info_func: Callable | None = None):  # fmt: skip
        self.group_size, self.task_type = group_size, task_type
        self.transform = transform_group_func or (lambda group, task_type: group)
        self.is_valid = is_valid_group_func or default_is_valid_group
        self.meta = get_group_data_meta_info_func or default_group_meta
        self.groups: dict[Any, list[dict]] = {}
        self.since_read: dict[Any, list[dict]] = {}
        self.lock = threading.RLock()
        self.total_written = self.total_read = 0

    def write(self, item: dict) -> dict:
        with self.lock:
            key = item["instance_id"]
            self.groups.setdefault(key, []).append(item)
            self.since_read.setdefault(key, []).append(copy.deepcopy(item))  # transform may edit rewards in place
            self.total_written += 1
        return item

    def ready_groups(self) -> dict[Any, list[dict]]:
        with self.lock:
            return {k: g for k, g in self.groups.items() if self.is_valid((k, g), self.group_size, self.task_type)}

    def __len__(self) -> int:
        return sum(len(g) for g in self.ready_groups().values())

    def read(self) -> dict[str, Any]:
        """Pop every ready group -> ``{"data": [trajectory, ...], "meta_info": {...}}`` (empty data if none is ready)."""
        with self.lock:
            ready = self.ready_groups()
            if not ready:
                return {"data": [], "meta_info": {}}
            meta = dict(self.meta(self.since_read))
            meta["finished_groups"] = []
            data: list[dict] = []
            for key, group in ready.items():
                data.extend(self.transform((key, group), self.task_type)[1])
                self.groups.pop(key, None)
            self.since_read = {}
            self.total_read += len(data)
            return {"data": data, "meta_info": meta}

    def stats(self) -> dict[str, int]:
        with self.lock:
            return {"written": self.total_written, "read": self.total_read, "pending_groups": len(self.groups),
                    "ready_samples": len(self)}  # fmt: skip


class BufferService:
    """The buffer plus the generator registry; ``start_rollout`` swaps in a buffer configured for the task."""

    def __init__(self, generator_dirs: tuple[str, ...] = ()):
        self.generator_dirs = generator_dirs
        self.buffer = RolloutBuffer()
        self.worker: threading.Thread | None = None

    def start_rollout(self, payload: dict) -> str | None:
        """None on success, else the reason. The generator runs on a daemon thread."""
        gens = discover_generators(*self.generator_dirs)
        task = payload.get("task_type")
        if task not in gens:
            return f"no generator for task_type {task!r} (available: {sorted(gens)})"
        g = gens[task]
        self.buffer = RolloutBuffer(int(payload["num_repeat_per_sample"]), task, g["transform_group"],
                                    g["is_valid_group"], g["get_group_data_meta_info"])  # fmt: skip

        def body():
            try:
                g["run_rollout"](payload)
                logger.info("rollout for task %s finished", task)
            except Exception:  # noqa: BLE001
                logger.exception("generator for task %s failed", task)

        self.worker = threading.Thread(target=body, daemon=True, name=f"generator-{task}")
        self.worker.start()
        return None


def build_app(service: BufferService):
    from aiohttp import web

    app = web.Application(client_max_size=1 << 30)

    def reply(success: bool, message: str = "", data=None, status: int = 200):
        return web.json_response({"success": success, "message": message, "data": data}, status=status)

    async def write(request):
        try:
            item = service.buffer.write(await request.json())
        except Exception as e:  # noqa: BLE001
            return reply(False, f"write failed: {e!r}", status=500)
        return reply(True, "written", {"data": [item], "meta_info": "write to buffer"})

    async def read(_request):
        out = service.buffer.read()
        if not out["data"]:
            return reply(False, "no complete group yet", {"data": [], "meta_info": out["meta_info"]})
        return reply(True, f"{len(out['data'])} trajectories", out)

    async def start(request):
        why = service.start_rollout(await request.json())
        if why:
            return web.json_response({"message": why}, status=400)
        return web.json_response({"message": "Rollout started"})

    async def stats(_request):
        return web.json_response(service.buffer.stats())

    app.router.add_post("/buffer/write", write)
    app.router.add_post("/get_rollout_data", read)
    app.router.add_post("/start_rollout", start)
    app.router.add_get("/stats", stats)
    return app


def main(argv=None):
    from aiohttp import web

    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8889)
    ap.add_argument("--generator-dir", action="append", default=[])
    a = ap.parse_args(argv)
    web.run_app(build_app(BufferService(tuple(a.generator_dir))), host=a.host, port=a.port, access_log=None)


if __name__ == "__main__":
    main()
