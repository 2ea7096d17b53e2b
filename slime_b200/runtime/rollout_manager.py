"""Rollout orchestration: engine server groups, routers, the data source and the generate/eval loop.

Layout (one box, one process per engine):

    RolloutManager (actor)
      ├─ servers: {model name -> RolloutServer}          one router per model
      │     └─ server_groups: [ServerGroup]              homogeneous engines (regular | prefill | decode | ...)
      │            └─ all_engines: [RolloutEngineActor handle | None]   None = dead, restarted by recover()
      ├─ data_source, generate_rollout / eval functions (loaded from --*-path flags)
      ├─ rollout_engine_lock (Lock actor: serialises weight broadcasts to shared engines)
      └─ RolloutHealthMonitor per group (``--use-fault-tolerance``)

``generate(rollout_id)`` returns one object-store reference per trainer DP rank (the per-rank
payload carries the micro-batch schedule), exactly what ``TrainActor.train`` consumes.
Parity: slime/ray/rollout.py:46-365 (groups/servers), :366-826 (manager), :827-1153 (ports, router, start).
"""

from __future__ import annotations

import dataclasses
import itertools
import logging
import random
import time
from typing import Any

from slime_b200.engine.engine_actor import RolloutEngineActor
from slime_b200.engine.sglang_config import SglangConfig
from slime_b200.observability import logging_utils
from slime_b200.observability.rollout_data_utils import (load_debug_rollout_data, save_debug_rollout_data,
                                                         validate_rollout_id_annotated)  # fmt: skip
from slime_b200.observability.rollout_metrics import log_eval_rollout_data, log_rollout_data
from slime_b200.rollout.base_types import call_rollout_fn
from slime_b200.rollout.train_data import convert_samples_to_train_data, split_train_data_by_dp
from slime_b200.runtime import actors, object_store
from slime_b200.utils.health_monitor import RolloutHealthMonitor
from slime_b200.utils.http_utils import find_available_port, init_http_client
from slime_b200.utils.misc import Box, get_current_node_ip, load_function

logger = logging.getLogger(__name__)

GPU_MEMORY_TYPE_WEIGHTS = "weights"
GPU_MEMORY_TYPE_KV_CACHE = "kv_cache"
GPU_MEMORY_TYPE_CUDA_GRAPH = "cuda_graph"

EngineActor = actors.remote(RolloutEngineActor)

_current_rollout_id = -1


def set_current_rollout_id(rollout_id: int):
    global _current_rollout_id
    _current_rollout_id = rollout_id
    from slime_b200.rollout import sample_hooks

    sample_hooks.set_current_rollout_id(rollout_id)  # what sample hooks receive as ``rollout_id``


def get_current_rollout_id() -> int:
    return _current_rollout_id


# ------------------------------------------------------------------------------- server groups
@dataclasses.dataclass
class ServerGroup:
    """Engines that share worker type, GPUs-per-engine and overrides."""

    args: Any
    pg: Any  # runtime.placement.PlacementGroup or None on CPU
    all_engines: list
    num_gpus_per_engine: int
    num_new_engines: int = 0
    worker_type: str = "regular"
    rank_offset: int = 0
    gpu_offset: int = 0
    overrides: dict = dataclasses.field(default_factory=dict)
    needs_offload: bool = False
    model_path: str | None = None
    router_ip: str | None = None
    router_port: int | None = None

    @property
    def nodes_per_engine(self) -> int:
        return max(1, self.num_gpus_per_engine // self.args.num_gpus_per_node)

    @property
    def engines(self) -> list:
        """The node-0 process of every engine (the one that owns the HTTP server)."""
        return self.all_engines[:: self.nodes_per_engine]

    @property
    def parallel_config(self) -> dict:
        o = self.overrides
        pp = o.get("pp_size") or getattr(self.args, "sglang_pp_size", None) or 1
        return {"tp_size": o.get("tp_size") or max(1, self.num_gpus_per_engine // pp), "pp_size": pp,
                "dp_size": o.get("dp_size") or getattr(self.args, "sglang_dp_size", None) or 1,
                "ep_size": o.get("ep_size") or getattr(self.args, "sglang_ep_size", None) or 1}  # fmt: skip

    def start_engines(self, port_cursor: int) -> tuple[list, int]:
        """Spawn an actor for every empty slot and kick off ``init``; returns (pending init refs, next free port)."""
        if self.worker_type == "placeholder":
            self.num_new_engines = 0
            return [], port_cursor
        per_node = min(self.num_gpus_per_engine, self.args.num_gpus_per_node)
        host = get_current_node_ip()
        fresh = []
        for i, e in enumerate(self.all_engines):
            if e is not None:
                continue
            gpu_index = self.gpu_offset + i * per_node
            base_gpu = self.pg.gpu(gpu_index).gpu_id if self.pg is not None and self.pg.count else gpu_index
            h = EngineActor.options(name=f"engine-{self.rank_offset + i}", max_concurrency=8).remote(
                self.args, self.rank_offset + i, self.worker_type, base_gpu, self.overrides, self.model_path)
            self.all_engines[i] = h
            fresh.append((i, h))
        self.num_new_engines = len(fresh)
        refs = []
        for i, h in fresh:
            port = find_available_port(port_cursor)
            nccl_port = find_available_port(port + 1)
            dist_port = find_available_port(nccl_port + 1)
            port_cursor = dist_port + 1
            refs.append(h.init.remote(host, port, nccl_port, f"{host}:{dist_port}", self.router_ip, self.router_port))
        return refs, port_cursor

    def offload(self) -> list:
        if not self.needs_offload:
            return []
        return [e.release_memory_occupation.remote() for e in self.engines if e is not None]

    def onload(self, tags: list[str] | None = None) -> list:
        if not self.needs_offload:
            return []
        return [e.resume_memory_occupation.remote(tags=tags) for e in self.engines if e is not None]


@dataclasses.dataclass
class RolloutServer:
    """One model behind one router."""

    server_groups: list[ServerGroup]
    router_ip: str | None = None
    router_port: int | None = None
    model_name: str = "default"
    update_weights: bool = True
    router: Any = None

    @property
    def engines(self) -> list:
        return [e for g in self.server_groups for e in g.engines]

    @property
    def all_engines(self) -> list:
        return [e for g in self.server_groups for e in g.all_engines]

    @property
    def num_new_engines(self) -> int:
        return sum(g.num_new_engines for g in self.server_groups)

    @num_new_engines.setter
    def num_new_engines(self, value: int):
        for g in self.server_groups:
            g.num_new_engines = value

    @property
    def engine_gpu_counts(self) -> list[int]:
        return [g.num_gpus_per_engine for g in self.server_groups for _ in g.engines]

    @property
    def engine_gpu_offsets(self) -> list[int]:
        return [g.gpu_offset + j * g.num_gpus_per_engine for g in self.server_groups for j in range(len(g.engines))]

    @property
    def engine_parallel_configs(self) -> list[dict]:
        return [g.parallel_config for g in self.server_groups for _ in g.engines]

    def recover(self, port_cursor: int = 15000) -> int:
        """Restart dead engines of every group; fresh engines resume weights only (the trainer re-syncs them and
        KV / graphs come back with ``onload_kv``). Returns how many engines were started."""
        refs, fresh_before = [], []
        for g in self.server_groups:
            dead = [i for i, e in enumerate(g.all_engines) if e is None]
            if not dead:
                g.num_new_engines = 0
                continue
            logger.warning("recovering %d dead engine(s) of group %s/%s", len(dead), self.model_name, g.worker_type)
            r, port_cursor = g.start_engines(port_cursor)
            refs += r
            fresh_before += [g.all_engines[i] for i in dead if g.needs_offload]
        if refs:
            actors.get(refs)
        if fresh_before:
            actors.get([e.release_memory_occupation.remote() for e in fresh_before])
            actors.get([e.resume_memory_occupation.remote(tags=[GPU_MEMORY_TYPE_WEIGHTS]) for e in fresh_before])
        return self.num_new_engines

    def offload(self):
        return actors.get([r for g in self.server_groups for r in g.offload()])

    def onload(self, tags: list[str] | None = None):
        return actors.get([r for g in self.server_groups for r in g.onload(tags)])

    def onload_weights(self):
        return self.onload([GPU_MEMORY_TYPE_WEIGHTS])

    def onload_kv(self):
        return self.onload([GPU_MEMORY_TYPE_KV_CACHE, GPU_MEMORY_TYPE_CUDA_GRAPH])


# --------------------------------------------------------------------------------- start-up
def _start_router(args, *, has_pd_disaggregation: bool = False, force_new: bool = False, overrides: dict | None = None):
    """Launch the in-tree router on a thread of this process unless the user pointed at an existing one."""
    if not force_new and getattr(args, "sglang_router_ip", None) is not None:
        return args.sglang_router_ip, args.sglang_router_port, None
    from slime_b200.engine.router import Router

    ip = get_current_node_ip()
    port = getattr(args, "sglang_router_port", None) if not force_new else None
    if port is None:
        port = find_available_port(random.randint(3000, 4000))
    kw = dict(policy=getattr(args, "sglang_router_policy", None) or "cache_aware",
              request_timeout_secs=getattr(args, "sglang_router_request_timeout_secs", None) or 14400)  # fmt: skip
    kw.update(overrides or {})
    router = Router(host=ip, port=port, **kw)
    router.pd_disaggregation = has_pd_disaggregation
    router.start(block=False)
    logger.info("router for rollout engines listening at %s:%s (policy %s)", ip, port, kw["policy"])
    return ip, port, router


def _resolve_sglang_config(args) -> SglangConfig:
    if getattr(args, "sglang_config", None):
        return SglangConfig.from_yaml(args.sglang_config, args)
    return SglangConfig.from_prefill_num_servers(args)


def start_rollout_servers(args, pg) -> tuple[dict[str, RolloutServer], list]:
    """Create routers and engine groups for every configured model; engine ``init`` calls are left pending so
    the caller can overlap them with loading the data source."""
    if getattr(args, "rollout_external_engine_addrs", None):
        from slime_b200.engine import external

        if getattr(args, "rollout_external_engine_infos", None) is None:
            external.apply_external_engine_info_to_args(args, logger)

        def make_engine(rank, info):  # HTTP front only: the engine process itself belongs to someone else
            return EngineActor.options(name=f"external-engine-{rank}", max_concurrency=8).remote(
                args, rank, info.worker_type, 0, None, None)

        return external.start_external_rollout_servers(args, start_router=_start_router, make_engine=make_engine)
    cfg = _resolve_sglang_config(args)
    servers: dict[str, RolloutServer] = {}
    pending, port_cursor = [], 15000
    gpu_offset = rank_offset = 0
    for mi, m in enumerate(cfg.models):
        ip, port, router = _start_router(args, has_pd_disaggregation=m.has_pd_disaggregation, force_new=mi > 0,
                                         overrides=m.router_overrides)  # fmt: skip
        if mi == 0:
            args.sglang_router_ip, args.sglang_router_port = ip, port
        groups = []
        for gc in m.server_groups:
            n_engines = 0 if gc.worker_type == "placeholder" else gc.num_gpus // gc.num_gpus_per_engine
            nodes_per = max(1, gc.num_gpus_per_engine // args.num_gpus_per_node)
            if pg is not None and hasattr(pg, "count"):
                from slime_b200.runtime.rollout_validation import validate_server_group_gpu_indices

                validate_server_group_gpu_indices(
                    worker_type=gc.worker_type, gpu_offset=gpu_offset, num_gpus_per_engine=gc.num_gpus_per_engine,
                    num_gpus_per_engine_on_node=min(gc.num_gpus_per_engine, args.num_gpus_per_node), num_engines=n_engines,
                    num_available_gpus=pg.count, rollout_num_gpus=getattr(args, "rollout_num_gpus", None),
                    rollout_num_gpus_per_engine=getattr(args, "rollout_num_gpus_per_engine", None))  # fmt: skip
            g = ServerGroup(args=args, pg=pg, all_engines=[None] * (n_engines * nodes_per),
                            num_gpus_per_engine=gc.num_gpus_per_engine, worker_type=gc.worker_type,
                            rank_offset=rank_offset, gpu_offset=gpu_offset, overrides=dict(gc.overrides),
                            needs_offload=bool(args.offload_rollout), model_path=m.model_path, router_ip=ip,
                            router_port=port)  # fmt: skip
            refs, port_cursor = g.start_engines(port_cursor)
            pending += refs
            groups.append(g)
            gpu_offset += gc.num_gpus
            rank_offset += n_engines
        servers[m.name] = RolloutServer(groups, ip, port, m.name, bool(m.update_weights), router)
    args.sglang_model_routers = {name: (s.router_ip, s.router_port) for name, s in servers.items()}
    return servers, pending


# --------------------------------------------------------------------------------- the manager
class RolloutManager:
    """Runs rollouts and turns samples into per-DP-rank training payloads."""

    def __init__(self, args, pg=None):
        logging_utils.configure_logger()
        self.args, self.pg = args, pg
        pending: list = []
        if args.debug_train_only:
            self.servers: dict[str, RolloutServer] = {}
        else:
            init_http_client(args)
            self.servers, pending = start_rollout_servers(args, pg)
        self.data_source = load_function(args.data_source_path)(args)
        self.generate_rollout = load_function(args.rollout_function_path)
        self.eval_generate_rollout = load_function(args.eval_function_path)
        self.custom_reward_post_process_func = (load_function(args.custom_reward_post_process_path)
                                                if args.custom_reward_post_process_path else None)  # fmt: skip
        self.custom_convert_samples_to_train_data_func = (load_function(args.custom_convert_samples_to_train_data_path)
                                                          if args.custom_convert_samples_to_train_data_path else None)  # fmt: skip
        if pending:
            actors.get(pending)
        logging_utils.init_tracking(args, primary=False)
        self.rollout_engine_lock = actors.Lock.remote()
        self.rollout_id = -1
        self._live_refs: list[list] = []
        self.train_parallel_config: dict | None = None
        self._health_monitors: list[RolloutHealthMonitor] = []
        self._ci_fault_injection_pending = False
        if not args.debug_train_only and args.use_fault_tolerance:
            for srv in self.servers.values():
                for g in srv.server_groups:
                    mon = RolloutHealthMonitor(g, args)
                    if mon.start():
                        self._health_monitors.append(mon)
            self._ci_fault_injection_pending = bool(getattr(args, "ci_test", False))

    # ------------------------------------------------------------------ accessors
    @property
    def server(self) -> RolloutServer | None:
        return next(iter(self.servers.values()), None)

    def _get_updatable_server(self) -> RolloutServer | None:
        return next((s for s in self.servers.values() if s.update_weights), None)

    @property
    def rollout_engines(self) -> list:
        return [e for s in self.servers.values() for e in s.engines]

    def get_updatable_engines_and_lock(self):
        s = self._get_updatable_server()
        if s is None:
            return [], self.rollout_engine_lock, 0, [], [], []
        return (s.engines, self.rollout_engine_lock, s.num_new_engines, s.engine_gpu_counts, s.engine_gpu_offsets,
                s.engine_parallel_configs)  # fmt: skip

    def get_engine_urls(self) -> list[str]:
        return actors.get([e.get_url.remote() for e in self.rollout_engines if e is not None])

    def get_router_address(self, model_name: str | None = None):
        s = self.servers.get(model_name) if model_name else self.server
        return (s.router_ip, s.router_port) if s else None

    def get_num_rollout_per_epoch(self) -> int:
        assert self.args.rollout_global_dataset
        return len(self.data_source) // self.args.rollout_batch_size

    def set_train_parallel_config(self, config: dict):
        self.train_parallel_config = config

    # ------------------------------------------------------------------ generate / eval
    def generate(self, rollout_id: int):
        start = time.time()
        self.rollout_id = rollout_id
        set_current_rollout_id(rollout_id)
        self.health_monitoring_resume()
        if self._ci_fault_injection_pending and rollout_id >= 2:
            self._try_ci_fault_injection()
        data, metrics = self._get_rollout_data(rollout_id)
        save_debug_rollout_data(self.args.save_debug_rollout_data, data, rollout_id=rollout_id, evaluation=False)
        log_rollout_data(rollout_id, self.args, data, metrics, time.time() - start)
        if self.args.debug_rollout_only:
            return None
        train_data = self._convert_samples_to_train_data(data)
        return self._split_train_data_by_dp(train_data)

    def eval(self, rollout_id: int):
        if self.args.debug_train_only:
            return None
        set_current_rollout_id(rollout_id)
        self.health_monitoring_resume()
        result = call_rollout_fn(self.eval_generate_rollout, self.args, rollout_id, self.data_source, evaluation=True)
        save_debug_rollout_data(self.args.save_debug_rollout_data, result.data, rollout_id=rollout_id, evaluation=True)
        return log_eval_rollout_data(rollout_id, self.args, result.data, result.metrics)

    def _get_rollout_data(self, rollout_id: int):
        if self.args.load_debug_rollout_data:
            return load_debug_rollout_data(self.args.load_debug_rollout_data, rollout_id=rollout_id,
                                           subsample_ratio=self.args.load_debug_rollout_data_subsample), None  # fmt: skip
        out = call_rollout_fn(self.generate_rollout, self.args, rollout_id, self.data_source, evaluation=False)
        data = out.samples
        validate_rollout_id_annotated(data)
        while data and isinstance(data[0], list):
            data = list(itertools.chain.from_iterable(data))
        return data, out.metrics

    def _convert_samples_to_train_data(self, samples):
        if self.custom_convert_samples_to_train_data_func is not None:
            return self.custom_convert_samples_to_train_data_func(self.args, samples)
        return convert_samples_to_train_data(self.args, samples)  # applies --custom-reward-post-process-path itself

    def _split_train_data_by_dp(self, data: dict) -> list:
        cfg = self.train_parallel_config or {"dp_size": 1, "cp_size": 1, "vpp_size": 1}
        parts = split_train_data_by_dp(self.args, data, cfg)
        refs = [Box(object_store.put(p)) for p in parts]
        # payloads live in shared memory until two newer rollouts exist (async training reads one rollout behind)
        self._live_refs.append(refs)
        while len(self._live_refs) > 3:
            for old in self._live_refs.pop(0):
                object_store.free(old.inner)
        return refs

    # ------------------------------------------------------------------ persistence
    def save(self, rollout_id: int):
        self.data_source.save(rollout_id)

    def load(self, rollout_id: int | None = None):
        self.data_source.load(rollout_id)

    # ------------------------------------------------------------------ memory
    def offload(self):
        self.health_monitoring_pause()
        for s in self.servers.values():
            s.offload()

    def onload(self, tags: list[str] | None = None):
        for s in self.servers.values():
            s.onload(tags)

    def onload_weights(self):
        for s in self.servers.values():
            s.onload_weights()

    def onload_kv(self):
        for s in self.servers.values():
            s.onload_kv()

    # ------------------------------------------------------------------ fault tolerance
    def recover_updatable_engines(self) -> int:
        """Called by the driver before a weight update: health checks are paused (engines may be offloaded or
        mid-update) and dead engines of the updatable model are restarted."""
        self.health_monitoring_pause()
        s = self._get_updatable_server()
        if self.rollout_id == -1 or s is None:
            return 0
        return s.recover()

    def clear_updatable_num_new_engines(self):
        s = self._get_updatable_server()
        if s is not None:
            s.num_new_engines = 0

    def health_monitoring_pause(self):
        for m in self._health_monitors:
            m.pause()

    def health_monitoring_resume(self):
        for m in self._health_monitors:
            m.resume()

    def num_dead_engines(self) -> int:
        return sum(e is None for s in self.servers.values() for e in s.all_engines)

    def _try_ci_fault_injection(self):
        """One-shot host-side fault: ask engine 0 to stop serving, then give the monitor time to notice."""
        self._ci_fault_injection_pending = False
        s = self.server
        if not (s and s.server_groups and s.server_groups[0].all_engines and s.server_groups[0].all_engines[0]):
            return
        logger.info("fault injection: simulating a crash of engine 0")
        try:
            s.server_groups[0].all_engines[0].simulate_crash.remote()
            wait_s = self.args.rollout_health_check_interval + self.args.rollout_health_check_timeout + 5
            deadline = time.time() + wait_s
            while time.time() < deadline and s.server_groups[0].all_engines[0] is not None:
                time.sleep(0.05)
        except Exception as e:  # noqa: BLE001
            logger.warning("fault injection failed: %r", e)

    def check_weights(self, action: str):
        return actors.get([e.weights_checker.remote(action=action) for e in self.rollout_engines if e is not None])

    def dispose(self):
        for m in self._health_monitors:
            m.stop()
        for s in self.servers.values():
            for e in s.all_engines:
                if e is not None:
                    try:
                        actors.get(e.shutdown.remote(), timeout=10)
                    except Exception:  # noqa: BLE001
                        pass
                    actors.kill(e)
            if s.router is not None:
                s.router.shutdown()
        actors.kill(self.rollout_engine_lock)
        for refs in self._live_refs:
            for r in refs:
                object_store.free(r.inner)
        logging_utils.finish_tracking(self.args)
        # per-process rollout state (router address, semaphores, pending tasks) belongs to this manager's args: a
        # manager created later in the same process must not inherit it
        try:
            from slime_b200.rollout.sglang_rollout import GenerateState

            GenerateState.clear_instances()
        except Exception:  # noqa: BLE001
            pass


actors.remote(RolloutManager)
