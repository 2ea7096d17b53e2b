"""Rollout engines that were launched by someone else (``--rollout-external-engine-addrs host:port ...``).

The framework does not start these servers; it asks each one what it is (``GET /server_info``), derives worker type,
GPU count and parallel layout, puts a thin ``RolloutEngineActor`` in front of each (HTTP only, no GPU) and registers
them with a router. Weight sync then works exactly as for in-house engines (NCCL broadcast group or disk); memory
offload and restart-on-failure do not apply: the processes are not ours to stop.
Parity: slime/backends/sglang_utils/external.py:15-250.
"""

from __future__ import annotations

import dataclasses
import logging
from urllib.parse import urlparse

import requests

logger = logging.getLogger(__name__)


def _first_int(d: dict, *keys, default=None):
    for k in keys:
        if d.get(k):
            return int(d[k])
    return default


@dataclasses.dataclass(frozen=True)
class ExternalEngineInfo:
    url: str
    host: str
    port: int
    worker_type: str
    num_gpus: int
    disaggregation_bootstrap_port: int | None = None
    server_info: dict = dataclasses.field(default_factory=dict)

    @property
    def is_pd_worker(self) -> bool:
        return self.worker_type in ("prefill", "decode")

    @property
    def parallel_config(self) -> dict[str, int]:
        si = self.server_info
        pp = _first_int(si, "pp_size", "pipeline_parallel_size", default=1)
        return {
            "tp_size": _first_int(si, "tp_size", "tensor_parallel_size", default=max(1, self.num_gpus // pp)),
            "pp_size": pp,
            "ep_size": _first_int(si, "ep_size", "expert_parallel_size", default=1),
            "moe_dp_size": _first_int(si, "moe_dp_size", "moe_data_parallel_size", default=1),
        }

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)


def normalize_external_engine_addr(addr: str) -> str:
    """``host:port`` or ``http://host:port`` -> ``http://host:port`` (IPv6 hosts in brackets)."""
    url = (addr if "://" in addr else f"http://{addr}").rstrip("/")
    u = urlparse(url)
    if u.scheme != "http" or u.hostname is None or u.port is None:
        raise ValueError(f"invalid external engine address {addr!r}: expected host:port or http://host:port")
    return url


def get_server_info(url: str, timeout: float = 30.0) -> dict:
    problems = []
    for path in ("/server_info", "/get_server_info"):
        try:
            r = requests.get(url + path, timeout=timeout)
            r.raise_for_status()
            return r.json()
        except Exception as e:  # noqa: BLE001
            problems.append(f"{path}: {e}")
    raise RuntimeError(f"no server info from {url}: {'; '.join(problems)}")


def _infer_worker_type(info: dict) -> str:
    if info.get("encoder_only"):
        return "encoder"
    mode = info.get("disaggregation_mode")
    return mode if mode in ("prefill", "decode") else "regular"


def discover_external_engines(addrs: list[str], timeout: float = 30.0) -> list[ExternalEngineInfo]:
    out = []
    for addr in addrs:
        url = normalize_external_engine_addr(addr)
        u = urlparse(url)
        si = get_server_info(url, timeout)
        pp = _first_int(si, "pp_size", "pipeline_parallel_size", default=1)
        tp = _first_int(si, "tp_size", "tensor_parallel_size", default=1)
        boot = si.get("disaggregation_bootstrap_port")
        out.append(ExternalEngineInfo(url=url, host=u.hostname, port=u.port, worker_type=_infer_worker_type(si),
                                      num_gpus=_first_int(si, "num_gpus", "num_gpus_per_engine", default=tp * pp),
                                      disaggregation_bootstrap_port=None if boot is None else int(boot), server_info=si))  # fmt: skip
    return out


def apply_external_engine_info_to_args(args, logger=None) -> None:
    """Probe the engines once, early, and record the topology on ``args`` (``rollout_num_gpus`` follows from it)."""
    addrs = args.rollout_external_engine_addrs
    if not addrs:
        raise ValueError("--rollout-external-engine-addrs is empty")
    infos = discover_external_engines(addrs)
    args.rollout_external_engine_infos = [i.to_dict() for i in infos]
    args.rollout_num_engines = len(infos)
    args.rollout_num_gpus = sum(i.num_gpus for i in infos)
    if logger is not None:
        logger.info("external engines: %s", [(i.url, i.worker_type, i.num_gpus) for i in infos])


def external_engine_infos_from_args(args) -> list[ExternalEngineInfo]:
    raw = getattr(args, "rollout_external_engine_infos", None)
    if raw is None:
        raise RuntimeError("external engines were not probed: call apply_external_engine_info_to_args first")
    return [ExternalEngineInfo(**r) if isinstance(r, dict) else r for r in raw]


@dataclasses.dataclass
class ExternalRolloutServer:
    """Same surface as ``RolloutServer`` for engines this framework did not start."""

    engines: list
    engine_gpu_counts: list[int]
    engine_gpu_offsets: list[int]
    engine_parallel_configs: list[dict[str, int]]
    router_ip: str | None = None
    router_port: int | None = None
    model_name: str = "default"
    update_weights: bool = True
    num_new_engines: int = 0
    server_groups: list = dataclasses.field(default_factory=list)
    router: object = None

    @property
    def all_engines(self):
        return self.engines

    def recover(self):
        logger.warning("external engines cannot be restarted from here; recover() does nothing")
        return 0

    def offload(self):
        return []

    def onload(self, tags: list[str] | None = None):
        return []

    onload_weights = onload_kv = offload


def start_external_rollout_servers(args, *, start_router, make_engine) -> tuple[dict[str, ExternalRolloutServer], list]:
    """``make_engine(rank, info) -> actor handle``; returns the servers and the pending ``init`` futures."""
    infos = external_engine_infos_from_args(args)
    ip, port, router = start_router(args, has_pd_disaggregation=any(i.is_pd_worker for i in infos))
    args.sglang_router_ip, args.sglang_router_port = ip, port
    engines, counts, offsets, pending, off = [], [], [], [], 0
    for rank, info in enumerate(infos):
        h = make_engine(rank, info)
        engines.append(h)
        counts.append(info.num_gpus)
        offsets.append(off)
        off += info.num_gpus
        pending.append(h.init.remote(info.host, info.port, None, f"{info.host}:{info.port}", ip, port, external_url=info.url))
    args.sglang_model_routers = {"default": (ip, port)}
    srv = ExternalRolloutServer(engines, counts, offsets, [i.parallel_config for i in infos], ip, port, "default", True,
                                len(engines), router=router)  # fmt: skip
    return {"default": srv}, pending
