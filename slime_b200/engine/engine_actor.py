"""Rollout-engine actor: owns one engine server (HTTP) and exposes its control surface as methods.

Replaces ``SGLangEngine`` (slime/backends/sglang_utils/sglang_engine.py:88-503): compute the server
arguments from ``--sglang-*`` flags and YAML overrides, start the server, wait for ``/health_generate``,
register with the router (``POST /workers``), and forward control calls. In this framework the engine runs
*inside* the actor's process (no second subprocess), so the HTTP listener and the scheduler thread live
next to the actor's RPC loop. ``simulate_crash`` is host-side fault injection: it stops the server and
makes every later call fail, nothing is done to the GPU.
"""

from __future__ import annotations

import dataclasses
import logging
import time

import requests

from slime_b200.engine.server_args import ServerArgs

logger = logging.getLogger(__name__)


def get_base_gpu_id(args, rank: int) -> int:
    per = args.rollout_num_gpus_per_engine
    n = min(args.num_gpus_per_node, per)
    return (rank * per) % args.num_gpus_per_node if per <= args.num_gpus_per_node else 0 if n else 0


def compute_server_args(args, rank: int, host: str, port: int, nccl_port: int | None = None, dist_init_addr: str | None = None,
                        worker_type: str = "regular", base_gpu_id: int | None = None, overrides: dict | None = None,
                        model_path: str | None = None) -> tuple[ServerArgs, list[str]]:  # fmt: skip
    """Server arguments the framework always forces, then every ``--sglang-<field>`` given on the CLI, then
    YAML ``overrides`` (which win). The second value lists the fields an external engine must agree on."""
    pp = getattr(args, "sglang_pp_size", None) or 1
    kw = dict(
        model_path=model_path or args.hf_checkpoint, trust_remote_code=True,
        random_seed=args.seed + rank * args.num_gpus_per_node, enable_memory_saver=bool(args.offload_rollout),
        host=host, port=port, nccl_port=nccl_port, nnodes=max(1, args.rollout_num_gpus_per_engine // args.num_gpus_per_node),
        node_rank=0, dist_init_addr=dist_init_addr, base_gpu_id=get_base_gpu_id(args, rank) if base_gpu_id is None else base_gpu_id,
        gpu_id_step=1, tp_size=max(1, args.rollout_num_gpus_per_engine // pp), dp_size=getattr(args, "sglang_dp_size", None) or 1,
        pp_size=pp, ep_size=getattr(args, "sglang_ep_size", None) or 1, skip_server_warmup=True,
        enable_draft_weights_cpu_backup=True, enable_metrics=True,
    )  # fmt: skip
    if worker_type == "prefill":
        kw.update(disaggregation_mode="prefill", load_balance_method="follow_bootstrap_room")
    elif worker_type == "decode":
        kw.update(disaggregation_mode="decode", load_balance_method="prefill_round_robin_balance")
    elif worker_type == "encoder":
        kw.update(encoder_only=True)
    if getattr(args, "use_rollout_routing_replay", False):
        kw["enable_return_routed_experts"] = True
    must_match = ["tp_size", "dp_size", "pp_size", "ep_size", "disaggregation_mode", "model_path"]
    names = {f.name for f in dataclasses.fields(ServerArgs)}
    for k, v in vars(args).items():
        if k.startswith("sglang_") and v is not None:
            field_name = k[len("sglang_") :]
            if field_name in names and field_name not in kw:
                kw[field_name] = v
    for k, v in (overrides or {}).items():
        kw[k] = v
    if kw.get("enable_memory_saver"):
        kw["disable_cuda_graph"] = kw.get("disable_cuda_graph", False)  # decode graphs are re-captured after resume
    unknown = [k for k in kw if k not in names]
    for k in unknown:
        logger.warning("server argument %s is unknown to this engine and is dropped", k)
        kw.pop(k)
    if getattr(args, "load_format", None):
        kw["load_format"] = args.load_format
    return ServerArgs(**kw), must_match


def _wait_server_healthy(url: str, timeout: float = 600.0, is_alive=lambda: True):
    deadline = time.time() + timeout
    while time.time() < deadline:
        try:
            if requests.get(f"{url}/health_generate", timeout=30).status_code == 200:
                return
        except requests.RequestException:
            pass
        if not is_alive():
            raise RuntimeError(f"engine at {url} died during start-up")
        time.sleep(0.5)
    raise TimeoutError(f"engine at {url} not healthy after {timeout}s")


class RolloutEngineActor:
    """One engine = one actor process. ``init`` starts the server; the rest are thin HTTP wrappers so the
    same calls work for engines this framework did not launch (external engines)."""

    def __init__(self, args, rank: int, worker_type: str = "regular", base_gpu_id: int | None = None,
                 overrides: dict | None = None, model_path: str | None = None):  # fmt: skip
        self.args, self.rank, self.worker_type = args, rank, worker_type
        self.base_gpu_id, self.overrides, self.model_path = base_gpu_id, overrides, model_path
        self.server = None
        self.url = None
        self.router = None
        self.worker_id = None
        self.crashed = False

    def init(self, host: str, port: int, nccl_port: int | None = None, dist_init_addr: str | None = None,
             router_ip: str | None = None, router_port: int | None = None, external_url: str | None = None):  # fmt: skip
        from slime_b200.engine.http_server import launch_server

        self.router = (router_ip, router_port) if router_ip else None
        if external_url:
            self.url = external_url.rstrip("/")
        else:
            sa, _ = compute_server_args(self.args, self.rank, host, port, nccl_port, dist_init_addr, self.worker_type,
                                        self.base_gpu_id, self.overrides, self.model_path)  # fmt: skip
            self.server_args = sa
            self.server = launch_server(sa, block=False)
            self.url = self.server.url
        _wait_server_healthy(self.url)
        if self.router is not None:
            r = requests.post(f"http://{router_ip}:{router_port}/workers",
                              json={"url": self.url, "worker_type": self.worker_type,
                                    "bootstrap_port": getattr(getattr(self, "server_args", None), "disaggregation_bootstrap_port", None)},
                              timeout=30)  # fmt: skip
            r.raise_for_status()
            self.worker_id = r.json().get("id")
        return self.url

    # ---------------------------------------------------------------- http plumbing
    def _call(self, path: str, payload: dict | None = None, method: str = "post", timeout: float | None = 600.0):
        if self.crashed:
            raise RuntimeError("engine crashed (simulated)")
        fn = requests.post if method == "post" else requests.get
        kw = {"json": payload or {}} if method == "post" else {}
        r = fn(f"{self.url}{path}", timeout=timeout, **kw)
        r.raise_for_status()
        try:
            return r.json()
        except ValueError:
            return r.text

    def health_generate(self, timeout: float = 30.0) -> bool:
        if self.crashed:
            raise RuntimeError("engine crashed (simulated)")
        r = requests.get(f"{self.url}/health_generate", params={"timeout": timeout}, timeout=timeout + 5)
        r.raise_for_status()
        return True

    def flush_cache(self):
        return self._call("/flush_cache", method="get")

    def pause_generation(self):
        return self._call("/pause_generation")

    def continue_generation(self):
        return self._call("/continue_generation")

    def release_memory_occupation(self, tags: list[str] | None = None):
        self.flush_cache()
        return self._call("/release_memory_occupation", {"tags": tags})

    def resume_memory_occupation(self, tags: list[str] | None = None):
        return self._call("/resume_memory_occupation", {"tags": tags})

    def get_weight_version(self):
        return self._call("/get_weight_version", method="get")["weight_version"]

    def weights_checker(self, action: str):
        return self._call("/weights_checker", {"action": action})

    def update_weights_from_tensor(self, serialized_named_tensors, load_format="flattened_bucket", flush_cache=False, weight_version=None):
        return self._call("/update_weights_from_tensor", {"serialized_named_tensors": serialized_named_tensors,
                                                          "load_format": load_format, "flush_cache": flush_cache,
                                                          "weight_version": weight_version})  # fmt: skip

    def update_weights(self, named_tensors, version=None, flush_cache=False):
        """Same-process fast path used by the colocated updater when it holds a handle to this object."""
        if self.server is None:
            raise RuntimeError("in-process update needs a locally hosted engine")
        return self.server.engine.update_weights(named_tensors, version, flush_cache)

    def update_weights_flat(self, flat, meta: list[tuple], version=None, flush_cache=False):
        """Colocated sync across processes: ``flat`` is one uint8 device buffer (it arrives as a CUDA IPC
        mapping of the trainer's bucket when sent through the actor channel) and ``meta`` lists
        ``(name, dtype string, shape, byte offset)`` views into it. Returns after the copies retired, so the
        trainer may reuse the bucket."""
        import torch

        if self.server is None:
            raise RuntimeError("in-process update needs a locally hosted engine")
        named = []
        for name, dt, shape, off in meta:
            dtype = getattr(torch, dt)
            n = int(torch.Size(shape).numel()) * torch.empty((), dtype=dtype).element_size()
            named.append((name, flat[off : off + n].view(dtype).view(shape)))
        missing = self.server.engine.update_weights(named, version, flush_cache)
        if flat.is_cuda:
            torch.cuda.synchronize(flat.device)
        return missing

    def update_weights_from_disk(self, model_path: str, load_format=None, weight_version=None):
        return self._call("/update_weights_from_disk", {"model_path": model_path, "load_format": load_format,
                                                        "weight_version": weight_version})  # fmt: skip

    def pull_weights(self, local_checkpoint_dir: str, source_dir: str, target_version: int):
        return self._call("/pull_weights", {"local_checkpoint_dir": local_checkpoint_dir, "source_dir": source_dir,
                                            "target_version": target_version})  # fmt: skip

    def init_weights_update_group(self, master_address, master_port, rank_offset, world_size, group_name, backend="nccl"):
        return self._call("/init_weights_update_group", {"master_address": master_address, "master_port": master_port,
                                                         "rank_offset": rank_offset, "world_size": world_size,
                                                         "group_name": group_name, "backend": backend})  # fmt: skip

    def destroy_weights_update_group(self, group_name):
        return self._call("/destroy_weights_update_group", {"group_name": group_name})

    def update_weights_from_distributed(self, names, dtypes, shapes, group_name, weight_version=None, load_format=None, flush_cache=False):
        return self._call("/update_weights_from_distributed", {"names": names, "dtypes": dtypes, "shapes": shapes,
                                                               "group_name": group_name, "weight_version": weight_version,
                                                               "load_format": load_format, "flush_cache": flush_cache})  # fmt: skip

    def post_process_weights(self, restore_weights_before_load=False, post_process_quantization=False):
        return self._call("/post_process_weights", {"restore_weights_before_load": restore_weights_before_load,
                                                    "post_process_quantization": post_process_quantization})  # fmt: skip

    def start_profile(self, **kw):
        return self._call("/start_profile", kw)

    def stop_profile(self):
        return self._call("/stop_profile")

    def get_url(self):
        return self.url

    def parallel_config(self) -> dict:
        sa = getattr(self, "server_args", None)
        return {"tp_size": getattr(sa, "tp_size", 1), "dp_size": getattr(sa, "dp_size", 1), "pp_size": getattr(sa, "pp_size", 1),
                "ep_size": getattr(sa, "ep_size", 1)}  # fmt: skip

    # ------------------------------------------------------------------ lifecycle
    def shutdown(self):
        if self.router is not None and self.worker_id is not None:
            try:
                requests.delete(f"http://{self.router[0]}:{self.router[1]}/workers/{self.worker_id}", timeout=10)
            except requests.RequestException:
                pass
        if self.server is not None:
            self.server.shutdown()
            self.server = None

    def simulate_crash(self):
        """Fault injection for the health monitor (host side only): the server stops answering."""
        logger.warning("simulating a crash of engine %s", self.url)
        self.shutdown()
        self.crashed = True
