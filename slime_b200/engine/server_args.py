"""Rollout-engine server arguments.

Every field is exposed on the trainer CLI as ``--sglang-<field>`` (the prefix
is kept so existing launch recipes run unchanged; parity:
slime/backends/sglang_utils/arguments.py:41-144). Fields the engine does not
use are accepted for compatibility and ignored with a warning at start-up.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass


@dataclass
class ServerArgs:
    model_path: str | None = None
    tokenizer_path: str | None = None
    trust_remote_code: bool = True
    dtype: str = "bfloat16"
    kv_cache_dtype: str = "auto"
    quantization: str | None = None  # None | "fp8" (128x128 block-scaled e4m3)
    context_length: int | None = None
    host: str = "127.0.0.1"
    port: int = 30000
    nccl_port: int | None = None
    dist_init_addr: str | None = None
    nnodes: int = 1
    node_rank: int = 0
    base_gpu_id: int = 0
    gpu_id_step: int = 1
    tp_size: int = 1
    dp_size: int = 1
    pp_size: int = 1
    ep_size: int = 1
    random_seed: int = 0
    mem_fraction_static: float = 0.85
    max_running_requests: int = 512
    max_total_tokens: int | None = None
    max_prefill_tokens: int = 16384
    chunked_prefill_size: int = 8192
    page_size: int = 16
    schedule_policy: str = "fcfs"
    disable_radix_cache: bool = False
    disable_cuda_graph: bool = False
    cuda_graph_max_bs: int = 256
    cuda_graph_bs: list[int] | None = None
    enable_memory_saver: bool = False
    enable_metrics: bool = True
    skip_server_warmup: bool = True
    enable_return_routed_experts: bool = False
    enable_deterministic_inference: bool = False
    enable_fp32_moe_router: bool = False
    attention_backend: str = "b200"
    sampling_backend: str = "b200"
    moe_a2a_backend: str = "p2p"
    deepep_mode: str = "auto"
    moe_dense_tp_size: int | None = None
    enable_dp_attention: bool = False
    enable_dp_lm_head: bool = False
    disaggregation_mode: str = "null"  # null | prefill | decode
    disaggregation_bootstrap_port: int = 8998
    disaggregation_transfer_backend: str = "p2p"
    disaggregation_ib_device: str | None = None
    load_balance_method: str = "round_robin"
    speculative_algorithm: str | None = None
    speculative_num_steps: int = 3
    speculative_eagle_topk: int = 1
    speculative_num_draft_tokens: int = 4
    speculative_draft_model_path: str | None = None
    speculative_draft_attention_backend: str | None = None
    enable_draft_weights_cpu_backup: bool = True
    watchdog_timeout: float = 300.0
    log_level: str = "warning"
    encoder_only: bool = False
    language_only: bool = False
    disable_overlap_schedule: bool = False
    nsa_prefill_backend: str | None = None
    nsa_decode_backend: str | None = None
    mamba_scheduler_strategy: str | None = None
    enable_hierarchical_cache: bool = False  # evicted prefix pages move to pinned host memory instead of being dropped
    hicache_ratio: float = 2.0  # host pages per device page
    hicache_size: int = 0  # host pool in GB (overrides the ratio when > 0)
    release_hicache: bool = False
    weight_version: str = "default"
    load_format: str = "auto"  # auto | dummy (random init)
    server_concurrency: int = 512
    config: str | None = None  # YAML topology (--sglang-config)

    def url(self) -> str:
        return f"http://{self.host}:{self.port}"

    @classmethod
    def from_kwargs(cls, **kw) -> "ServerArgs":
        names = {f.name for f in dataclasses.fields(cls)}
        unknown = sorted(set(kw) - names)
        if unknown:
            import logging

            logging.getLogger(__name__).warning("dropping server args unknown to this engine: %s", unknown)
        return cls(**{k: v for k, v in kw.items() if k in names})


# fields set by the framework itself, never by --sglang-* flags
SKIPPED_FIELDS = {
    "model_path", "trust_remote_code", "random_seed", "enable_memory_saver", "host", "port", "nccl_port", "nnodes",
    "node_rank", "dist_init_addr", "base_gpu_id", "gpu_id_step", "tp_size", "skip_server_warmup", "enable_metrics",
    "enable_return_routed_experts",
}  # fmt: skip

ROUTER_FLAGS = [
    ("--sglang-router-ip", dict(type=str, default=None)),
    ("--sglang-router-port", dict(type=int, default=None)),
    ("--sglang-router-request-timeout-secs", dict(type=int, default=14400)),
    ("--sglang-router-policy", dict(type=str, default=None)),
    ("--router-policy", dict(type=str, default="cache_aware", choices=["cache_aware", "round_robin", "random", "power_of_two", "consistent_hashing"])),
    ("--router-balance-abs-threshold", dict(type=int, default=32)),
    ("--router-balance-rel-threshold", dict(type=float, default=1.1)),
    ("--use-slime-router", dict(action="store_true")),
    ("--prefill-num-servers", dict(type=int, default=None)),
]
