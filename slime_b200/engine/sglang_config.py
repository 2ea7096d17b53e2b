"""Multi-model / multi-group rollout deployment described in YAML (``--sglang-config``).

    sglang:
      - name: actor
        model_path: /ckpt/policy          # defaults to --hf-checkpoint
        update_weights: true              # inferred: model_path == --hf-checkpoint
        server_groups:
          - {worker_type: regular, num_gpus: 4, num_gpus_per_engine: 2, overrides: {mem_fraction_static: 0.8}}
      - name: reward
        model_path: /ckpt/rm
        server_groups: [{worker_type: regular, num_gpus: 2}]

Each model gets its own router; only models with ``update_weights`` take part in weight sync;
``sum(num_gpus) == --rollout-num-gpus``; ``regular`` groups cannot be mixed with ``prefill``/``decode``
groups inside one model. Parity: slime/backends/sglang_utils/sglang_config.py:11-207.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import yaml

WORKER_TYPES = ("regular", "prefill", "decode", "encoder", "placeholder")


@dataclass
class ServerGroupConfig:
    worker_type: str = "regular"
    num_gpus: int = 0
    num_gpus_per_engine: int | None = None
    overrides: dict = field(default_factory=dict)
    name: str | None = None

    def __post_init__(self):
        if self.worker_type not in WORKER_TYPES:
            raise ValueError(f"unknown worker_type {self.worker_type!r}; expected one of {WORKER_TYPES}")
        if self.num_gpus < 0:
            raise ValueError("num_gpus must be >= 0")


@dataclass
class ModelConfig:
    name: str
    model_path: str | None = None
    update_weights: bool | None = None
    server_groups: list[ServerGroupConfig] = field(default_factory=list)
    router_overrides: dict = field(default_factory=dict)

    def resolve(self, args) -> None:
        if self.model_path is None:
            self.model_path = args.hf_checkpoint
        if self.update_weights is None:
            self.update_weights = self.model_path == args.hf_checkpoint
        kinds = {g.worker_type for g in self.server_groups if g.worker_type != "placeholder"}
        if "regular" in kinds and kinds & {"prefill", "decode"}:
            raise ValueError(f"model {self.name}: regular groups cannot be mixed with prefill/decode groups")
        if ("prefill" in kinds) != ("decode" in kinds):
            raise ValueError(f"model {self.name}: prefill and decode groups must come together")
        for g in self.server_groups:
            if g.num_gpus_per_engine is None:
                g.num_gpus_per_engine = args.rollout_num_gpus_per_engine
            if g.worker_type != "placeholder" and g.num_gpus % g.num_gpus_per_engine != 0:
                raise ValueError(f"model {self.name}: group num_gpus {g.num_gpus} not divisible by num_gpus_per_engine")

    @property
    def num_gpus(self) -> int:
        return sum(g.num_gpus for g in self.server_groups)

    @property
    def has_pd_disaggregation(self) -> bool:
        return any(g.worker_type == "prefill" for g in self.server_groups)


@dataclass
class SglangConfig:
    models: list[ModelConfig]

    @classmethod
    def from_yaml(cls, path: str, args=None) -> "SglangConfig":
        with open(path) as f:
            doc = yaml.safe_load(f) or {}
        entries = doc.get("sglang", doc.get("models", doc if isinstance(doc, list) else []))
        models = []
        for e in entries:
            groups = [ServerGroupConfig(**g) for g in e.get("server_groups", [])]
            models.append(ModelConfig(name=e["name"], model_path=e.get("model_path"), update_weights=e.get("update_weights"),
                                      server_groups=groups, router_overrides=e.get("router", {}) or {}))  # fmt: skip
        cfg = cls(models)
        if args is not None:
            cfg.resolve(args)
        return cfg

    @classmethod
    def from_prefill_num_servers(cls, args) -> "SglangConfig":
        """Single model; ``--prefill-num-servers N`` splits the engines into N prefill servers and the rest decode."""
        per = args.rollout_num_gpus_per_engine
        total = args.rollout_num_gpus
        n_pre = getattr(args, "prefill_num_servers", None)
        if n_pre:
            groups = [ServerGroupConfig("prefill", n_pre * per, per), ServerGroupConfig("decode", total - n_pre * per, per)]
        else:
            groups = [ServerGroupConfig("regular", total, per)]
        cfg = cls([ModelConfig(name="default", model_path=args.hf_checkpoint, update_weights=True, server_groups=groups)])
        cfg.resolve(args)
        return cfg

    def resolve(self, args) -> None:
        names = [m.name for m in self.models]
        if len(set(names)) != len(names):
            raise ValueError(f"duplicate model names in sglang config: {names}")
        for m in self.models:
            m.resolve(args)
        total = sum(m.num_gpus for m in self.models)
        if args.rollout_num_gpus is not None and total != args.rollout_num_gpus:
            raise ValueError(f"sglang config places {total} GPUs but --rollout-num-gpus is {args.rollout_num_gpus}")

    @property
    def updatable_models(self) -> list[ModelConfig]:
        return [m for m in self.models if m.update_weights]
