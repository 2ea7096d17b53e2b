"""Per-dataset evaluation settings (``--eval-config`` YAML / ``--eval-prompt-data``).

Resolution order for every field: dataset entry > ``eval.defaults`` > the
matching CLI flags (eval-specific flag first, rollout flag second).
Parity: slime/utils/eval_config.py:135 (EvalDatasetConfig), :216, :259.
"""

from __future__ import annotations

from collections.abc import Iterable
from dataclasses import dataclass, field, fields
from typing import Any

# field -> CLI attributes consulted (in order) when neither dataset nor defaults set it
_ARG_FALLBACKS: dict[str, tuple[str, ...]] = {
    "n_samples_per_eval_prompt": ("n_samples_per_eval_prompt", "n_samples_per_prompt"),
    "temperature": ("eval_temperature", "rollout_temperature"),
    "top_p": ("eval_top_p", "rollout_top_p"),
    "top_k": ("eval_top_k", "rollout_top_k"),
    "max_response_len": ("eval_max_response_len", "rollout_max_response_len"),
    "min_eval_samples": (),
    "stop": ("rollout_stop",),
    "stop_token_ids": ("rollout_stop_token_ids",),
    "min_new_tokens": ("eval_min_new_tokens",),
    "input_key": ("eval_input_key", "input_key"),
    "label_key": ("eval_label_key", "label_key"),
    "tool_key": ("eval_tool_key", "tool_key"),
    "metadata_key": ("metadata_key",),
    "multimodal_keys": ("multimodal_keys",),
    "apply_chat_template": ("apply_chat_template",),
    "apply_chat_template_kwargs": ("apply_chat_template_kwargs",),
    "custom_rm_path": ("eval_custom_rm_path", "custom_rm_path"),
}


def pick_from_args(args: Any, attrs: tuple[str, ...]) -> Any:
    for a in attrs:
        v = getattr(args, a, None)
        if v is not None:
            return v
    return None


@dataclass
class EvalDatasetConfig:
    """Settings of one evaluation dataset."""

    name: str
    path: str
    rm_type: str | None = None
    custom_rm_path: str | None = None
    input_key: str | None = None
    label_key: str | None = None
    tool_key: str | None = None
    metadata_key: str | None = None
    multimodal_keys: dict[str, str] | None = None
    apply_chat_template: bool | None = None
    apply_chat_template_kwargs: dict[str, Any] | None = None
    n_samples_per_eval_prompt: int | None = None
    temperature: float | None = None
    top_p: float | None = None
    top_k: int | None = None
    max_response_len: int | None = None
    stop: list[str] | None = None
    stop_token_ids: list[int] | None = None
    min_new_tokens: int | None = None
    repetition_penalty: float | None = None
    skip_special_tokens: bool | None = None
    no_stop_trim: bool | None = None
    custom_generate_function_path: str | None = None
    app_service: str | None = None
    eval_task_timeout: int | None = None
    min_eval_samples: int | None = None
    eval_early_stop_remaining: int | None = None
    eval_early_stop_idle_timeout: float | None = None
    message_processor: dict[str, Any] | None = None
    reward_model: dict[str, Any] | None = None
    remote_environment: dict[str, Any] | None = None
    metadata_overrides: dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if self.metadata_overrides is None:
            self.metadata_overrides = {}
        if not isinstance(self.metadata_overrides, dict):
            raise TypeError("metadata_overrides must be a mapping.")
        if self.min_eval_samples is not None and self.min_eval_samples <= 0:
            raise ValueError("min_eval_samples must be positive when set.")

    @property
    def cache_key(self) -> tuple[Any, ...]:
        return (self.name, self.path, self.input_key, self.label_key, self.tool_key, self.metadata_key)

    def inject_metadata(self, sample_metadata: Any) -> dict[str, Any]:
        md = dict(sample_metadata) if isinstance(sample_metadata, dict) else {}
        if self.rm_type is not None:
            md["rm_type"] = self.rm_type
        md.update(self.metadata_overrides)
        return md


def ensure_dataset_list(config: Any) -> list[dict[str, Any]]:
    """Accept a list of dataset dicts or a mapping ``name -> dict``."""
    if config is None:
        return []
    if isinstance(config, dict):
        return [{**(cfg or {}), "name": (cfg or {}).get("name", name)} for name, cfg in config.items()]
    if isinstance(config, (list, tuple)):
        out = []
        for item in config:
            d = dict(item or {})
            if "name" not in d:
                raise ValueError("Each evaluation dataset entry must include a `name` field.")
            out.append(d)
        return out
    raise TypeError("eval.datasets must be either a list or a mapping.")


def build_eval_dataset_configs(args: Any, raw_config: Iterable[dict[str, Any]], defaults: dict[str, Any]):
    defaults = defaults or {}
    valid = {f.name for f in fields(EvalDatasetConfig)} | set(_ARG_FALLBACKS)
    unknown = set(defaults) - valid
    if unknown:
        raise ValueError(f"Unknown key(s) in eval.defaults: {sorted(unknown)}. Valid keys: {sorted(valid)}.")
    out = []
    for cfg in raw_config:
        d = dict(cfg or {})
        for name, arg_attrs in _ARG_FALLBACKS.items():
            if name in d:
                continue
            d[name] = defaults[name] if name in defaults else pick_from_args(args, arg_attrs)
        for k, v in defaults.items():
            d.setdefault(k, v)
        out.append(EvalDatasetConfig(**d))
    return out
