"""Rollout-side metrics: ``rollout/*`` (response lengths, zero-std groups, prefix-cache hit rate, speculative
acceptance, top-p kept vocabulary, repetition, truncation), ``perf/*`` (tokens per GPU per second, longest-sample
speed, per-request engine timings taken from the ``sglang_generate`` trace span) and ``eval/*``.
Parity: slime/observability/rollout_metrics.py:45-271 (same keys).
"""

from __future__ import annotations

import logging
import math
from typing import Any

import numpy as np

from slime_b200.observability import logging_utils
from slime_b200.observability.metric_utils import (compute_pass_rate, compute_rollout_step, compute_statistics,
                                                   dict_add_prefix, has_repetition)  # fmt: skip
from slime_b200.utils.misc import group_by, load_function
from slime_b200.utils.types import Sample

logger = logging.getLogger(__name__)

# metric key -> attribute on the generate span
_REQUEST_FIELDS = {
    "request/e2e_latency": "e2e_latency", "request/queue_time": "queue_time", "decode/throughput": "decode_throughput",
    "prefill/bootstrap_queue_duration": "pd_prefill_bootstrap_queue_duration",
    "prefill/bootstrap_duration": "pd_prefill_bootstrap_duration",
    "prefill/alloc_wait_duration": "pd_prefill_alloc_wait_duration",
    "prefill/forward_duration": "pd_prefill_forward_duration",
    "prefill/transfer_queue_duration": "pd_prefill_transfer_queue_duration",
    "prefill/transfer_speed_gb_s": "pd_transfer_speed_gb_s", "prefill/transfer_total_mb": "pd_transfer_total_mb",
    "prefill/retry_count": "pd_prefill_retry_count", "decode/prealloc_duration": "pd_decode_prealloc_duration",
    "decode/bootstrap_duration": "pd_decode_bootstrap_duration", "decode/alloc_wait_duration": "pd_decode_alloc_wait_duration",
    "decode/transfer_duration": "pd_decode_transfer_duration", "decode/forward_duration": "pd_decode_forward_duration",
}  # fmt: skip


def _zero_std(args, samples) -> dict:
    if args.advantage_estimator == "ppo":
        return {}
    counts: dict[str, int] = {}
    for g in group_by(samples, lambda s: s.group_index).values():
        rewards = [s.get_reward_value(args) for s in g]
        if all(r == rewards[0] for r in rewards):
            key = f"zero_std/count_{round(rewards[0], 1)}"
            counts[key] = counts.get(key, 0) + 1
    return counts


def _spec(args, samples) -> dict:
    if getattr(args, "sglang_speculative_algorithm", None) is None:
        return {}
    n = len(samples)
    return {"spec_accept_rate": sum(s.spec_info.spec_accept_rate for s in samples) / n,
            "spec_accept_length": sum(s.spec_info.spec_accept_length for s in samples) / n}  # fmt: skip


def _prefix_cache(samples) -> dict:
    cached = sum(s.prefix_cache_info.cached_tokens for s in samples)
    total = sum(s.prefix_cache_info.total_prompt_tokens for s in samples)
    return {"prefix_cache_hit_rate": cached / total if total else 0.0, "avg_cached_tokens_per_sample": cached / len(samples)}


def _reward_cat(args, samples) -> dict:
    key = getattr(args, "log_reward_category", None)
    if key is None:
        return {}
    return {f"error_cat/{cat}": len(g) / len(samples) for cat, g in group_by(samples, lambda s: s.reward[key]).items()}


def _top_p_kept(samples) -> dict:
    kept = tokens = 0
    for s in samples:
        offs = s.rollout_top_p_token_offsets
        if offs is None or s.response_length == 0 or s.remove_sample:
            continue
        offs = np.asarray(offs, dtype=np.int64)
        if offs.size == 0:
            continue
        if offs.size != s.response_length + 1:
            raise ValueError(f"top-p offsets length {offs.size} != response length + 1 ({s.response_length + 1})")
        per_tok = np.diff(offs)
        if s.loss_mask is None:
            kept, tokens = kept + int(per_tok.sum()), tokens + s.response_length
        else:
            m = np.asarray(s.loss_mask, dtype=bool)
            kept, tokens = kept + int(per_tok[m].sum()), tokens + int(m.sum())
    return {"top_p_kept_vocab_per_token": kept / tokens} if tokens else {}


def compute_metrics_from_samples(args, samples: list[Sample]) -> dict:
    out = dict_add_prefix(compute_statistics([s.effective_response_length for s in samples]), "response_len/")
    out |= _zero_std(args, samples) | _spec(args, samples) | _prefix_cache(samples) | _reward_cat(args, samples)
    out |= _top_p_kept(samples)
    out["repetition_frac"] = float(np.mean([has_repetition(s.response) for s in samples]))
    out["truncated_ratio"] = float(np.mean([s.status == Sample.Status.TRUNCATED for s in samples]))
    return out


def _request_perf(samples) -> dict:
    vals: dict[str, list[float]] = {}
    for s in samples:
        tr = getattr(s, "trace", None)
        if not isinstance(tr, dict):
            continue
        for ev in tr.get("events") or []:
            if ev.get("type") != "span_end" or ev.get("name") != "sglang_generate" or not isinstance(ev.get("attrs"), dict):
                continue
            for key, src in _REQUEST_FIELDS.items():
                v = ev["attrs"].get(src)
                if isinstance(v, (int, float)) and not isinstance(v, bool) and math.isfinite(v):
                    vals.setdefault(key, []).append(float(v))
    out = {}
    for key, v in vals.items():
        out |= dict_add_prefix(compute_statistics(v), f"{key}/")
    return out


def compute_perf_metrics_from_samples(args, samples, rollout_time: float) -> dict:
    idle = [s.non_generation_time for s in samples]
    out = {"rollout_time": rollout_time}
    if max(idle) > 0:
        out |= dict_add_prefix(compute_statistics(idle), "non_generation_time/")
    for key, lens in (("", [s.response_length for s in samples]), ("effective_", [s.effective_response_length for s in samples])):
        longest = max(lens)
        if args.rollout_num_gpus:
            out[f"{key}tokens_per_gpu_per_sec"] = sum(lens) / rollout_time / args.rollout_num_gpus
        out[f"longest_{key}sample_tokens_per_sec"] = longest / rollout_time
        if max(idle) > 0:
            t = [i for i, n in zip(idle, lens, strict=True) if n == longest]
            mean_idle = sum(t) / len(t)
            out[f"longest_{key}sample_non_generation_time"] = mean_idle
            out[f"longest_{key}sample_tokens_per_sec_without_non_generation"] = longest / (rollout_time - mean_idle)
    return out | _request_perf(samples)


def log_rollout_data(rollout_id, args, samples, rollout_extra_metrics, rollout_time) -> dict | None:
    if getattr(args, "custom_rollout_log_function_path", None):
        if load_function(args.custom_rollout_log_function_path)(rollout_id, args, samples, rollout_extra_metrics, rollout_time):
            return None
    if getattr(args, "load_debug_rollout_data", None):
        return None
    log = dict(rollout_extra_metrics or {})
    log |= dict_add_prefix(compute_metrics_from_samples(args, samples), "rollout/")
    log |= dict_add_prefix(compute_perf_metrics_from_samples(args, samples, rollout_time), "perf/")
    logger.info("perf %s: %s", rollout_id, log)
    log["rollout/step"] = compute_rollout_step(args, rollout_id)
    logging_utils.log(args, log, step_key="rollout/step")
    return log


def log_eval_rollout_data(rollout_id, args, data: dict, extra_metrics: dict[str, Any] | None = None) -> dict | None:
    if getattr(args, "custom_eval_rollout_log_function_path", None):
        if load_function(args.custom_eval_rollout_log_function_path)(rollout_id, args, data, extra_metrics):
            return None
    log = dict(extra_metrics or {})
    for name, d in data.items():
        rewards = d["rewards"]
        log[f"eval/{name}"] = sum(rewards) / len(rewards)
        if d.get("samples") is not None:
            log |= dict_add_prefix(compute_metrics_from_samples(args, d["samples"]), f"eval/{name}/")
        if "truncated" in d:
            log[f"eval/{name}-truncated_ratio"] = sum(d["truncated"]) / len(d["truncated"])
        if getattr(args, "log_passrate", False):
            log |= dict_add_prefix(compute_pass_rate(rewards, args.n_samples_per_eval_prompt), f"eval/{name}-")
    logger.info("eval %s: %s", rollout_id, log)
    log["eval/step"] = compute_rollout_step(args, rollout_id)
    logging_utils.log(args, log, step_key="eval/step")
    return log
