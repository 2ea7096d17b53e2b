"""Small metric helpers shared by rollout / eval / train logging.

Metric names match slime/observability/metric_utils.py:11-137 so dashboards built for the reference keep
working: ``pass@k`` uses the unbiased estimator 1 - C(n-c, k)/C(n, k); repetition is flagged when the last
10k characters of a response compress more than 10x.
"""

from __future__ import annotations

import math
import zlib
from typing import Any

import numpy as np


def dict_add_prefix(d: dict[str, Any], prefix: str) -> dict[str, Any]:
    return {prefix + k: v for k, v in d.items()}


def compute_statistics(values) -> dict[str, float]:
    v = np.asarray(values, dtype=np.float64)
    return {"mean": float(v.mean()), "median": float(np.median(v)), "max": float(v.max()), "min": float(v.min())}


def _pass_at_k(n: int, c: int, k: int) -> float:
    if n - c < k:
        return 1.0
    # 1 - prod_{i=n-c+1..n} (1 - k/i), evaluated in log space for long groups
    i = np.arange(n - c + 1, n + 1, dtype=np.float64)
    return float(1.0 - np.exp(np.log1p(-k / i).sum()))


def compute_pass_rate(flat_rewards, group_size: int, num_groups: int | None = None) -> dict[str, float]:
    if group_size == 1:
        return {}
    num_groups = len(flat_rewards) // group_size if num_groups is None else num_groups
    if len(flat_rewards) != num_groups * group_size:
        raise ValueError(f"{len(flat_rewards)} rewards do not form {num_groups} groups of {group_size}")
    correct = (np.asarray(flat_rewards).reshape(num_groups, group_size) == 1).sum(axis=1)
    out = {}
    for e in range(int(math.log2(group_size)) + 1):
        k = 1 << e
        out[f"pass@{k}"] = float(np.mean([_pass_at_k(group_size, int(c), k) for c in correct]))
    return out


def compression_ratio(data: str | bytes, level: int = 9) -> tuple[float, float]:
    raw = data.encode("utf-8") if isinstance(data, str) else data
    if not raw:
        return float("inf"), 0.0
    comp = len(zlib.compress(raw, level))
    return len(raw) / comp, 100.0 * (1.0 - comp / len(raw))


def has_repetition(text: str | None) -> bool:
    return bool(text) and len(text) > 10000 and compression_ratio(text[-10000:])[0] > 10


def compute_rollout_step(args, rollout_id: int) -> int:
    if getattr(args, "wandb_always_use_train_step", False):
        return rollout_id * args.rollout_batch_size * args.n_samples_per_prompt // args.global_batch_size
    return rollout_id
