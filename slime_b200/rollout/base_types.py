"""Return types of rollout functions (parity: slime/rollout/base_types.py:7-26)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from slime_b200.utils.types import Sample


@dataclass
class RolloutFnTrainOutput:
    samples: list[list[Sample]]
    metrics: dict[str, Any] | None = None


@dataclass
class RolloutFnEvalOutput:
    data: dict[str, dict[str, Any]]
    metrics: dict[str, Any] | None = None


def call_rollout_fn(fn, *args, evaluation: bool, **kwargs):
    """Call a rollout function and wrap legacy return shapes (bare list / bare dict)."""
    out = fn(*args, **kwargs, evaluation=evaluation)
    if isinstance(out, (RolloutFnTrainOutput, RolloutFnEvalOutput)):
        return out
    return RolloutFnEvalOutput(data=out) if evaluation else RolloutFnTrainOutput(samples=out)
