"""Dynamic-sampling filter protocol (parity: slime/rollout/filter_hub/base_types.py:6-53)."""

from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass


@dataclass
class DynamicFilterOutput:
    keep: bool
    reason: str | None = None
    keep_when_insufficient: bool = False  # fallback pool when not enough groups pass


def should_drop_dynamic_filter_output(output) -> bool:
    return not (output.keep if isinstance(output, DynamicFilterOutput) else bool(output))


def call_dynamic_filter(fn, *args, **kwargs) -> DynamicFilterOutput:
    if fn is None:
        return DynamicFilterOutput(keep=True)
    out = fn(*args, **kwargs)
    if not isinstance(out, DynamicFilterOutput):
        out = DynamicFilterOutput(keep=bool(out))
    return out


class MetricGatherer:
    """Counts drop reasons over one rollout: ``rollout/dynamic_filter/drop_<reason>``."""

    def __init__(self):
        self._drops = defaultdict(int)

    def on_dynamic_filter_drop(self, reason: str | None):
        if reason:
            self._drops[reason] += 1

    def collect(self):
        return {f"rollout/dynamic_filter/drop_{k}": v for k, v in self._drops.items()}
