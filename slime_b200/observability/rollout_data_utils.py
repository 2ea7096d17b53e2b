"""Debug dumps of rollout data and the ``rollout_id`` contract check.

``--save-debug-rollout-data PATH_{rollout_id}.pt`` stores ``{"rollout_id", "samples": [Sample.to_dict()]}``
(eval dumps use ``eval_<id>``); ``--load-debug-rollout-data`` replays a dump instead of generating, optionally
keeping only the head and tail ``subsample_ratio`` of the rows.
Parity: slime/observability/rollout_data_utils.py:92-153.
"""

from __future__ import annotations

import logging
from pathlib import Path

import torch

from slime_b200.utils.types import Sample

logger = logging.getLogger(__name__)


def validate_rollout_id_annotated(node, depth: int = 0) -> None:
    """A rollout function may return one rollout as several training samples (``list[list[list[Sample]]]``).
    Such sibling lists (depth >= 2, more than one element) must carry one shared non-None ``rollout_id`` so the
    loss reducer counts the rollout once. The ordinary ``list[list[Sample]]`` shape is not checked."""
    if isinstance(node, Sample):
        return
    if not isinstance(node, list):
        raise TypeError(f"unexpected node of type {type(node).__name__} in rollout output")
    if node and isinstance(node[0], Sample):
        if depth >= 2 and len(node) > 1:
            ids = [s.rollout_id for s in node]
            unset = [i for i, r in enumerate(ids) if r is None]
            if unset:
                raise ValueError(f"compact rollout of {len(node)} samples has no rollout_id at positions {unset}; "
                                 "set Sample.rollout_id on every sibling")  # fmt: skip
            if len(set(ids)) != 1:
                raise ValueError(f"samples of one compact rollout must share rollout_id, got {ids}")
        return
    for child in node:
        validate_rollout_id_annotated(child, depth + 1)


def save_debug_rollout_data(path_template: str | None, data, *, rollout_id: int, evaluation: bool) -> None:
    if path_template is None:
        return
    path = Path(path_template.format(rollout_id=f"eval_{rollout_id}" if evaluation else str(rollout_id)))
    path.parent.mkdir(parents=True, exist_ok=True)
    if evaluation:
        samples = [s.to_dict() for info in data.values() for s in info["samples"]]
    else:
        samples = [s.to_dict() for s in data]
    logger.info("saving %d debug rollout samples to %s", len(samples), path)
    torch.save({"rollout_id": rollout_id, "samples": samples}, path)


def load_debug_rollout_data(path_template: str, *, rollout_id: int, subsample_ratio: float | None = None) -> list[Sample]:
    rows = torch.load(path_template.format(rollout_id=rollout_id), weights_only=False)["samples"]
    samples = [Sample.from_dict(r) for r in rows]
    if subsample_ratio is not None:
        keep = int(len(samples) * subsample_ratio)
        head, tail = keep // 2, keep - keep // 2
        samples = samples[:head] + (samples[-tail:] if tail else [])
        logger.info("debug rollout data subsampled %d -> %d rows", len(rows), len(samples))
    return samples
