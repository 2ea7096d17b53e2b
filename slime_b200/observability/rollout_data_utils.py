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


def validate_rollout_routed_experts_for_replay(routed_experts, args) -> None:
    """Refuse expert-route records that rollout routing replay cannot use: a wrong shape, no rows, or a mixture-of-experts
    layer whose routes are zero for every token (an engine stage that did not report its layers: replaying that would send
    every token to expert 0). Dense layers are zero by construction. Parity:
    slime/observability/rollout_data_utils.py:55-89 in the reference."""
    if not routed_experts:
        raise ValueError("R3 is enabled but no rollout routed-experts tensors were returned.")
    layers, topk = int(args.num_layers), int(args.moe_router_topk)
    freq = getattr(args, "moe_layer_freq", None)
    moe_layers = [i for i, f in enumerate(freq[:layers]) if int(f) != 0] if isinstance(freq, (list, tuple)) else list(range(layers))
    for n, routes in enumerate(routed_experts):
        routes = torch.as_tensor(routes)
        if routes.ndim != 3 or tuple(routes.shape[1:]) != (layers, topk):
            raise ValueError(f"Invalid rollout routed-experts shape for R3: sample={n}, got={tuple(routes.shape)}, expected=(*, {layers}, {topk}).")
        if routes.shape[0] == 0:
            raise ValueError(f"R3 sample {n} has no routed-experts rows.")
        if topk > 1:  # with one route per token "all zero" can be a real answer
            missing = [i for i in moe_layers if not torch.count_nonzero(routes[:, i, :])]
            if missing:
                raise ValueError(f"R3 routed-experts capture is all zero for MoE layers {missing} in sample {n}: the rollout "
                                 "engine's stages did not report these layers; refusing to replay expert 0 everywhere.")  # fmt: skip


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
