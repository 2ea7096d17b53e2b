"""Replay a saved rollout dump as if it had just been generated, with the engines still running.

    --rollout-function-path slime.rollout.forge_load.generate_rollout --load-forge-rollout-data PATH

``PATH`` is either one file reused by every rollout or a template with ``{rollout_id}`` (the layout
``--save-debug-rollout-data`` writes; a missing training file falls back to rollout 0, eval files are ``eval_<id>``).
Unlike ``--load-debug-rollout-data`` this leaves engines, router, weight sync and the colocated offload / onload cycle
switched on, which is the point: it measures the memory and timing of a full step on a fixed, reproducible batch.
Parity: slime/rollout/forge_load.py:41-114.
"""

from __future__ import annotations

import logging
import os

import torch

from slime_b200.rollout.base_types import RolloutFnEvalOutput, RolloutFnTrainOutput
from slime_b200.utils.types import Sample

logger = logging.getLogger(__name__)


def _dump_path(args, rollout_id: int, evaluation: bool) -> str | None:
    template = getattr(args, "load_forge_rollout_data", None)
    if not template:
        raise RuntimeError("--load-forge-rollout-data is not set (a dump file, or a template with {rollout_id})")
    templated = "{rollout_id}" in template
    if evaluation and not templated:
        return None  # a single literal file is training data
    path = template.format(rollout_id=f"eval_{rollout_id}" if evaluation else str(rollout_id))
    if os.path.exists(path):
        return path
    if not evaluation:
        first = template.format(rollout_id="0")
        if os.path.exists(first):
            logger.info("forge_load: %s is missing, replaying %s instead", path, first)
            return first
    return None


def _load(path: str) -> list[Sample]:
    return [Sample.from_dict(d) for d in torch.load(path, weights_only=False)["samples"]]


def generate_rollout(args, rollout_id, data_source, evaluation: bool = False):
    path = _dump_path(args, rollout_id, evaluation)
    if evaluation:
        if path is None:
            logger.info("forge_load: no eval dump for rollout %d, returning an empty result", rollout_id)
            return RolloutFnEvalOutput(data={})
        samples = _load(path)
        key = args.eval_reward_key or args.reward_key
        rewards = [0.0 if s.reward is None else (s.reward[key] if key else s.reward) for s in samples]
        return RolloutFnEvalOutput(data={"forge_eval": {
            "rewards": rewards, "truncated": [s.status == Sample.Status.TRUNCATED for s in samples], "samples": samples}})  # fmt: skip
    if path is None:
        raise RuntimeError(f"forge_load: no dump for rollout {rollout_id} under {args.load_forge_rollout_data!r}")
    samples = _load(path)
    logger.info("forge_load: %d samples for rollout %d from %s", len(samples), rollout_id, os.path.basename(path))
    return RolloutFnTrainOutput(samples=samples)
