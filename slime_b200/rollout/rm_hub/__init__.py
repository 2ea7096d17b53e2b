"""Reward dispatch (parity: slime/rollout/rm_hub/__init__.py:34-110).

Priority: per-sample ``custom_rm_path`` > global ``--custom-rm-path`` > ``--rm-type`` (or the
sample's ``metadata['rm_type']``). Built-in types: remote_rm, deepscaler, dapo, math, f1, gpqa,
ifbench, random, and the ``boxed_`` prefix (score the last ``\\boxed{}`` content only).
"""

from __future__ import annotations

import asyncio
import inspect
import random

from slime_b200.utils.misc import load_function
from slime_b200.utils.types import Sample

_session = None


def _get_shared_session():
    global _session
    import aiohttp

    if _session is None or _session.closed:
        _session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=600))
    return _session


async def remote_rm(args, sample: Sample, max_retries: int = 10):
    """POST ``{prompt, response, label}`` to ``--rm-url``; the JSON reply is the reward."""
    payload = {"prompt": sample.prompt, "response": sample.response, "label": sample.label}
    session = _get_shared_session()
    for attempt in range(max_retries):
        try:
            async with session.post(args.rm_url, json=payload) as resp:
                resp.raise_for_status()
                return await resp.json()
        except Exception:
            if attempt == max_retries - 1:
                raise
            await asyncio.sleep(1.0)


async def _call(fn, *a, **k):
    out = fn(*a, **k)
    if inspect.isawaitable(out):
        out = await out
    return out


async def async_rm(args, sample: Sample, **kwargs):
    if sample.custom_rm_path is not None:
        return await _call(load_function(sample.custom_rm_path), args, sample, **kwargs)
    if getattr(args, "custom_rm_path", None) is not None:
        return await _call(load_function(args.custom_rm_path), args, sample, **kwargs)
    md = sample.metadata if isinstance(sample.metadata, dict) else {}
    rm_type = (md.get("rm_type") or getattr(args, "rm_type", None) or "").strip()
    response, label = sample.response, sample.label
    if rm_type.startswith("boxed_"):
        from slime_b200.rollout.rm_hub.math_utils import extract_boxed_answer

        response = extract_boxed_answer(response) or ""
        rm_type = rm_type[len("boxed_") :]
    if rm_type == "remote_rm":
        return await remote_rm(args, sample)
    if rm_type == "deepscaler":
        from slime_b200.rollout.rm_hub.deepscaler import get_deepscaler_rule_based_reward

        return get_deepscaler_rule_based_reward(response, label)
    if rm_type == "dapo":
        from slime_b200.rollout.rm_hub.math_dapo_utils import compute_score

        return compute_score(response, label)
    if rm_type == "math":
        from slime_b200.rollout.rm_hub.math_utils import grade_answer_verl

        return 1 if grade_answer_verl(response, label) else 0
    if rm_type == "f1":
        from slime_b200.rollout.rm_hub.f1 import f1_score

        return f1_score(response, label)[0]
    if rm_type == "gpqa":
        from slime_b200.rollout.rm_hub.gpqa import compute_gpqa_reward

        return compute_gpqa_reward(response, label, metadata=md)
    if rm_type == "ifbench":
        from slime_b200.rollout.rm_hub.ifbench import compute_ifbench_reward

        return compute_ifbench_reward(response, label, metadata=md)
    if rm_type == "random":
        return random.randint(0, 1)
    if rm_type:
        raise NotImplementedError(f"Rule-based RM for {rm_type} is not implemented.")
    raise NotImplementedError("Rule-based RM type is not specified.")


async def batched_async_rm(args, samples: list[Sample], **kwargs) -> list:
    """Group reward: a custom function sees the whole list; otherwise per-sample rewards run concurrently."""
    if getattr(args, "custom_rm_path", None) is not None and getattr(args, "group_rm", False):
        return await _call(load_function(args.custom_rm_path), args, samples, **kwargs)
    return await asyncio.gather(*[async_rm(args, s, **kwargs) for s in samples])
