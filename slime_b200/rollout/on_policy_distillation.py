"""On-policy distillation with a teacher behind an engine endpoint (``--use-opd --opd-type sglang``).

``reward_func`` sends the student's full token sequence to the teacher (``--rm-url``, a ``/generate`` endpoint) with
``max_new_tokens = 0`` and ``return_logprob`` so the teacher only scores it; ``post_process_rewards`` keeps the last
``response_length`` teacher log-probs on ``sample.teacher_log_probs`` and returns zero scalar rewards: the learning
signal is the reverse-KL penalty added to the advantages by the trainer.
Parity: slime/rollout/on_policy_distillation.py:8-67.
"""

from __future__ import annotations

import aiohttp
import torch

from slime_b200.utils.types import Sample


async def reward_func(args, sample: Sample, **kwargs):
    payload = {
        "input_ids": sample.tokens,
        "sampling_params": {"temperature": args.rollout_temperature, "max_new_tokens": 0, "skip_special_tokens": False},
        "return_logprob": True,
        "logprob_start_len": 0,
    }
    images = (sample.multimodal_inputs or {}).get("images") if sample.multimodal_inputs else None
    if images:
        from slime_b200.utils.processing_utils import encode_image_for_rollout_engine

        payload["image_data"] = [encode_image_for_rollout_engine(im) for im in images]
    async with aiohttp.ClientSession() as session:
        async with session.post(args.rm_url, json=payload) as resp:
            resp.raise_for_status()
            return await resp.json()


def post_process_rewards(args, samples: list[Sample], **kwargs):
    for s in samples:
        scored = s.get_reward_value(args)["meta_info"]["input_token_logprobs"]
        lp = torch.tensor([item[0] for item in scored[1:]], dtype=torch.float32)  # the first token has no log-prob
        s.teacher_log_probs = lp[-s.response_length :] if s.response_length else lp[:0]
    zeros = [0.0] * len(samples)
    return zeros, zeros
