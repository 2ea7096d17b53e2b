"""Streaming per-sample generation: consume the engine's SSE stream instead of one final JSON body.

    --rollout-function-path slime.rollout.sglang_rollout.generate_rollout \\
    --custom-generate-function-path slime.rollout.sglang_streaming_rollout.generate_streaming

What it buys is robustness to aborts: every chunk is folded into the sample as it arrives, so when partial-rollout
recycling or a weight update cuts generation short the partial tokens, text and log-probs are already on the
sample and nothing depends on the abort call returning them. The surrounding loop (semaphore, abort handling,
buffer hand-off) stays with ``sglang_rollout``.

Chunks are cumulative (each carries the full ``output_token_logprobs`` so far), so a chunk is applied by rewinding
the sample to its state at call entry and appending the whole list again.
Parity: slime/rollout/sglang_streaming_rollout.py:44-167.
"""

from __future__ import annotations

import json
import logging
from argparse import Namespace
from typing import Any

from slime_b200.observability.trace_utils import build_sglang_meta_trace_attrs, trace_span
from slime_b200.rollout.sglang_rollout import GenerateState, _prepare_prompt_ids
from slime_b200.utils import http_utils
from slime_b200.utils.processing_utils import encode_image_for_rollout_engine
from slime_b200.utils.types import Sample

__all__ = ["generate_streaming"]
logger = logging.getLogger(__name__)

_REWOUND_FIELDS = ("tokens", "response", "response_length", "rollout_log_probs", "rollout_top_p_token_ids",
                   "rollout_top_p_token_offsets", "loss_mask")  # fmt: skip


def _snapshot(sample: Sample) -> dict:
    snap = {}
    for f in _REWOUND_FIELDS:
        v = getattr(sample, f)
        snap[f] = list(v) if isinstance(v, list) else v
    snap["response"] = sample.response or ""
    return snap


def _rewind(sample: Sample, snap: dict) -> None:
    for f, v in snap.items():
        setattr(sample, f, list(v) if isinstance(v, list) else v)


def _sse_payloads(line: str):
    if not line or not line.startswith("data:"):
        return None
    body = line[5:].strip()
    if not body or body == "[DONE]":
        return None
    try:
        return json.loads(body)
    except json.JSONDecodeError:
        logger.warning("streaming rollout: skipping a chunk that is not JSON: %r", body[:120])
        return None


async def generate_streaming(args: Namespace, sample: Sample, sampling_params: dict[str, Any]) -> Sample:
    state = GenerateState(args)
    url = f"http://{args.sglang_router_ip}:{args.sglang_router_port}/generate"
    assert sample.status in (Sample.Status.PENDING, Sample.Status.ABORTED), f"Sample status is {sample.status}"
    prompt_ids = _prepare_prompt_ids(sample, state.tokenizer, state.processor)
    sampling_params["max_new_tokens"] -= sample.response_length
    assert sampling_params["max_new_tokens"] >= 0, f"max_new_tokens {sampling_params['max_new_tokens']} < 0"
    if sampling_params["max_new_tokens"] == 0:
        sample.status = Sample.Status.TRUNCATED
        return sample

    payload: dict[str, Any] = {"sampling_params": sampling_params, "return_logprob": True, "stream": True}
    if args.use_rollout_routing_replay:
        payload["return_routed_experts"] = True
    images = sample.multimodal_inputs.get("images") if sample.multimodal_inputs else None
    if images:
        payload["image_data"] = [encode_image_for_rollout_engine(im) for im in images]
        payload["text"] = sample.prompt
    else:
        payload["input_ids"] = prompt_ids
    if not sample.tokens:
        sample.tokens = prompt_ids
    headers = None
    if sample.session_id and getattr(args, "router_policy", None) == "consistent_hashing":
        headers = {"X-SMG-Routing-Key": sample.session_id}

    entry = _snapshot(sample)
    meta: dict[str, Any] = {}
    tokens: list[int] = []
    log_probs: list[float] = []
    text = ""
    client = http_utils._get_client()
    with trace_span(sample, "sglang_generate_stream", attrs={"max_new_tokens": sampling_params["max_new_tokens"]}) as span:
        async with client.stream("POST", url, json=payload, headers=headers) as response:
            response.raise_for_status()
            async for line in response.aiter_lines():
                chunk = _sse_payloads(line)
                if chunk is None:
                    continue
                meta = chunk.get("meta_info") or {}
                text = chunk.get("text", text)
                pairs = meta.get("output_token_logprobs")
                if pairs is not None:
                    tokens, log_probs = [p[1] for p in pairs], [p[0] for p in pairs]
                _rewind(sample, entry)
                sample.append_response_tokens(args, tokens=tokens, log_probs=log_probs, trainable=True, meta_info=meta,
                                              text=text, update_terminal_info=bool(meta.get("finish_reason")))  # fmt: skip
                if state.aborted:
                    break
        if meta.get("finish_reason"):
            span.update(build_sglang_meta_trace_attrs(meta))
    if state.aborted and not meta.get("finish_reason"):
        sample.status = Sample.Status.ABORTED
    return sample
