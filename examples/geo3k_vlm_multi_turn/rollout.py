"""Multi-turn rollout with images against a pluggable interaction environment.

    --custom-generate-function-path examples.geo3k_vlm_multi_turn.rollout.generate
    --custom-config-path examples/geo3k_vlm_multi_turn/config.yaml     # max_turns, rollout_interaction_env_path

Every assistant turn is one ``/generate`` call on the token ids accumulated so far, with all images seen so far in
``image_data`` (the engine gets processor-expanded ids, so every image placeholder run already has its full length). The
model's tokens and log-probs are appended with loss mask 1. The environment's reply is rendered through the chat template
after two throw-away messages whose rendering is then cut off, so that only the reply's own tokens (role markers, image
placeholders, generation prompt) are appended, with loss mask 0 and log-prob 0. The processor outputs of every turn
(``pixel_values``, ``image_grid_thw``) are concatenated in order into ``sample.multimodal_train_inputs`` for the trainer.
The token budget is ``rollout_max_context_len - len(tokens)`` (or what is left of ``max_new_tokens``).
(Same role as examples/geo3k_vlm_multi_turn/rollout.py:192-387 in the reference.)
"""

from __future__ import annotations

import importlib
import importlib.util
import os
import sys

import torch

from slime_b200.rollout.sglang_rollout import GenerateState
from slime_b200.utils.http_utils import post
from slime_b200.utils.processing_utils import encode_image_for_rollout_engine, process_vision_info
from slime_b200.utils.types import Sample

DEFAULT_ENV = "examples.geo3k_vlm_multi_turn.env_geo3k"
_FILLER = [{"role": "system", "content": "You are a helpful assistant."}, {"role": "user", "content": "I am a user."}]


def load_env_module(path: str | None):
    target = path or DEFAULT_ENV
    if target.endswith(".py") and os.path.exists(target):
        name = "rollout_env_" + os.path.splitext(os.path.basename(target))[0]
        spec = importlib.util.spec_from_file_location(name, target)
        module = importlib.util.module_from_spec(spec)
        sys.modules[name] = module
        spec.loader.exec_module(module)
        return module
    return importlib.import_module(target)


def _processor_call(processor, text, images):
    out = processor(text=text, images=images or None, return_tensors="pt")
    ids = out["input_ids"][0]
    extra = {k: v for k, v in out.items() if k not in ("input_ids", "attention_mask")} or None
    return [int(t) for t in (ids.tolist() if hasattr(ids, "tolist") else ids)], extra


def encode_observation(tokenizer, processor, message: dict, metadata: dict | None, use_template: bool, template_kw: dict | None):
    """Token ids of one environment message as they appear in the middle of a conversation, the images it carries (for
    the engine) and the processor outputs (for the trainer)."""
    tools = (metadata or {}).get("tools")
    kw = template_kw or {}
    cut = 0
    if use_template:
        before = tokenizer.apply_chat_template(_FILLER, tools=tools, tokenize=False, add_generation_prompt=False, **kw)
        text = tokenizer.apply_chat_template(_FILLER + [message], tools=tools, tokenize=False, add_generation_prompt=True, **kw)
        cut = len(tokenizer.encode(before, add_special_tokens=False))
    else:
        text = " ".join(p.get("text", "") for p in message["content"] if p.get("type") == "text")
    images = process_vision_info([message], processor).get("images", []) if processor is not None else []
    if processor is not None:
        ids, train_inputs = _processor_call(processor, text, images)
    else:
        ids, train_inputs = tokenizer.encode(text, add_special_tokens=False), None
    ids = ids[cut:]
    if ids and getattr(tokenizer, "bos_token_id", None) is not None and ids[0] == tokenizer.bos_token_id:
        ids = ids[1:]
    return ids, [encode_image_for_rollout_engine(im) for im in images], images, train_inputs


def merge_train_inputs(chunks: list[dict | None]) -> dict | None:
    keys = {k for c in chunks if c for k, v in c.items() if torch.is_tensor(v)}
    return {k: torch.cat([c[k] for c in chunks if c and torch.is_tensor(c.get(k))]) for k in sorted(keys)} or None


async def generate(args, sample: Sample, sampling_params: dict) -> Sample:
    assert not getattr(args, "partial_rollout", False), "partial rollout is not supported for interaction rollouts"
    max_turns = getattr(args, "max_turns", None)
    if max_turns is None:
        raise ValueError("max_turns must be set in the file named by --custom-config-path")
    state = GenerateState(args)
    tok, processor = state.tokenizer, state.processor
    url = f"http://{args.sglang_router_ip}:{args.sglang_router_port}/generate"
    sample.metadata = sample.metadata or {}
    env = load_env_module(getattr(args, "rollout_interaction_env_path", None)).build_env(sample=sample, args=args)
    sampling_params = dict(sampling_params)
    # first turn: the dataset prompt with its images
    images = list((sample.multimodal_inputs or {}).get("images") or [])
    train_chunks: list[dict | None] = []
    if processor is not None:
        prompt_ids, extra = _processor_call(processor, sample.prompt, images)
        train_chunks.append(extra)
    else:
        prompt_ids = tok.encode(sample.prompt, add_special_tokens=False)
    image_data = [encode_image_for_rollout_engine(im) for im in images]
    if not sample.tokens:
        sample.tokens = list(prompt_ids)
    sample.loss_mask, sample.rollout_log_probs = sample.loss_mask or [], sample.rollout_log_probs or []
    sample.response_length = len(sample.tokens) - len(prompt_ids)
    if getattr(args, "rollout_max_context_len", None) is not None:
        budget = args.rollout_max_context_len - len(sample.tokens)
    else:
        budget = sampling_params.get("max_new_tokens")
    try:
        env.reset()
        if budget is not None and budget <= 0:
            sample.status = Sample.Status.TRUNCATED
            return sample
        for turn in range(max_turns):
            if budget is not None:
                sampling_params["max_new_tokens"] = budget
            payload = {"input_ids": sample.tokens, "sampling_params": sampling_params, "return_logprob": True}
            if image_data:
                payload["image_data"] = image_data
            out = await post(url, payload)
            pairs = out["meta_info"].get("output_token_logprobs") or []
            sample.append_response_tokens(args, tokens=[p[1] for p in pairs], log_probs=[p[0] for p in pairs], trainable=True,
                                          meta_info=out["meta_info"])  # fmt: skip
            budget = None if budget is None else budget - len(pairs)
            finish = out["meta_info"]["finish_reason"]["type"]
            if finish in ("length", "abort"):
                sample.status = Sample.Status.TRUNCATED if finish == "length" else Sample.Status.ABORTED
                break
            if budget is not None and budget <= 0:
                sample.status = Sample.Status.TRUNCATED
                break
            observation, done, _ = env.step(out.get("text") or tok.decode([p[1] for p in pairs]))
            if done:
                sample.status = Sample.Status.COMPLETED
                break
            obs_ids, obs_image_data, obs_images, obs_train = encode_observation(
                tok, processor, env.format_observation(observation), sample.metadata, getattr(args, "apply_chat_template", False),
                getattr(args, "apply_chat_template_kwargs", None))  # fmt: skip
            sample.append_response_tokens(args, tokens=obs_ids, trainable=False)
            budget = None if budget is None else budget - len(obs_ids)
            if obs_images:
                image_data = image_data + obs_image_data
                sample.multimodal_inputs = {**(sample.multimodal_inputs or {}), "images": images + obs_images}
                images = images + obs_images
            if obs_train:
                train_chunks.append(obs_train)
            if budget is not None and budget <= 0:
                sample.status = Sample.Status.TRUNCATED
                break
            if turn + 1 >= max_turns:
                sample.status = Sample.Status.COMPLETED
        n_prompt = len(sample.tokens) - sample.response_length
        sample.multimodal_train_inputs = merge_train_inputs(train_chunks)
        sample.response = tok.decode(sample.tokens[n_prompt:], skip_special_tokens=False)
        if sample.status in (None, Sample.Status.PENDING):
            sample.status = Sample.Status.COMPLETED
        return sample
    finally:
        try:
            env.close()
        except Exception:  # noqa: BLE001
            pass
