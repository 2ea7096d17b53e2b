"""Default rollout function: asynchronous over-sampling against the rollout engines' HTTP API.

Contract (``--rollout-function-path``): ``generate_rollout(args, rollout_id, data_source, evaluation=False)``
returning ``RolloutFnTrainOutput`` / ``RolloutFnEvalOutput``. The loop keeps at least
``rollout_batch_size`` prompt groups in flight, consumes groups as they complete, applies the dynamic
sampling filter, stops at ``rollout_batch_size`` kept groups, aborts what is still running (optionally
returning partial groups to the data buffer) and sorts the result by sample index.
Parity: slime/rollout/sglang_rollout.py:83-649 (module name kept: it is the default dotted path).
"""

from __future__ import annotations

import asyncio
import copy
import inspect
import json
import logging
import uuid
from argparse import Namespace
from contextlib import contextmanager
from typing import Any

import numpy as np

from slime_b200.engine.server_control import abort_servers_until_idle
from slime_b200.observability.trace_utils import build_sglang_meta_trace_attrs, trace_function, trace_span
from slime_b200.rollout.base_types import RolloutFnEvalOutput, RolloutFnTrainOutput
from slime_b200.rollout.filter_hub.base_types import MetricGatherer, call_dynamic_filter
from slime_b200.rollout.rm_hub import async_rm, batched_async_rm
from slime_b200.rollout.sample_hooks import apply_rollout_sample_hooks
from slime_b200.utils.async_utils import run
from slime_b200.utils.data import Dataset
from slime_b200.utils.eval_config import EvalDatasetConfig
from slime_b200.utils.http_utils import get, post
from slime_b200.utils.misc import SingletonMeta, load_function
from slime_b200.utils.processing_utils import encode_image_for_rollout_engine, load_processor, load_tokenizer
from slime_b200.utils.types import Sample

logger = logging.getLogger(__name__)
__all__ = ["generate_rollout", "generate", "generate_and_rm", "generate_and_rm_group", "GenerateState", "get_model_url"]


def get_rollout_num_engines(args) -> int:
    n = getattr(args, "rollout_num_engines", None)
    if n:
        return n
    return max(1, (args.rollout_num_gpus or 1) // max(args.rollout_num_gpus_per_engine, 1))


def get_model_url(args, model_name: str, endpoint: str = "/generate") -> str:
    """URL of a named model's router in a multi-model deployment (``--sglang-config``)."""
    routers = getattr(args, "sglang_model_routers", None) or {}
    if model_name in routers:
        ip, port = routers[model_name]
    else:
        ip, port = args.sglang_router_ip, args.sglang_router_port
    return f"http://{ip}:{port}{endpoint}"


def should_drop_dynamic_filter_output(output, *, remaining_batch_size: int, target_data_size: int) -> bool:
    """Drop a filtered-out group unless it is flagged as a fallback and too few groups remain in flight."""
    if output.keep:
        return False
    return not (output.keep_when_insufficient and remaining_batch_size <= target_data_size)


class GenerateState(metaclass=SingletonMeta):
    """Per-process generation state: tokenizer, concurrency gate, in-flight tasks, abort flag."""

    def __init__(self, args: Namespace) -> None:
        self.args = args
        self.tokenizer = load_tokenizer(args.hf_checkpoint, trust_remote_code=True)
        self.processor = load_processor(args.hf_checkpoint, trust_remote_code=True)
        self.semaphore = asyncio.Semaphore(args.sglang_server_concurrency * get_rollout_num_engines(args))
        self.sampling_params: dict[str, Any] = dict(
            temperature=args.rollout_temperature, top_p=args.rollout_top_p, top_k=args.rollout_top_k,
            max_new_tokens=args.rollout_max_response_len, stop=args.rollout_stop, stop_token_ids=args.rollout_stop_token_ids,
            skip_special_tokens=args.rollout_skip_special_tokens, no_stop_trim=True, spaces_between_special_tokens=False,
        )  # fmt: skip
        if getattr(args, "rollout_ignore_eos", False):
            self.sampling_params["ignore_eos"] = True
        if args.rollout_top_p != 1.0:
            self.sampling_params["custom_params"] = {"return_top_p_token_ids": True}
        if getattr(args, "sglang_enable_deterministic_inference", False):
            self.group_sampling_seeds = [args.rollout_seed + i for i in range(args.n_samples_per_prompt)]
        self.dp_counts = [0] * (getattr(args, "sglang_dp_size", None) or 1)
        self.dp_rank = 0
        self.reset()

    @contextmanager
    def dp_rank_context(self):
        low = min(self.dp_counts)
        rank = int(np.random.choice([i for i, c in enumerate(self.dp_counts) if c == low]))
        self.dp_counts[rank] += 1
        self.dp_rank = rank
        try:
            yield rank
        finally:
            self.dp_counts[rank] -= 1

    def reset(self) -> None:
        self.remaining_batch_size = 0
        self.pendings: set = set()
        self.aborted = False

    def submit_generate_tasks(self, groups: list[list[Sample]]) -> None:
        for group in groups:
            self.pendings.add(asyncio.ensure_future(
                generate_and_rm_group(self.args, group, sampling_params=self.sampling_params.copy(), evaluation=False)
            ))  # fmt: skip
        self.remaining_batch_size += len(groups)


def _prepare_prompt_ids(sample: Sample, tokenizer, processor) -> list[int]:
    if sample.tokens:
        return list(sample.tokens)
    if processor is not None and sample.multimodal_inputs:
        out = processor(text=sample.prompt, **sample.multimodal_inputs)
        ids = out["input_ids"][0]
        sample.multimodal_train_inputs = {k: v for k, v in out.items() if k not in ("input_ids", "attention_mask")} or None
        return list(ids)
    if isinstance(sample.prompt, str):
        return tokenizer.encode(sample.prompt, add_special_tokens=False)
    return tokenizer.apply_chat_template(sample.prompt, tokenize=True, add_generation_prompt=True)


async def generate(args: Namespace, sample: Sample, sampling_params: dict[str, Any]) -> Sample:
    """One ``/generate`` round trip through the router; token ids and log-probs come from
    ``meta_info.output_token_logprobs`` (never from re-tokenising the text)."""
    state = GenerateState(args)
    url = f"http://{args.sglang_router_ip}:{args.sglang_router_port}/generate"
    assert sample.status in (Sample.Status.PENDING, Sample.Status.ABORTED), f"Sample status is {sample.status}"
    prompt_ids = _prepare_prompt_ids(sample, state.tokenizer, state.processor)
    sampling_params["max_new_tokens"] -= sample.response_length
    assert sampling_params["max_new_tokens"] >= 0, f"max_new_tokens {sampling_params['max_new_tokens']} < 0"
    if sampling_params["max_new_tokens"] == 0:
        sample.status = Sample.Status.TRUNCATED
        return sample
    payload: dict[str, Any] = {"sampling_params": sampling_params, "return_logprob": True}
    if args.use_rollout_routing_replay:
        payload["return_routed_experts"] = True
    images = sample.multimodal_inputs.get("images") if sample.multimodal_inputs else None
    if images:
        payload["image_data"] = [encode_image_for_rollout_engine(im) for im in images]
    if images and state.processor is None:
        payload["text"] = sample.prompt  # no processor on this side: the engine tokenises and sizes the placeholder runs
    else:
        payload["input_ids"] = prompt_ids  # (with images: already expanded by the processor, one run per image)
    if not sample.tokens:
        sample.tokens = prompt_ids
    headers = None
    if sample.session_id and getattr(args, "router_policy", None) == "consistent_hashing":
        headers = {"X-SMG-Routing-Key": sample.session_id}
    with trace_span(sample, "sglang_generate", attrs={"max_new_tokens": sampling_params["max_new_tokens"]}) as span:
        output = await post(url, payload, headers=headers)
        span.update(build_sglang_meta_trace_attrs(output["meta_info"]))
    pairs = output["meta_info"].get("output_token_logprobs") or []
    sample.append_response_tokens(args, tokens=[p[1] for p in pairs], log_probs=[p[0] for p in pairs], trainable=True,
                                  meta_info=output["meta_info"], text=output.get("text", ""))  # fmt: skip
    return sample


@trace_function("generate_and_rm", target="sample")
async def generate_and_rm(args: Namespace, sample, sampling_params: dict[str, Any], evaluation: bool = False):
    if args.partial_rollout and args.mask_offpolicy_in_partial_rollout and sample.response_length > 0:
        sample.loss_mask = [0] * sample.response_length  # tokens from an older policy do not train
    if sample.status in (Sample.Status.COMPLETED, Sample.Status.TRUNCATED):
        assert sample.response is not None
        if not args.group_rm:
            assert sample.reward is not None
        return sample
    state = GenerateState(args)
    async with state.semaphore:
        if state.aborted:
            sample.status = Sample.Status.ABORTED
            return sample
        with state.dp_rank_context():
            path = getattr(sample, "generate_function_path", None) or args.custom_generate_function_path
            if path is not None:
                fn = load_function(path)
                if "evaluation" in inspect.signature(fn).parameters:
                    sample = await fn(args, sample, sampling_params, evaluation=evaluation)
                else:
                    sample = await fn(args, sample, sampling_params)
            else:
                sample = await generate(args, sample, sampling_params)
    sample = await apply_rollout_sample_hooks(args, sample, evaluation=evaluation)
    if args.group_rm:
        return sample
    if isinstance(sample, list):  # a custom generate fanned one rollout out into several training samples
        if any(s.status == Sample.Status.ABORTED for s in sample):
            return sample
        need = [s for s in sample if s.reward is None]
        with trace_span(need, "reward_model"):
            rewards = await batched_async_rm(args, need)
        for s, r in zip(need, rewards):
            s.reward = r
        return sample
    if sample.status == Sample.Status.ABORTED:
        return sample
    if sample.reward is None:
        with trace_span(sample, "reward_model"):
            sample.reward = await async_rm(args, sample)
    return sample


@trace_function("generate_and_rm_group", target="group",
                attrs_getter=lambda args, group, sampling_params, evaluation=False: {"group_size": len(group)})  # fmt: skip
async def generate_and_rm_group(args: Namespace, group: list[Sample], sampling_params: dict[str, Any], evaluation: bool = False):
    state = GenerateState(args)
    if state.aborted:
        return group
    for s in group:
        if s.session_id is None:
            s.session_id = str(uuid.uuid4())
    tasks = []
    for i, s in enumerate(group):
        sp = sampling_params.copy()
        if getattr(args, "sglang_enable_deterministic_inference", False):
            sp["sampling_seed"] = state.group_sampling_seeds[i]
        tasks.append(asyncio.ensure_future(generate_and_rm(args, s, sp, evaluation=evaluation)))
    group = await asyncio.gather(*tasks)
    if not state.aborted and args.group_rm:
        with trace_span(group, "group_reward_model"):
            rewards = await batched_async_rm(args, group)
        for s, r in zip(group, rewards):
            s.reward = r
    return group


async def abort(args: Namespace, rollout_id: int) -> list[list[Sample]]:
    """Stop everything still in flight; with ``--partial-rollout`` the partial groups are handed back."""
    state = GenerateState(args)
    assert not state.aborted
    state.aborted = True
    workers = await get(f"http://{args.sglang_router_ip}:{args.sglang_router_port}/workers")
    await abort_servers_until_idle([w["url"] for w in workers["workers"]])
    partial, count = [], 0
    while state.pendings:
        done, state.pendings = await asyncio.wait(state.pendings, return_when=asyncio.FIRST_COMPLETED)
        if not args.partial_rollout:
            continue
        for task in done:
            group = task.result()
            for s in group:
                if s.response and "start_rollout_id" not in s.metadata:
                    s.metadata["start_rollout_id"] = rollout_id
            partial.append(group)
            count += len(group)
    if args.partial_rollout:
        logger.info("Collected %d partial samples into the data buffer", count)
    return partial


def _first_sample(group):
    return group[0][0] if isinstance(group[0], list) else group[0]


async def generate_rollout_async(args: Namespace, rollout_id: int, data_source) -> tuple[RolloutFnTrainOutput, list[list[Sample]]]:
    assert args.rollout_global_dataset
    state = GenerateState(args)
    dyn = load_function(args.dynamic_sampling_filter_path) if args.dynamic_sampling_filter_path is not None else None
    gatherer = MetricGatherer()
    target = args.rollout_batch_size
    data, all_data = [], []
    while len(data) < target:
        while state.remaining_batch_size < target:
            state.submit_generate_tasks(data_source(args.over_sampling_batch_size))
        done, state.pendings = await asyncio.wait(state.pendings, return_when=asyncio.FIRST_COMPLETED)
        for task in done:
            group = task.result()
            assert len(group) == args.n_samples_per_prompt
            all_data.append(group)
            verdict = call_dynamic_filter(dyn, args, group)
            if should_drop_dynamic_filter_output(verdict, remaining_batch_size=state.remaining_batch_size, target_data_size=target):
                gatherer.on_dynamic_filter_drop(reason=verdict.reason)
                state.remaining_batch_size -= 1
                continue
            if len(data) < target:
                data.append(group)
    s = _first_sample(data[-1])
    logger.info("Finish rollout %s: label=%s reward=%s", rollout_id, str(s.label)[:100], s.reward)
    partial = await abort(args, rollout_id)
    assert len(data) == args.rollout_batch_size, f"Got {len(data)} samples, expected {args.rollout_batch_size}"
    key = lambda g: _first_sample(g).index  # noqa: E731
    data.sort(key=key)
    all_data.sort(key=key)
    state.reset()
    if args.rollout_sample_filter_path is not None:
        load_function(args.rollout_sample_filter_path)(args, data)
    if args.rollout_all_samples_process_path is not None:
        load_function(args.rollout_all_samples_process_path)(args, all_data, data_source)
    return RolloutFnTrainOutput(samples=data, metrics=gatherer.collect()), partial


EVAL_PROMPT_DATASET: dict = {}


async def eval_rollout(args: Namespace, rollout_id: int):
    assert not args.group_rm, "Group RM is not supported for eval rollout"
    results = {}
    for r in await asyncio.gather(*[eval_rollout_single_dataset(args, rollout_id, cfg) for cfg in getattr(args, "eval_datasets", []) or []]):
        results.update(r)
    return RolloutFnEvalOutput(data=results), []


async def eval_rollout_single_dataset(args: Namespace, rollout_id: int, cfg: EvalDatasetConfig) -> dict:
    pick = lambda a, b: a if a is not None else b  # noqa: E731
    mm = pick(cfg.multimodal_keys, args.multimodal_keys)
    chat = pick(cfg.apply_chat_template, args.apply_chat_template)
    chat_kw = pick(cfg.apply_chat_template_kwargs, args.apply_chat_template_kwargs)
    cache_key = cfg.cache_key + (args.hf_checkpoint, chat, json.dumps(mm, sort_keys=True) if mm is not None else None,
                                 json.dumps(chat_kw, sort_keys=True) if chat_kw is not None else None)  # fmt: skip
    if cache_key not in EVAL_PROMPT_DATASET:
        EVAL_PROMPT_DATASET[cache_key] = Dataset(
            path=cfg.path, tokenizer=load_tokenizer(args.hf_checkpoint, trust_remote_code=True),
            processor=load_processor(args.hf_checkpoint, trust_remote_code=True), max_length=args.eval_max_prompt_len,
            prompt_key=cfg.input_key, label_key=cfg.label_key, multimodal_keys=mm, metadata_key=cfg.metadata_key,
            tool_key=cfg.tool_key, apply_chat_template=chat, apply_chat_template_kwargs=chat_kw,
        )  # fmt: skip
    dataset = EVAL_PROMPT_DATASET[cache_key]
    base = dict(
        temperature=cfg.temperature, top_p=cfg.top_p, top_k=cfg.top_k, max_new_tokens=cfg.max_response_len,
        stop=pick(cfg.stop, args.rollout_stop), stop_token_ids=pick(cfg.stop_token_ids, args.rollout_stop_token_ids),
        skip_special_tokens=pick(cfg.skip_special_tokens, args.rollout_skip_special_tokens),
        no_stop_trim=pick(cfg.no_stop_trim, True), spaces_between_special_tokens=False,
    )  # fmt: skip
    if cfg.repetition_penalty is not None:
        base["repetition_penalty"] = cfg.repetition_penalty
    min_new = pick(cfg.min_new_tokens, getattr(args, "eval_min_new_tokens", None))
    if min_new is not None:
        base["min_new_tokens"] = min_new
    tasks, idx = [], 0
    for prompt_sample in dataset.samples:
        for j in range(cfg.n_samples_per_eval_prompt):
            s = copy.deepcopy(prompt_sample)
            s.index = idx
            idx += 1
            s.metadata = cfg.inject_metadata(getattr(s, "metadata", None))
            s.custom_rm_path = cfg.custom_rm_path
            s.generate_function_path = getattr(cfg, "custom_generate_function_path", None)
            sp = dict(base)
            if getattr(args, "sglang_enable_deterministic_inference", False):
                sp["sampling_seed"] = args.rollout_seed + j
            tasks.append(asyncio.ensure_future(generate_and_rm(args, s, sampling_params=sp, evaluation=True)))
    data = []
    for coro in asyncio.as_completed(tasks):
        s = await coro
        data.extend(s) if isinstance(s, list) else data.append(s)
    data.sort(key=lambda s: s.index)
    key = args.eval_reward_key or args.reward_key
    return {cfg.name: {"rewards": [s.reward if not key else s.reward[key] for s in data],
                       "truncated": [s.status == Sample.Status.TRUNCATED for s in data], "samples": data}}  # fmt: skip


def generate_rollout(args: Namespace, rollout_id: int, data_source: Any, evaluation: bool = False):
    assert args.rollout_global_dataset
    if evaluation:
        output, _ = run(eval_rollout(args, rollout_id))
        return output
    output, partial = run(generate_rollout_async(args, rollout_id, data_source.get_samples))
    if partial:
        data_source.add_samples(partial)
    return output
