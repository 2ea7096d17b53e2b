"""Rollout function that trains from the stand-alone buffer service instead of generating in-process.

    --rollout-function-path slime_b200.plugins.rollout_buffer.rollout_buffer_example.generate_rollout
    --rollout-buffer-url http://buffer-host:8889 --rollout-task-type math

First call: ``POST /start_rollout`` tells the service which generator to run, where the engines are, the sampling
parameters, and which groups earlier steps already consumed (kept in the data source's metadata so a resumed run does
not train on them twice). Every call: poll ``/get_rollout_data`` until ``rollout_batch_size`` groups beyond what the
local data buffer already holds have arrived; keep the newest groups if more came; tokenise each trajectory's chat
messages into ids + loss mask (assistant tokens only) and hand the groups to the data buffer.
Parity: slime_plugins/rollout_buffer/rollout_buffer_example.py:23-307.
"""

from __future__ import annotations

import asyncio
import logging
import time
from typing import Any

import aiohttp
import requests

from slime_b200.utils.async_utils import run
from slime_b200.utils.mask_utils import MultiTurnLossMaskGenerator
from slime_b200.utils.types import Sample

logger = logging.getLogger(__name__)
__all__ = ["generate_rollout"]

POLL_SEC = 3.0
REQUIRED_KEYS = {"uid", "instance_id", "messages", "reward", "extra_info"}
_state = {"started": False, "tokenizer": None, "tokenizer_path": None}


def _timestamp(item: dict) -> float:
    ts = item.get("timestamp", (item.get("extra_info") or {}).get("timestamp"))
    return float(ts) if ts is not None else 0.0


def select_rollout_data(args, results: list[dict], need_groups: int) -> list[list[dict]]:
    """Group by ``instance_id`` and keep the ``need_groups`` groups whose latest trajectory is newest."""
    groups: dict[Any, list[dict]] = {}
    for item in results:
        groups.setdefault(item["instance_id"], []).append(item)
    ranked = sorted(groups.values(), key=lambda g: max(map(_timestamp, g)), reverse=True)
    return ranked[:need_groups]


def summarize_meta(all_meta: list[dict]) -> dict[str, float]:
    """Sample-weighted mean reward over every trajectory the generators wrote (before group filtering)."""
    total = sum(m.get("total_samples", 0) for m in all_meta)
    if not total:
        return {}
    return {"rollout/no_filter/total_samples": total,
            "rollout/no_filter/avg_reward": sum(m.get("avg_reward", 0) * m.get("total_samples", 0) for m in all_meta) / total}  # fmt: skip


def log_raw_info(args, all_meta: list[dict], rollout_id: int) -> dict:
    metrics = summarize_meta(all_meta)
    if not metrics:
        return metrics
    step = rollout_id
    if getattr(args, "wandb_always_use_train_step", False):
        step = rollout_id * args.rollout_batch_size * args.n_samples_per_prompt // args.global_batch_size
    try:
        from slime_b200.observability import logging_utils

        logging_utils.log(args, {**metrics, "rollout/step": step}, step_key="rollout/step")
    except Exception as e:  # noqa: BLE001
        logger.info("unfiltered rollout stats %d: %s (not logged to a tracker: %r)", rollout_id, metrics, e)
    return metrics


async def get_rollout_data(api_base_url: str, poll_sec: float = POLL_SEC) -> tuple[list[dict], dict]:
    """Block until the service returns at least one complete group -> ``(trajectories, meta_info)``."""
    waited_since = time.monotonic()
    async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=120)) as session:
        while True:
            async with session.post(f"{api_base_url}/get_rollout_data", json={}) as resp:
                resp.raise_for_status()
                body = await resp.json()
            if body["success"]:
                break
            await asyncio.sleep(poll_sec)
            if time.monotonic() - waited_since > 30:
                logger.info("rollout buffer has no complete group yet, still waiting")
                waited_since = time.monotonic()
    data, meta = body["data"], {}
    if isinstance(data, dict):
        data, meta = data["data"], data.get("meta_info") or {}
    elif data and "data" in data[0]:
        data = [d["data"] for d in data]
    for item in data:
        if not REQUIRED_KEYS.issubset(item):
            raise ValueError(f"trajectory lacks {sorted(REQUIRED_KEYS - set(item))}: {str(item)[:200]}")
    return data, meta


def start_rollout(api_base_url: str, args, metadata: dict, retry_sec: float = 2.0, max_tries: int | None = None) -> dict:
    consumed = [i for ids in (metadata or {}).values() for i in ids]
    payload = {"num_process": str(getattr(args, "rollout_num_process", 100)), "num_epoch": str(args.num_epoch or 3),
               "remote_engine_url": f"http://{args.sglang_router_ip}:{args.sglang_router_port}",
               "remote_buffer_url": args.rollout_buffer_url, "task_type": args.rollout_task_type,
               "input_file": args.prompt_data, "num_repeat_per_sample": str(args.n_samples_per_prompt),
               "max_tokens": str(args.rollout_max_response_len),
               "sampling_params": {"max_tokens": args.rollout_max_response_len, "temperature": args.rollout_temperature,
                                   "top_p": args.rollout_top_p},
               "tokenizer_path": args.hf_checkpoint, "skip_instance_ids": consumed}  # fmt: skip
    tries = 0
    while True:
        tries += 1
        try:
            r = requests.post(f"{api_base_url}/start_rollout", json=payload, timeout=10)
            r.raise_for_status()
            return r.json()
        except Exception as e:  # noqa: BLE001
            if max_tries is not None and tries >= max_tries:
                raise
            logger.warning("start_rollout failed (%r), retrying", e)
            time.sleep(retry_sec)


def _tokenizer(args):
    if _state["tokenizer"] is None or _state["tokenizer_path"] != args.hf_checkpoint:
        from slime_b200.utils.processing_utils import load_tokenizer

        _state["tokenizer"], _state["tokenizer_path"] = load_tokenizer(args.hf_checkpoint, trust_remote_code=True), args.hf_checkpoint
    return _state["tokenizer"]


def records_to_samples(args, groups: list[list[dict]], tokenizer) -> list[list[Sample]]:
    masker = MultiTurnLossMaskGenerator(tokenizer, tokenizer_type=args.loss_mask_type)
    out = []
    for group in groups:
        rows = []
        for rec in group:
            ids, mask = masker.get_loss_mask(rec["messages"])
            n = masker.get_response_lengths([mask])[0]
            truncated = (rec["extra_info"] or {}).get("finish_reason") == "length"
            rows.append(Sample(index=rec["instance_id"], prompt=rec["uid"], tokens=ids, response_length=n,
                               reward=rec["reward"], loss_mask=mask[-n:] if n else [],
                               status=Sample.Status.TRUNCATED if truncated else Sample.Status.COMPLETED,
                               metadata=dict(rec["extra_info"] or {})))  # fmt: skip
        out.append(rows)
    return out


async def generate_rollout_async(args, rollout_id: int, data_buffer, evaluation: bool = False):
    if evaluation:
        raise NotImplementedError("evaluation through the rollout buffer is not supported")
    if not _state["started"]:
        start_rollout(args.rollout_buffer_url, args, data_buffer.get_metadata())
        _state["started"] = True
    need = args.rollout_batch_size * args.n_samples_per_prompt - data_buffer.get_buffer_length()
    if need <= 0:
        return data_buffer.get_samples(args.rollout_batch_size)
    assert need % args.n_samples_per_prompt == 0, "the data buffer holds a partial group"
    results, all_meta, failures = [], [], 0
    limit = args.fetch_trajectory_retry_times
    while len(results) < need and (limit == -1 or failures < limit):
        try:
            data, meta = await get_rollout_data(args.rollout_buffer_url)
            results.extend(data)
            if meta:
                all_meta.append(meta)
        except Exception as e:  # noqa: BLE001
            failures += 1
            logger.warning("fetching trajectories failed (%d): %r", failures, e)
            await asyncio.sleep(POLL_SEC)
    log_raw_info(args, all_meta, rollout_id)
    groups = select_rollout_data(args, results, need // args.n_samples_per_prompt)
    finished = [g for m in all_meta for g in m.get("finished_groups", [])]
    if all_meta and "finished_groups" in all_meta[0]:
        data_buffer.update_metadata({str(rollout_id): finished})
    data_buffer.add_samples(records_to_samples(args, groups, _tokenizer(args)))
    return data_buffer.get_samples(args.rollout_batch_size)


def generate_rollout(args, rollout_id, data_buffer, evaluation=False):
    return run(generate_rollout_async(args, rollout_id, data_buffer, evaluation))
