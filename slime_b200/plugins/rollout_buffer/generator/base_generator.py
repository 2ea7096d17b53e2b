"""Single-turn math generator and the base class other task generators build on.

A generator reads prompts from a JSONL file (``{"prompt": [chat messages], "label": ..., "instance_id"?}``), produces
``num_repeat_per_sample`` trajectories per prompt by calling an OpenAI-compatible ``/v1/chat/completions`` endpoint
(the rollout router, an adapter or any engine that speaks it), scores each with a reward function and posts it to the
buffer service. Work is spread over a pool of threads (the work is waiting on HTTP; threads share the connection pool
and need no pickling of the rollout/reward callables). An aborted generation (weights are being updated) is resumed
from its partial text with ``continue_final_message``.

Module-level hooks the buffer service picks up: ``TASK_TYPE``, ``run_rollout``, ``is_valid_group``. ``normalize_group_data`` is
there for task generators that want GRPO normalisation done buffer-side (expose it as ``transform_group``); the math
task leaves rewards raw because the trainer normalises them itself. Parity: slime_plugins/rollout_buffer/generator/base_generator.py:15-351.
"""

from __future__ import annotations

import copy
import json
import logging
import queue
import random
import threading
import time
import uuid
from typing import Any, Callable

import requests

logger = logging.getLogger(__name__)

TASK_TYPE = "math"
DEFAULT_SAMPLING_PARAMS = {"top_p": 1}
ABORT_BACKOFF_SEC = 10.0
MAX_QUERY_ATTEMPTS = 6
_STOP = object()


class ChatClient:
    """The two calls a generator needs from an OpenAI-compatible server."""

    def __init__(self, base_url: str, api_key: str = "test", timeout: float = 3600.0):
        base_url = base_url.rstrip("/")
        self.base_url = base_url if base_url.endswith("/v1") else base_url + "/v1"
        self.headers = {"Authorization": f"Bearer {api_key}"}
        self.timeout = timeout
        self.session = requests.Session()

    def chat(self, **payload) -> dict:
        body = {k: v for k, v in payload.items() if v is not None and k != "extra_body"}
        body.update(payload.get("extra_body") or {})
        r = self.session.post(f"{self.base_url}/chat/completions", json=body, headers=self.headers, timeout=self.timeout)
        r.raise_for_status()
        return r.json()


def get_rule_based_math_reward(item: dict) -> float:
    from slime_b200.rollout.rm_hub.deepscaler import get_deepscaler_rule_based_reward

    last = item["messages"][-1]
    assert last["role"] == "assistant", f"last message must be the assistant's, got {last['role']}"
    return get_deepscaler_rule_based_reward(last["content"], item["label"]) if last.get("content") else 0


def query_single_turn(client: ChatClient, messages: list[dict], sampling_params: dict, tools=None):
    """One assistant turn -> ``(messages + [assistant], finish_reason)``; partial text survives aborts."""
    budget = sampling_params.get("max_tokens")
    text, used, finish = None, 0, "stop"
    for _ in range(MAX_QUERY_ATTEMPTS):
        req = {"messages": copy.deepcopy(messages), **sampling_params, "model": "custom", "stream": False,
               "seed": random.randint(1, 10_000_000), "tools": tools}  # fmt: skip
        if text is not None:
            req["messages"].append({"role": "assistant", "content": text})
            req["extra_body"] = {"continue_final_message": True}
            if budget is not None:
                req["max_tokens"] = max(0, budget - used)
        if req.get("max_tokens") == 0:
            break
        try:
            resp = client.chat(**req)
            choice = resp["choices"][0]
        except Exception as e:  # noqa: BLE001
            logger.warning("chat query failed: %r", e)
            continue
        finish = choice.get("finish_reason") or "stop"
        piece = choice["message"].get("content")
        if piece:
            text = piece if text is None else text + piece
        if finish != "abort":
            break
        used += (resp.get("usage") or {}).get("completion_tokens", 0)
        time.sleep(ABORT_BACKOFF_SEC)
    out = messages[:-1] if messages and messages[-1]["role"] == "assistant" else list(messages)
    return out + [{"role": "assistant", "content": text}], finish


class BaseGenerator:
    def __init__(self, remote_engine_url: str, remote_buffer_url: str, num_repeat_per_sample: int = 1,
                 queue_size: int = 1_000_000, num_process: int = 10, task_type: str = "math", max_tokens: int = 4096,
                 num_repeats: int = 10, skip_instance_ids: list | None = None, sampling_params: dict | None = None,
                 pause_between_repeats_sec: float = 300.0, client: ChatClient | None = None):  # fmt: skip
        self.remote_buffer_url = remote_buffer_url.rstrip("/")
        self.num_repeat_per_sample, self.num_workers, self.queue_size = num_repeat_per_sample, num_process, queue_size
        self.task_type, self.num_repeats, self.pause = task_type, num_repeats, pause_between_repeats_sec
        self.sampling_params = {**DEFAULT_SAMPLING_PARAMS, **(sampling_params or {}), "max_tokens": max_tokens}
        # groups the trainer already consumed (it sends their ids on restart): each is skipped once per trajectory
        self.skip = list(skip_instance_ids) * num_repeat_per_sample if skip_instance_ids else []
        self.client = client or ChatClient(remote_engine_url)
        self.sent = 0

    # ------------------------------------------------------------------ pieces subclasses may override
    def load_items(self, input_file: str) -> list[dict]:
        items = []
        with open(input_file) as f:
            for i, line in enumerate(f):
                if line.strip():
                    item = json.loads(line)
                    item.setdefault("instance_id", i)
                    items.append(item)
        return items

    def send_data_to_buffer(self, data: dict) -> bool:
        for _ in range(2):
            try:
                if requests.post(f"{self.remote_buffer_url}/buffer/write", json=data, timeout=60).status_code == 200:
                    self.sent += 1
                    return True
            except Exception as e:  # noqa: BLE001
                logger.warning("write to buffer failed: %r", e)
        return False

    def make_trajectory(self, item: dict, rollout_func: Callable, reward_func: Callable) -> dict:
        messages, finish = rollout_func(self.client, item["prompt"], self.sampling_params)
        item = {**item, "messages": messages}
        reward = reward_func(item)
        extra = {**item, **self.sampling_params, "rollout_index": 1, "reward": reward, "extra_info": {},
                 "timestamp": str(time.time()), "finish_reason": finish,
                 "round_number": sum(m["role"] == "assistant" for m in messages)}  # fmt: skip
        uid, instance_id = extra.pop("uid", None) or str(uuid.uuid4()), extra.pop("instance_id")
        return {"uid": uid, "messages": messages, "reward": reward, "instance_id": instance_id, "extra_info": extra}

    # -------------------------------------------------------------------------------------- the run
    def run(self, input_file: str, rollout_func: Callable, reward_func: Callable) -> str:
        tasks: queue.Queue = queue.Queue(self.queue_size)

        def feed():
            items = self.load_items(input_file)
            random.shuffle(items)
            for rep in range(self.num_repeats):
                for item in items:
                    for _ in range(self.num_repeat_per_sample):
                        if item["instance_id"] in self.skip:
                            self.skip.remove(item["instance_id"])
                            continue
                        tasks.put({**copy.deepcopy(item), "uid": str(uuid.uuid4())})
                if rep + 1 < self.num_repeats and self.pause > 0:
                    time.sleep(self.pause)
            for _ in range(self.num_workers):
                tasks.put(_STOP)

        def work():
            while (item := tasks.get()) is not _STOP:
                try:
                    self.send_data_to_buffer(self.make_trajectory(item, rollout_func, reward_func))
                except Exception:  # noqa: BLE001
                    logger.exception("trajectory for instance %s failed", item.get("instance_id"))

        threads = [threading.Thread(target=feed, daemon=True, name="generator-feed")]
        threads += [threading.Thread(target=work, daemon=True, name=f"generator-{i}") for i in range(self.num_workers)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        return "finished"

    def entry(self, input_file: str, rollout_func: Callable, reward_func: Callable, num_epoch: int = 1):
        for _ in range(num_epoch):
            self.run(input_file, rollout_func, reward_func)


def run_rollout(data: dict[str, Any]):
    """Entry the buffer service calls with the trainer's ``/start_rollout`` payload."""
    time.sleep(float(data.get("startup_delay_sec", 10)))  # the service answers /start_rollout before it is idle again
    sp = dict(data.get("sampling_params") or {})
    gen = BaseGenerator(data["remote_engine_url"], data["remote_buffer_url"],
                        num_repeat_per_sample=int(data["num_repeat_per_sample"]),
                        max_tokens=int(sp.get("max_tokens", data.get("max_tokens", 4096))),
                        num_process=int(data.get("num_process", 100)), task_type=data["task_type"],
                        skip_instance_ids=data.get("skip_instance_ids"), sampling_params=sp,
                        num_repeats=int(data.get("num_repeats", 10)),
                        pause_between_repeats_sec=float(data.get("pause_between_repeats_sec", 300)))  # fmt: skip
    gen.entry(data["input_file"], query_single_turn, get_rule_based_math_reward, int(data.get("num_epoch", 1)))


def normalize_group_data(group, epsilon: float = 1e-8, algo: str = "grpo"):
    """GRPO normalisation inside one group. Rewards outside [0, 1] are sentinels (format penalties and the like): they
    neither enter the statistics nor get rescaled. An all-zero group stays as it is; zero variance maps to 0."""
    assert algo == "grpo", "only grpo normalisation is implemented"
    key, items = group
    raw = [it["reward"] for it in items]
    inside = [r for r in raw if 0 <= r <= 1]
    if inside and set(inside) != {0}:
        mean = sum(inside) / len(inside)
        std = (sum((r - mean) ** 2 for r in inside) / len(inside)) ** 0.5
        norm = [(0.0 if std < epsilon else (r - mean) / (std + epsilon)) if 0 <= r <= 1 else r for r in raw]
    else:
        norm = raw
    for it, r, n in zip(items, raw, norm):
        it["reward"], it["raw_reward"] = n, r
    return key, items


def is_valid_group(group, min_valid_group_size: int, task_type: str = TASK_TYPE) -> bool:
    """Complete (enough trajectories) and every one of the required count has a non-empty final answer."""
    items = group[1] if isinstance(group, tuple) else group
    answered = sum(bool((it["messages"][-1].get("content") or "").strip()) for it in items)
    return len(items) >= min_valid_group_size and answered >= min_valid_group_size
