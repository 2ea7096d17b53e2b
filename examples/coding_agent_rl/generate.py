"""Coding-agent RL: one rollout = one agent session on one repository task.

    --custom-generate-function-path examples.coding_agent_rl.generate.generate

Stages: sandbox + workspace (``tasks.prepare_workspace``) -> the agent works on the task, its model calls going through
a chat-protocol adapter that forwards them to the rollout engine and records tokens and log-probs per turn -> ``git
diff`` -> the patch is graded in a fresh sandbox (``tasks.grade``) -> the adapter turns the session into ``Sample``
rows carrying the reward. Environment:

    CODING_AGENT        mini (default; ``mini_agent.MiniAgentHarness``) | claude_code | codex
    CODING_SANDBOX      local (default; a scratch directory on this host) | e2b
    CODING_TIME_BUDGET  seconds an agent may run (default 1800); CODING_EVAL_TIMEOUT for the test command (600)
    CODING_ADAPTER_HOST address the sandbox reaches the adapter at (default 127.0.0.1)

Same role as examples/coding_agent_rl/generate.py:182-283 in the reference.
"""

from __future__ import annotations

import asyncio
import logging
import os
import secrets
import time

from slime_b200.agent.adapters import AnthropicAdapter, OpenAIAdapter
from slime_b200.agent.aiohttp_threaded import serve_in_thread
from slime_b200.agent.sandbox import E2BSandbox, LocalSandbox
from slime_b200.utils.misc import SingletonMeta
from slime_b200.utils.types import Sample

from . import tasks
from .mini_agent import MiniAgentHarness

logger = logging.getLogger(__name__)


def _agent():
    name = os.environ.get("CODING_AGENT", "mini")
    if name == "mini":
        return MiniAgentHarness, OpenAIAdapter
    from slime_b200.agent.harness import ClaudeCodeHarness, CodexHarness

    table = {"claude_code": (ClaudeCodeHarness, AnthropicAdapter), "codex": (CodexHarness, OpenAIAdapter)}
    if name not in table:
        raise ValueError(f"CODING_AGENT={name!r} is not one of mini, claude_code, codex")
    return table[name]


def sandbox_factory(image: str | None = None):
    if os.environ.get("CODING_SANDBOX", "local") == "e2b":
        return lambda: E2BSandbox(image or os.environ["CODING_E2B_IMAGE"])
    return lambda: LocalSandbox()


class AdapterService(metaclass=SingletonMeta):
    """One adapter per process, served from its own thread; sessions are told apart by their id."""

    def __init__(self, args):
        from slime_b200.utils.processing_utils import load_tokenizer

        _, adapter_cls = _agent()
        tok = load_tokenizer(args.hf_checkpoint, trust_remote_code=True)
        engine = f"http://{args.sglang_router_ip}:{args.sglang_router_port}"
        self.adapter = adapter_cls(tokenizer=tok, engine_url=engine)
        bind = os.environ.get("CODING_ADAPTER_BIND", "127.0.0.1")
        self.handle = serve_in_thread(self.adapter.app, host=bind, port=int(os.environ.get("CODING_ADAPTER_PORT", "0")),
                                      thread_name="coding-adapter", runner_kwargs={"handler_cancellation": True})  # fmt: skip
        self.url = f"http://{os.environ.get('CODING_ADAPTER_HOST', '127.0.0.1')}:{self.handle.port}"


def _abort(sample: Sample, reason: str) -> list[Sample]:
    sample.status = Sample.Status.ABORTED
    sample.reward = 0.0
    sample.metadata = {**(sample.metadata or {}), "abort_reason": reason}
    return [sample]


async def generate(args, sample: Sample, sampling_params: dict, evaluation: bool = False) -> list[Sample]:
    try:
        task = tasks.get_task(sample)
    except ValueError as e:
        return _abort(sample, f"bad_task: {e}")
    service = AdapterService(args)
    adapter, harness = service.adapter, _agent()[0]()
    sid = f"{task.instance_id}-{secrets.token_hex(4)}"
    budget = int(os.environ.get("CODING_TIME_BUDGET", "1800"))
    adapter.open_session(sid, sampling_defaults=dict(sampling_params),
                         max_context_tokens=getattr(args, "rollout_max_context_len", None) or 0)  # fmt: skip
    t0 = time.time()
    make = sandbox_factory(task.image)
    try:
        async with make() as sb:
            await tasks.prepare_workspace(sb, task)
            await harness.install_cli(sb)
            exit_code = await harness.run(sb, workdir=tasks.WORKDIR, session_id=sid, adapter_url=service.url,
                                          time_budget_sec=budget, prompt=task.problem)  # fmt: skip
            diff = await tasks.git_diff(sb)
        reward, details = await tasks.grade(task, diff, make, timeout_sec=int(os.environ.get("CODING_EVAL_TIMEOUT", "600")))
    except (asyncio.CancelledError, KeyboardInterrupt):
        await adapter.drop_session(sid)
        raise
    except Exception as e:  # noqa: BLE001 - a broken sandbox must not take the rollout down
        logger.exception("coding task %s failed", task.instance_id)
        await adapter.drop_session(sid)
        return _abort(sample, f"error: {e!r}")
    extra = {"instance_id": task.instance_id, "agent_exit_code": exit_code, "patch_chars": len(diff), "seconds": time.time() - t0,
             **details}  # fmt: skip
    rows = await adapter.finish_session(sid, base_sample=sample, reward=reward, extra_metadata=extra)
    if not rows:  # the agent never reached the model
        return _abort(sample, "no_turns")
    return rows
