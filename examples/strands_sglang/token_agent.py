"""A small tool-calling agent whose model client keeps the exact token trajectory of the conversation.

Agent frameworks work on messages; RL training needs the token ids the policy actually produced, with the log-probs
the engine reported for them. ``TokenTrackingModel`` is the piece in between: every completion is requested from the
rollout engine by token ids (the conversation so far, as tracked), the answer's ids and log-probs are appended with loss
mask 1, and whatever the chat template places between two assistant turns (tool results, role markers, the generation
prompt) is appended as the token delta of two renderings with loss mask 0. Nothing the model wrote is ever tokenised
again. ``ToolAgent`` is the loop on top: complete -> parse tool calls -> run tools -> complete, with a hook
(``ToolLimiter``) that ends the episode after a number of tool rounds. ``tool`` turns a typed Python function into a
tool with a JSON schema, the way agent SDKs declare tools.
Same role as the ``strands`` / ``strands_sglang`` packages used by examples/strands_sglang/generate_with_strands.py in
the reference (``SGLangModel``, ``ToolLimiter``, ``Agent``).
"""

from __future__ import annotations

import asyncio
import inspect
import json
from dataclasses import dataclass, field

from slime_b200.agent.parsing import parse_model_output
from slime_b200.utils.http_utils import post

_JSON_TYPES = {str: "string", int: "integer", float: "number", bool: "boolean", list: "array", dict: "object"}


class ToolLimitReached(Exception):
    """Raised by ``ToolLimiter`` to end an episode; the tokens so far stay valid."""


class ContextBudgetExceeded(Exception):
    pass


def tool(fn):
    """Declare ``fn`` as a tool: name, description (docstring) and a JSON schema from the annotated signature."""
    props, required = {}, []
    for name, p in inspect.signature(fn).parameters.items():
        props[name] = {"type": _JSON_TYPES.get(p.annotation, "string")}
        if p.default is inspect.Parameter.empty:
            required.append(name)
    fn.tool_spec = {"type": "function", "function": {"name": fn.__name__, "description": (fn.__doc__ or "").strip(),
                                                     "parameters": {"type": "object", "properties": props, "required": required}}}  # fmt: skip
    return fn


@dataclass
class Trajectory:
    token_ids: list[int] = field(default_factory=list)
    loss_mask: list[int] = field(default_factory=list)
    logprobs: list[float] = field(default_factory=list)
    initial_prompt_length: int = 0  # system + first user message: the prompt segment

    def extend(self, ids, mask: int, logprobs=None):
        self.token_ids += list(ids)
        self.loss_mask += [mask] * len(ids)
        self.logprobs += list(logprobs) if logprobs is not None else [0.0] * len(ids)


class TokenTrackingModel:
    def __init__(self, tokenizer, url: str, sampling_params: dict, max_context_len: int | None = None):
        self.tokenizer, self.url, self.max_context_len = tokenizer, url, max_context_len
        self.sampling_params = dict(sampling_params)
        self.rollout = Trajectory()
        self.last_meta: dict = {}

    def reset(self):
        self.rollout = Trajectory()
        self.last_meta = {}

    def _render(self, messages, tools) -> list[int]:
        out = self.tokenizer.apply_chat_template(messages, tokenize=True, add_generation_prompt=True, tools=tools or None)
        return list(out["input_ids"] if isinstance(out, dict) else out)

    def _sync_context(self, messages, tools):
        """Bring the tracked ids up to the rendering of ``messages``: the first call takes the whole rendering as the
        prompt, later calls append what follows the tracked ids (their tail is searched for in the rendering, since a
        template may re-serialise an assistant turn slightly differently from what the model wrote)."""
        rendered = self._render(messages, tools)
        tr = self.rollout
        if not tr.token_ids:
            tr.extend(rendered, 0)
            tr.initial_prompt_length = len(rendered)
            return
        have = tr.token_ids
        if rendered[: len(have)] == have:
            delta = rendered[len(have) :]
        else:
            tail, delta = have[-8:], None
            for start in range(len(rendered) - len(tail), -1, -1):
                if rendered[start : start + len(tail)] == tail:
                    delta = rendered[start + len(tail) :]
                    break
            if delta is None:  # no anchor: keep what follows the common prefix
                n = 0
                while n < min(len(have), len(rendered)) and have[n] == rendered[n]:
                    n += 1
                delta = rendered[max(n, len(have)) :] if len(rendered) > len(have) else []
        tr.extend(delta, 0)

    async def complete(self, messages: list[dict], tools: list[dict]) -> tuple[str, dict]:
        """One assistant turn. Returns (text, finish_reason)."""
        self._sync_context(messages, tools)
        tr = self.rollout
        params = dict(self.sampling_params)
        spent = len(tr.token_ids) - tr.initial_prompt_length
        budget = params.get("max_new_tokens", 1 << 30) - spent
        if self.max_context_len is not None:
            budget = min(budget, self.max_context_len - len(tr.token_ids))
        if budget <= 0:
            raise ContextBudgetExceeded(f"{len(tr.token_ids)} tokens tracked, none left to generate")
        params["max_new_tokens"] = budget
        out = await post(self.url, {"input_ids": tr.token_ids, "return_logprob": True, "sampling_params": params})
        pairs = out["meta_info"].get("output_token_logprobs") or []
        ids = [p[1] for p in pairs]
        tr.extend(ids, 1, [p[0] for p in pairs])
        self.last_meta = out["meta_info"]
        return out.get("text") or self.tokenizer.decode(ids), out["meta_info"].get("finish_reason") or {}


class ToolLimiter:
    """Hook: counts tool rounds (parallel calls of one assistant turn are one round) and calls; ends the episode when
    the round limit is reached."""

    def __init__(self, max_tool_iters: int | None = None, max_tool_calls: int | None = None):
        self.max_tool_iters, self.max_tool_calls = max_tool_iters, max_tool_calls
        self.tool_iter_count = self.tool_call_count = 0

    def before_tools(self, calls: list[dict]):
        if self.max_tool_iters is not None and self.tool_iter_count >= self.max_tool_iters:
            raise ToolLimitReached(f"{self.tool_iter_count} tool rounds")
        if self.max_tool_calls is not None and self.tool_call_count + len(calls) > self.max_tool_calls:
            raise ToolLimitReached(f"{self.tool_call_count} tool calls")
        self.tool_iter_count += 1
        self.tool_call_count += len(calls)


class ToolAgent:
    def __init__(self, model: TokenTrackingModel, tools=(), hooks=(), system_prompt: str | None = None, max_turns: int = 32):
        self.model, self.hooks, self.max_turns = model, list(hooks), max_turns
        self.tools = {t.tool_spec["function"]["name"]: t for t in tools}
        self.specs = [t.tool_spec for t in tools]
        self.messages = [{"role": "system", "content": system_prompt}] if system_prompt else []

    async def _run_tool(self, use: dict) -> str:
        fn = self.tools.get(use["name"])
        if fn is None:
            return f"Error: unknown tool {use['name']!r}"
        try:
            res = fn(**use["arguments"])
            if inspect.isawaitable(res):
                res = await res
            return res if isinstance(res, str) else json.dumps(res)
        except Exception as e:  # a tool failure is an observation, not the end of the episode
            return f"Error: {type(e).__name__}: {e}"

    async def invoke_async(self, prompt: str) -> str:
        """Runs until the model answers without a tool call. Returns the final text."""
        self.messages.append({"role": "user", "content": prompt})
        for turn in range(self.max_turns):
            text, finish = await self.model.complete(self.messages, self.specs)
            if finish.get("type") in ("length", "abort"):
                raise ContextBudgetExceeded(f"generation ended with {finish.get('type')}")
            parsed = parse_model_output(text, self.specs)
            if not parsed.tool_uses:
                self.messages.append({"role": "assistant", "content": parsed.text or text})
                return parsed.text or text
            calls = [{"id": f"call_{turn}_{i}", "type": "function", "function": {"name": u["name"], "arguments": json.dumps(u["arguments"])}}
                     for i, u in enumerate(parsed.tool_uses)]  # fmt: skip
            self.messages.append({"role": "assistant", "content": parsed.text or "", "tool_calls": calls})
            for h in self.hooks:
                h.before_tools(calls)
            results = await asyncio.gather(*(self._run_tool(u) for u in parsed.tool_uses))
            for c, u, r in zip(calls, parsed.tool_uses, results):
                self.messages.append({"role": "tool", "tool_call_id": c["id"], "name": u["name"], "content": r})
        raise ToolLimitReached(f"{self.max_turns} turns")
