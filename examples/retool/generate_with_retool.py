"""Tool-integrated reasoning: the policy interleaves text with calls to a Python interpreter.

    --custom-generate-function-path examples.retool.generate_with_retool.generate
    --custom-rm-path examples.retool.generate_with_retool.reward_func

Conversation format: the system turn lists the tool (Qwen-style ``<tools>`` block); the model calls it with

    <tool_call>
    {"name": "code_interpreter", "arguments": {"code": "print(2**10)"}}
    </tool_call>

or simply writes a fenced ``python`` block followed by ``</code>``-less stop; both are accepted. Generation stops at
``</tool_call>`` (kept in the text), the snippet runs in ``python_tool.run_python`` and its output comes back as

    <|im_start|>user\\n<tool_response>\\n...\\n</tool_response><|im_end|>\\n<|im_start|>assistant\\n

Those observation tokens join ``sample.tokens`` with loss mask 0 and log-prob 0; the model's own tokens keep the ids and
log-probs the engine returned (no re-tokenisation). At most ``MAX_TURNS`` tool calls per sample; the response budget is
shared by all turns. Reward: DAPO-style math score of the final ``Answer:`` / boxed answer, with a small bonus per
successful tool call while the answer is still wrong (so that early training learns to call the tool at all).
Same role as examples/retool/generate_with_retool.py:215-432 in the reference.
"""

from __future__ import annotations

import json
import re

from slime_b200.rollout.sglang_rollout import GenerateState
from slime_b200.utils.http_utils import post
from slime_b200.utils.types import Sample

from .python_tool import TOOL_SPEC, run_python

MAX_TURNS = 8
TOOL_BONUS = 0.05
_CALL = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)
_FENCE = re.compile(r"```python\s*(.*?)```", re.S)

SYSTEM_TOOLS = (
    "# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
    "You are provided with function signatures within <tools></tools> XML tags:\n<tools>\n" + json.dumps(TOOL_SPEC) +
    "\n</tools>\n\nFor each function call, return a json object with function name and arguments within "
    "<tool_call></tool_call> XML tags:\n<tool_call>\n{\"name\": <function-name>, \"arguments\": <args-json-object>}\n</tool_call>"
)  # fmt: skip


def build_prompt(messages_or_text) -> str:
    """ChatML prompt with the tool block in the system turn."""
    msgs = messages_or_text if isinstance(messages_or_text, list) else [{"role": "user", "content": str(messages_or_text)}]
    system = "You are a helpful assistant."
    if msgs and msgs[0].get("role") == "system":
        system, msgs = msgs[0]["content"], msgs[1:]
    parts = [f"<|im_start|>system\n{system}\n\n{SYSTEM_TOOLS}<|im_end|>\n"]
    for m in msgs:
        parts.append(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n")
    parts.append("<|im_start|>assistant\n")
    return "".join(parts)


def extract_code(text: str) -> str | None:
    """The snippet of the LAST tool call in ``text`` (json form first, fenced block as a fallback)."""
    calls = _CALL.findall(text)
    if calls:
        try:
            obj = json.loads(calls[-1])
            if obj.get("name") == "code_interpreter":
                args = obj.get("arguments", {})
                args = json.loads(args) if isinstance(args, str) else args
                return args.get("code")
        except (json.JSONDecodeError, AttributeError, TypeError):
            return None
        return None
    fenced = _FENCE.findall(text)
    return fenced[-1] if fenced and text.rstrip().endswith("```") else None


def format_observation(output: str) -> str:
    return f"<|im_end|>\n<|im_start|>user\n<tool_response>\n{output}\n</tool_response><|im_end|>\n<|im_start|>assistant\n"


async def generate(args, sample: Sample, sampling_params: dict) -> Sample:
    state = GenerateState(args)
    tok = state.tokenizer
    url = f"http://{args.sglang_router_ip}:{args.sglang_router_port}/generate"
    if not sample.tokens:
        prompt = build_prompt(sample.prompt)
        sample.tokens = tok.encode(prompt, add_special_tokens=False)
    budget = sampling_params["max_new_tokens"]
    max_turns = getattr(args, "retool_max_turns", MAX_TURNS)
    calls = ok_calls = 0
    for turn in range(max_turns + 1):
        remaining = budget - sample.response_length
        if remaining <= 0:
            sample.status = Sample.Status.TRUNCATED
            break
        sp = {**sampling_params, "max_new_tokens": remaining, "stop": ["</tool_call>"], "no_stop_trim": True}
        out = await post(url, {"input_ids": sample.tokens, "sampling_params": sp, "return_logprob": True})
        pairs = out["meta_info"].get("output_token_logprobs") or []
        text = out.get("text", "")
        sample.append_response_tokens(args, tokens=[p[1] for p in pairs], log_probs=[p[0] for p in pairs], trainable=True,
                                      meta_info=out["meta_info"], text=text)  # fmt: skip
        if sample.status in (Sample.Status.TRUNCATED, Sample.Status.ABORTED):
            break
        code = extract_code(text)
        if code is None or turn == max_turns:
            break
        ok, result = await run_python(code)
        calls += 1
        ok_calls += int(ok)
        obs = format_observation(result)
        sample.append_response_tokens(args, tokens=tok.encode(obs, add_special_tokens=False), trainable=False, text=obs)
        sample.status = Sample.Status.PENDING
    if sample.status == Sample.Status.PENDING:
        sample.status = Sample.Status.COMPLETED
    sample.metadata = {**(sample.metadata or {}), "tool_calls": calls, "tool_calls_ok": ok_calls}
    return sample


async def reward_func(args, sample: Sample, **kwargs) -> float:
    from slime_b200.rollout.rm_hub import math_dapo_utils

    score = math_dapo_utils.compute_score(sample.response or "", str(sample.label))
    value = float(score["score"] if isinstance(score, dict) else score)
    if value <= 0:
        value += TOOL_BONUS * min((sample.metadata or {}).get("tool_calls_ok", 0), 2)
    return value
