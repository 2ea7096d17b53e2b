"""Math with a Python tool, driven by an agent loop that works on messages while the sample is built from tokens.

    --custom-generate-function-path examples.strands_sglang.generate_with_strands.generate
    --custom-rm-path examples.strands_sglang.generate_with_strands.reward_func

Do not pass ``--apply-chat-template``: the agent renders the conversation itself, a templated prompt would be wrapped
twice. The sample's tokens, loss mask and log-probs come from the model client's trajectory (see ``token_agent.py``);
an episode that ends early (tool-round limit, context budget, an error in the loop) is kept as TRUNCATED with the tokens
it has. The reward is the DAPO math score; failed answers lose a little less when the model did use the tool.
Same role as examples/strands_sglang/generate_with_strands.py in the reference.
"""

from __future__ import annotations

import logging

from examples.retool.python_tool import run_python
from slime_b200.rollout.sglang_rollout import GenerateState
from slime_b200.utils.types import Sample

from .token_agent import ToolAgent, ToolLimiter, TokenTrackingModel, tool

logger = logging.getLogger(__name__)

SYSTEM_PROMPT = (
    "You are a helpful math-solving assistant with access to the `execute_python_code` tool.\n\n"
    "Guidelines:\n"
    "- For any numerical or symbolic computation, use the `execute_python_code` tool instead of computing in your head.\n"
    "- Break the problem into clear steps and call the tool whenever a step needs computation.\n"
    "- After your reasoning, give the final result inside \\boxed{}."
)
MAX_TOOL_ITERS = 5


@tool
async def execute_python_code(code: str) -> str:
    """Execute Python code and return what it prints."""
    _, text = await run_python(code)
    return text


async def generate(args, sample: Sample, sampling_params: dict) -> Sample:
    assert not getattr(args, "partial_rollout", False), "partial rollout is not supported by this agent loop"
    state = GenerateState(args)
    model = TokenTrackingModel(state.tokenizer, f"http://{args.sglang_router_ip}:{args.sglang_router_port}/generate",
                               sampling_params, max_context_len=getattr(args, "rollout_max_context_len", None))  # fmt: skip
    limiter = ToolLimiter(max_tool_iters=getattr(args, "strands_max_tool_iters", MAX_TOOL_ITERS))
    agent = ToolAgent(model, tools=[execute_python_code], hooks=[limiter], system_prompt=SYSTEM_PROMPT)
    prompt = sample.prompt if isinstance(sample.prompt, str) else sample.prompt[0]["content"]
    try:
        await agent.invoke_async(prompt)
        sample.status = Sample.Status.COMPLETED
    except Exception as e:  # every early end keeps the trajectory
        sample.status = Sample.Status.TRUNCATED
        logger.warning("truncated: %s: %s", type(e).__name__, e)
    tr = model.rollout
    n = tr.initial_prompt_length
    sample.tokens = list(tr.token_ids)
    sample.loss_mask = tr.loss_mask[n:]
    sample.rollout_log_probs = tr.logprobs[n:]
    sample.response_length = len(tr.token_ids) - n
    sample.response = state.tokenizer.decode(tr.token_ids[n:], skip_special_tokens=False)
    sample.metadata = {**(sample.metadata or {}), "tool_iters": limiter.tool_iter_count, "tool_calls": limiter.tool_call_count}
    return sample


async def reward_func(args, sample: Sample, **kwargs) -> float:
    from slime_b200.rollout.rm_hub import math_dapo_utils

    label = str(sample.label or "")
    res = math_dapo_utils.compute_score(sample.response or "", label, strict_box_verify=False)
    if res["pred"] == "[INVALID]":
        res = math_dapo_utils.compute_score(sample.response or "", label, strict_box_verify=True)
    score = float(res["score"])
    if score < 0:  # a wrong answer costs a little less when the tool was used
        tool_iters = (sample.metadata or {}).get("tool_iters", 0)
        score = min(-0.6, score + (tool_iters - 2) / 2 * 0.1)
    return score
