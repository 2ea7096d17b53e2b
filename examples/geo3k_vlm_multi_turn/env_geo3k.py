"""Geometry-3K with an answer-checking tool: the model may call ``calc_score`` (alias ``calc_geo3k_reward``) with a
candidate answer, ``<tool_call>{"name": "calc_score", "arguments": {"answer": "..."}}</tool_call>``, and is told
whether it matches the reference; it can then revise or commit. A turn without a tool call ends the episode. On the turn
before the last the feedback says that no further check is possible.
(Same role as examples/geo3k_vlm_multi_turn/env_geo3k.py in the reference.)
"""

from __future__ import annotations

import json
import re

from slime_b200.rollout.rm_hub.math_utils import grade_answer_verl

from .base_env import BaseInteractionEnv

TOOL_CALL = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.DOTALL)
TOOL_NAMES = ("calc_score", "calc_geo3k_reward")
USAGE = ('Call `calc_score` as <tool_call>{"name": "calc_score", "arguments": {"answer": "<your answer>"}}</tool_call> '
         "to check your solution.")  # fmt: skip


def parse_tool_call(text: str) -> dict | None:
    """The last well-formed tool call of a response: ``{"name", "arguments"}`` (OpenAI-style nesting accepted)."""
    found = TOOL_CALL.findall(text)
    if not found:
        return None
    try:
        payload = json.loads(found[-1])
    except json.JSONDecodeError:
        return None
    fn = payload.get("function") or {}
    name, arguments = payload.get("name") or fn.get("name"), payload.get("arguments") or fn.get("arguments") or {}
    if isinstance(arguments, str):
        try:
            arguments = json.loads(arguments)
        except json.JSONDecodeError:
            return None
    return {"name": name, "arguments": arguments} if name and isinstance(arguments, dict) else None


class Geo3kEnv(BaseInteractionEnv):
    def __init__(self, ground_truth: str | None, max_turns: int | None):
        self.ground_truth = None if ground_truth is None else str(ground_truth)
        self.max_turns = max_turns
        self.reset()

    def reset(self):
        self.turn, self.tool_calls, self.last_tool_score = 0, [], None
        return {}, {"ground_truth_available": self.ground_truth is not None}

    def score(self, answer: str) -> float:
        if not self.ground_truth:
            return 0.0
        answer = answer.strip()
        for cand in ([answer] if "\\boxed" in answer else [answer, "\\boxed{" + answer + "}"]):
            try:
                if grade_answer_verl(cand, self.ground_truth):
                    return 1.0
            except Exception:  # noqa: BLE001  an unparsable candidate is a wrong one
                continue
        return 0.0

    def _feedback(self, score: float, answer: str) -> str:
        if score == 1.0:
            return (f"calc_score result: {score}. Parsed answer '{answer}' matches the reference. "
                    "You can now stop reasoning and give the final solution in \\boxed{}.")  # fmt: skip
        text = (f"calc_score result: {score}. Parsed answer '{answer}' does not match the reference. Your answer is wrong: "
                "try a different line of reasoning and do not repeat the same answer.")  # fmt: skip
        # the reminder arrives one turn early, so that the model reads it before its last turn
        warn_from = None if self.max_turns is None else max(self.max_turns - 2, 0) if self.max_turns >= 2 else self.max_turns - 1
        if warn_from is not None and self.turn - 1 >= warn_from:
            text += (" You have one chance left, so do not call the tool again: give your final answer as "
                     "Answer: \\boxed{$Answer}.")  # fmt: skip
        return text

    def step(self, response_text: str):
        self.turn += 1
        last = self.max_turns is not None and self.turn >= self.max_turns
        call = parse_tool_call(response_text)
        info = {"tool_call": call, "tool_executed": False}
        if call is None:
            return {"obs_str": "No tool call detected; ending the episode.", "role": "tool"}, True, info
        if call["name"].strip() not in TOOL_NAMES:
            return {"obs_str": f"Tool `{call['name']}` is not supported. {USAGE}", "role": "tool"}, last, info
        answer = str(call["arguments"].get("answer") or "")
        if not answer.strip():
            return {"obs_str": f"The tool call carries no `answer`. {USAGE}", "role": "tool"}, last, {**info, "answer_missing": True}
        s = self.score(answer)
        self.last_tool_score = s
        self.tool_calls.append({"name": call["name"], "answer": answer, "score": s})
        info.update(self.tool_calls[-1], tool_executed=True)
        return {"obs_str": self._feedback(s, answer), "role": "tool", "tool_score": s}, last, info


def build_env(sample=None, args=None, **_):
    max_turns = getattr(args, "max_turns", None)
    if max_turns is None:
        raise ValueError("max_turns must be set in the file named by --custom-config-path")
    return Geo3kEnv(None if sample is None or sample.label is None else sample.label, max_turns)
