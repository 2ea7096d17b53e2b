"""Solver -> selector pipeline returning several training samples for one prompt.

    --custom-generate-function-path examples.multi_agent.agent_system.generate_with_multi_agents

``num_parallel`` solvers answer the problem independently; a selector then reads all candidate answers and names the
best one. Every model call becomes its own ``Sample`` (prompt = what that agent saw, response = what it produced, token
ids and log-probs from the engine). All of them are stamped with the parent's ``rollout_id`` / ``index`` /
``group_index`` so the trainer treats them as one rollout when it splits steps and normalises the loss. Rewards:
each solver is graded on its own answer; the selector gets the grade of the answer it picked; if the final
(selected) answer is correct every reward is scaled by ``correct_reward_weight``, otherwise by
``incorrect_reward_weight``: the team is rewarded for the outcome, the members for their part.
Parity: examples/multi_agent/agent_system.py:198-296 and rollout_with_multi_agents.py:16-33 (hook and fan-out contract).
"""

from __future__ import annotations

import asyncio
import copy
import random
import re

from slime_b200.rollout.rm_hub import async_rm
from slime_b200.rollout.sglang_rollout import GenerateState
from slime_b200.utils.http_utils import post
from slime_b200.utils.types import Sample

CONFIG = {"num_parallel": 3, "correct_reward_weight": 1.2, "incorrect_reward_weight": 0.8}
SOLVER_PROMPT = "Solve the problem. Put the final answer in \\boxed{{}}.\n\nProblem: {problem}\n"
SELECTOR_PROMPT = ("Several candidate solutions to a problem follow. Reply with 'Best: <number>' for the most convincing one.\n\n"
                   "Problem: {problem}\n\n{candidates}\n")  # fmt: skip


def _child(parent: Sample, prompt_text: str, role: str) -> Sample:
    s = Sample(index=parent.index, group_index=parent.group_index, rollout_id=parent.rollout_id, prompt=prompt_text,
               label=parent.label, metadata={**(parent.metadata or {}), "agent_role": role})  # fmt: skip
    return s


async def call_model(args, sample: Sample, sampling_params: dict) -> Sample:
    """One engine call for ``sample.prompt`` (text); fills tokens, response, log-probs and status."""
    state = GenerateState(args)
    ids = state.tokenizer.encode(sample.prompt, add_special_tokens=False)
    sample.tokens = list(ids)
    url = f"http://{args.sglang_router_ip}:{args.sglang_router_port}/generate"
    out = await post(url, {"input_ids": ids, "sampling_params": dict(sampling_params), "return_logprob": True})
    pairs = out["meta_info"].get("output_token_logprobs") or []
    sample.append_response_tokens(args, tokens=[p[1] for p in pairs], log_probs=[p[0] for p in pairs], trainable=True,
                                  meta_info=out["meta_info"], text=out.get("text", ""))  # fmt: skip
    if sample.status == Sample.Status.PENDING:
        sample.status = Sample.Status.COMPLETED
    return sample


def pick_index(selector_text: str, n: int) -> int:
    m = re.findall(r"Best:\s*(\d+)", selector_text or "")
    k = int(m[-1]) - 1 if m else -1
    return k if 0 <= k < n else random.randrange(n)


async def run_agent_system(args, sample: Sample, sampling_params: dict) -> list[Sample]:
    n = getattr(args, "num_parallel", CONFIG["num_parallel"])
    problem = sample.prompt if isinstance(sample.prompt, str) else str(sample.prompt)
    solvers = [_child(sample, SOLVER_PROMPT.format(problem=problem), "solver") for _ in range(n)]
    solvers = list(await asyncio.gather(*[call_model(args, s, copy.deepcopy(sampling_params)) for s in solvers]))
    cands = "\n\n".join(f"Candidate {i + 1}:\n{s.response}" for i, s in enumerate(solvers))
    selector = await call_model(args, _child(sample, SELECTOR_PROMPT.format(problem=problem, candidates=cands), "selector"),
                                copy.deepcopy(sampling_params))  # fmt: skip
    grades = await asyncio.gather(*[async_rm(args, s) for s in solvers])
    for s, g in zip(solvers, grades):
        s.reward = float(g)
    chosen = pick_index(selector.response, n)
    selector.reward = solvers[chosen].reward
    selector.metadata["selected_candidate"] = chosen
    final_correct = solvers[chosen].reward > 0
    w = getattr(args, "correct_reward_weight" if final_correct else "incorrect_reward_weight",
                CONFIG["correct_reward_weight" if final_correct else "incorrect_reward_weight"])  # fmt: skip
    out = solvers + [selector]
    for s in out:
        s.reward *= w
        s.metadata["final_correct"] = final_correct
    return out


async def generate_with_multi_agents(args, sample: Sample, sampling_params: dict, evaluation: bool = False) -> list[Sample]:
    samples = await run_agent_system(args, sample, sampling_params)
    random.shuffle(samples)
    return samples
