"""Search-augmented generation as a custom generate function (tool loop of at most ``max_turns`` turns).

    --custom-generate-function-path examples.search_r1.generate_with_search.generate
    --custom-rm-path examples.search_r1.generate_with_search.reward_func

Per turn the engine is stopped at ``</search>`` or ``</answer>`` (``sampling_params.stop`` with ``no_stop_trim`` so the
closing tag stays in the text). After a ``<search>query</search>`` the retrieved passages are appended as
``<information>...</information>``: those observation tokens enter ``sample.tokens`` with loss mask 0 and log-prob 0.0,
because the policy did not produce them. Generated token ids and log-probs are taken from
``meta_info.output_token_logprobs`` and never re-tokenised. The reward is exact match of the ``<answer>`` against the
label plus a small bonus for a well-formed trace.

The retriever is a function ``async search(args, query) -> list[str]``: by default a word-overlap ranker over
``args.search_corpus`` (a list of passages, e.g. from ``--custom-config-path``); set ``args.search_url`` to POST
``{"queries": [...], "topk": k}`` to a retrieval server instead.
Parity: examples/search-r1/generate_with_search.py:145-293 and qa_em_format.py (same hooks and token bookkeeping).
"""

from __future__ import annotations

import re
import string

from slime_b200.rollout.sglang_rollout import GenerateState
from slime_b200.utils.http_utils import post
from slime_b200.utils.types import Sample

CONFIG = {"max_turns": 2, "topk": 3, "format_bonus": 0.1}
_SEARCH = re.compile(r"<search>(.*?)</search>", re.S)
_ANSWER = re.compile(r"<answer>(.*?)</answer>", re.S)


async def search(args, query: str) -> list[str]:
    topk = getattr(args, "search_topk", CONFIG["topk"])
    url = getattr(args, "search_url", None)
    if url:
        out = await post(url, {"queries": [query], "topk": topk})
        hits = out.get("result", [[]])[0]
        return [h["document"]["contents"] if isinstance(h, dict) else str(h) for h in hits]
    corpus = getattr(args, "search_corpus", None) or []
    words = set(_normalize(query).split())
    ranked = sorted(corpus, key=lambda p: -len(words & set(_normalize(p).split())))
    return ranked[:topk]


def format_observation(passages: list[str]) -> str:
    body = "\n".join(f"Doc {i + 1}: {p}" for i, p in enumerate(passages))
    return f"\n\n<information>{body}</information>\n\n"


async def generate(args, sample: Sample, sampling_params: dict) -> Sample:
    state = GenerateState(args)
    tok = state.tokenizer
    url = f"http://{args.sglang_router_ip}:{args.sglang_router_port}/generate"
    prompt_ids = tok.encode(sample.prompt, add_special_tokens=False) if isinstance(sample.prompt, str) else list(sample.prompt)
    if not sample.tokens:
        sample.tokens = list(prompt_ids)
    budget = sampling_params["max_new_tokens"]
    max_turns = getattr(args, "search_max_turns", CONFIG["max_turns"])
    for turn in range(max_turns + 1):
        remaining = budget - sample.response_length
        if remaining <= 0:
            sample.status = Sample.Status.TRUNCATED
            break
        sp = {**sampling_params, "max_new_tokens": remaining, "stop": ["</search>", "</answer>"], "no_stop_trim": True}
        out = await post(url, {"input_ids": sample.tokens, "sampling_params": sp, "return_logprob": True})
        pairs = out["meta_info"].get("output_token_logprobs") or []
        sample.append_response_tokens(args, tokens=[p[1] for p in pairs], log_probs=[p[0] for p in pairs], trainable=True,
                                      meta_info=out["meta_info"], text=out.get("text", ""))  # fmt: skip
        if sample.status in (Sample.Status.TRUNCATED, Sample.Status.ABORTED):
            break
        text = out.get("text", "")
        query = _SEARCH.findall(text)
        if "</answer>" in text or not query or turn == max_turns:
            break
        obs = format_observation(await search(args, query[-1].strip()))
        obs_ids = tok.encode(obs, add_special_tokens=False)
        # tool output: part of the context, not of the objective
        sample.append_response_tokens(args, tokens=obs_ids, trainable=False, text=obs)
        sample.status = Sample.Status.PENDING
    if sample.status == Sample.Status.PENDING:
        sample.status = Sample.Status.COMPLETED
    return sample


def _normalize(s: str) -> str:
    s = "".join(ch for ch in s.lower() if ch not in set(string.punctuation))
    return " ".join(w for w in s.split() if w not in ("a", "an", "the"))


def compute_score(response: str, label, format_bonus: float = CONFIG["format_bonus"]) -> float:
    answers = _ANSWER.findall(response)
    well_formed = len(answers) == 1 and response.count("<search>") == response.count("</search>")
    if not answers:
        return 0.0
    golds = label if isinstance(label, (list, tuple)) else [label]
    hit = any(_normalize(answers[-1]) == _normalize(str(g)) for g in golds)
    return (1.0 if hit else 0.0) + (format_bonus if well_formed and not hit else 0.0)


async def reward_func(args, sample: Sample, **kwargs) -> float:
    return compute_score(sample.response or "", sample.label)
