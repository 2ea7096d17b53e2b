"""The worked examples (custom generate functions) against a scripted engine: hook contracts and token bookkeeping."""

import asyncio
from argparse import Namespace

import pytest

from slime_b200.agent.aiohttp_threaded import serve_in_thread
from slime_b200.rollout import sglang_rollout
from slime_b200.utils.types import Sample


class WordTok:
    """Stable word-level tokenizer: id = 100 + index in an append-only vocabulary."""

    def __init__(self):
        self.vocab = {}

    def encode(self, text, add_special_tokens=False):
        return [self.vocab.setdefault(w, 100 + len(self.vocab)) for w in text.split()]

    def decode(self, ids, **kw):
        inv = {v: k for k, v in self.vocab.items()}
        return " ".join(inv[i] for i in ids)


@pytest.fixture
def engine(monkeypatch):
    """A fake /generate: answers come from ``script`` (a function of the decoded prompt), tokenised with WordTok."""
    from aiohttp import web

    tok = WordTok()
    state = {"script": lambda prompt: "ok", "calls": []}

    async def generate(request):
        body = await request.json()
        prompt = tok.decode(body["input_ids"])
        text = state["script"](prompt)
        state["calls"].append((prompt, body["sampling_params"]))
        ids = tok.encode(text)
        budget = body["sampling_params"]["max_new_tokens"]
        finish = {"type": "length"} if len(ids) > budget else {"type": "stop"}
        ids = ids[:budget]
        return web.json_response({"text": tok.decode(ids), "output_ids": ids,
                                  "meta_info": {"output_token_logprobs": [[-0.5, i, None] for i in ids], "finish_reason": finish,
                                                "prompt_tokens": len(body["input_ids"]), "completion_tokens": len(ids)}})

    app = web.Application()
    app.router.add_post("/generate", generate)
    h = serve_in_thread(app, host="127.0.0.1")
    monkeypatch.setattr(sglang_rollout, "load_tokenizer", lambda *a, **k: tok)
    monkeypatch.setattr(sglang_rollout, "load_processor", lambda *a, **k: None)
    sglang_rollout.GenerateState.clear_instances()
    args = Namespace(hf_checkpoint="tok", sglang_router_ip="127.0.0.1", sglang_router_port=h.port, sglang_server_concurrency=4,
                     rollout_num_gpus=1, rollout_num_gpus_per_engine=1, rollout_temperature=1.0, rollout_top_p=1.0,
                     rollout_top_k=-1, rollout_max_response_len=64, rollout_stop=None, rollout_stop_token_ids=None,
                     rollout_skip_special_tokens=False, n_samples_per_prompt=1, rm_type="math", custom_rm_path=None,
                     partial_rollout=False, use_rollout_routing_replay=False)
    yield args, state, tok
    h.stop()
    sglang_rollout.GenerateState.clear_instances()


def test_search_example_masks_observations(engine):
    from examples.search_r1 import generate_with_search as ex

    args, state, tok = engine
    args.search_corpus = ["Paris is the capital of France .", "Berlin is in Germany .", "The Seine crosses Paris ."]
    args.search_topk = 1

    def script(prompt):
        if "<information>" in prompt:
            return "so <answer> Paris </answer>"
        return "hm <search> capital of France </search>"

    state["script"] = script
    s = Sample(index=0, prompt="what is the capital of France ?", label="Paris")
    out = asyncio.run(ex.generate(args, s, {"max_new_tokens": 64, "temperature": 1.0}))
    assert out.status == Sample.Status.COMPLETED and len(state["calls"]) == 2
    assert state["calls"][0][1]["stop"] == ["</search>", "</answer>"] and state["calls"][0][1]["no_stop_trim"] is True
    n_prompt = len(tok.encode("what is the capital of France ?"))
    assert out.response_length == len(out.tokens) - n_prompt == len(out.loss_mask) == len(out.rollout_log_probs)
    first = len(tok.encode("hm <search> capital of France </search>"))
    obs = len(tok.encode(ex.format_observation(["Paris is the capital of France ."])))
    assert out.loss_mask == [1] * first + [0] * obs + [1] * len(tok.encode("so <answer> Paris </answer>"))
    assert out.rollout_log_probs[first : first + obs] == [0.0] * obs and out.rollout_log_probs[0] == -0.5
    assert "Doc 1: Paris is the capital" in out.response
    assert asyncio.run(ex.reward_func(args, out)) == 1.0
    assert ex.compute_score("<answer> Rome </answer>", "Paris") == pytest.approx(0.1) and ex.compute_score("no tags", "x") == 0
    # budget: the second turn only gets what the first left
    assert state["calls"][1][1]["max_new_tokens"] == 64 - first - obs


def test_multi_agent_example_fans_out_one_rollout(engine):
    from examples.multi_agent import agent_system as ex

    args, state, _tok = engine
    args.num_parallel = 3
    n = {"solver": 0}

    def script(prompt):
        if prompt.startswith("Several candidate"):
            return "Best: 2"
        n["solver"] += 1
        return "thus </think> \\boxed{4}" if n["solver"] == 2 else "thus </think> \\boxed{5}"

    state["script"] = script
    args.rm_type = "deepscaler"
    parent = Sample(index=7, group_index=3, rollout_id=7, prompt="2 + 2 = ?", label="4")
    outs = asyncio.run(ex.generate_with_multi_agents(args, parent, {"max_new_tokens": 32}))
    assert len(outs) == 4 and all(isinstance(s, Sample) for s in outs)
    assert {(s.index, s.group_index, s.rollout_id) for s in outs} == {(7, 3, 7)}
    roles = sorted(s.metadata["agent_role"] for s in outs)
    assert roles == ["selector", "solver", "solver", "solver"]
    sel = next(s for s in outs if s.metadata["agent_role"] == "selector")
    # the three solver calls run concurrently, so which of them drew the correct answer varies; the selector always
    # names candidate 2, and the team weight follows from whether that candidate was the correct one
    correct = sel.metadata["final_correct"]
    w = 1.2 if correct else 0.8
    assert sel.metadata["selected_candidate"] == 1 and sel.reward == pytest.approx(w if correct else 0.0)
    assert sorted(round(s.reward, 3) for s in outs if s.metadata["agent_role"] == "solver") == [0.0, 0.0, w]
    assert all(s.response_length == len(s.rollout_log_probs) > 0 and s.status == Sample.Status.COMPLETED for s in outs)


def test_retool_example_runs_the_interpreter_between_turns(engine):
    from examples.retool import generate_with_retool as ex

    args, state, tok = engine
    call = '<tool_call> {"name": "code_interpreter", "arguments": {"code": "print(6*7)"}} </tool_call>'

    def script(prompt):
        if "<tool_response>" in prompt:
            assert "<tool_response> 42 </tool_response>" in prompt
            return "so Answer: 42"
        return "compute " + call

    state["script"] = script
    s = Sample(index=0, prompt="what is 6 times 7 ?", label="42")
    out = asyncio.run(ex.generate(args, s, {"max_new_tokens": 200, "temperature": 1.0}))
    assert out.status == Sample.Status.COMPLETED and len(state["calls"]) == 2
    assert state["calls"][0][1]["stop"] == ["</tool_call>"] and state["calls"][0][1]["no_stop_trim"] is True
    assert out.metadata["tool_calls"] == 1 and out.metadata["tool_calls_ok"] == 1
    first, obs = len(tok.encode("compute " + call)), len(tok.encode(ex.format_observation("42")))
    assert out.loss_mask == [1] * first + [0] * obs + [1] * 3
    assert out.response_length == len(out.loss_mask) == len(out.rollout_log_probs)
    assert asyncio.run(ex.reward_func(args, out)) == 1.0
    # a wrong final answer still earns the tool bonus; a broken snippet does not
    out.label = "43"
    assert asyncio.run(ex.reward_func(args, out)) == pytest.approx(-1.0 + ex.TOOL_BONUS)
    assert ex.extract_code('<tool_call>{"name": "other", "arguments": {}}</tool_call>') is None
    assert ex.extract_code("<tool_call>{broken</tool_call>") is None
    ok, text = asyncio.run(ex.run_python("import time\nprint(1/0)"))
    assert not ok and "ZeroDivisionError" in text
