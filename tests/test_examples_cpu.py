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


def test_coding_agent_example_fixes_a_bug_and_is_graded_in_a_clean_sandbox(monkeypatch):
    """Whole session on this host: the in-sandbox agent calls the adapter twice (a file rewrite, then a plain reply), the
    patch is extracted with git, applied to a fresh workspace with a hidden test, and the rows carry reward 1."""
    import json

    from examples.coding_agent_rl import generate as ex
    from examples.coding_agent_rl import tasks
    from slime_b200.agent import adapters
    from slime_b200.agent.trajectory import TurnRecord
    from slime_b200.utils import processing_utils
    from slime_b200.utils.misc import SingletonMeta

    class Tok:
        def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=True, tools=None):
            text = "".join(f"[{m['role']}]{m.get('content') or ''}" + "".join(json.dumps(c["function"]) for c in m.get("tool_calls", []))
                           for m in messages)  # fmt: skip
            return [ord(c) for c in text + ("[assistant]" if add_generation_prompt else "")]

        def decode(self, ids, skip_special_tokens=False):
            return "".join(chr(i) for i in ids)

    fixed = "def add(a, b):\\n    return a + b\\n"
    outputs = ['I will fix it.<tool_call>{"name": "write_file", "arguments": {"path": "calc.py", "content": "' + fixed + '"}}</tool_call>',
               "The subtraction was a typo; fixed."]  # fmt: skip

    async def fake(prompt_ids, session, body, *, adapter, session_id=None):
        text = outputs.pop(0)
        return TurnRecord(prompt_ids=list(prompt_ids), output_ids=[ord(c) for c in text], finish_reason="stop",
                          output_log_probs=[-0.25] * len(text))  # fmt: skip

    monkeypatch.setattr(adapters, "call_engine_generate", fake)
    monkeypatch.setattr(processing_utils, "load_tokenizer", lambda *a, **k: Tok())
    monkeypatch.setenv("CODING_AGENT", "mini")
    monkeypatch.setenv("CODING_SANDBOX", "local")
    SingletonMeta._instances.pop(ex.AdapterService, None)
    args = Namespace(hf_checkpoint="tok", sglang_router_ip="127.0.0.1", sglang_router_port=1, rollout_max_context_len=4096)
    task = {"instance_id": "calc-1", "problem": "add() in calc.py returns the wrong result. Fix it.",
            "files": {"calc.py": "def add(a, b):\n    return a - b\n", "README.md": "calc\n"},
            "test_files": {"test_calc.py": "from calc import add\nassert add(2, 3) == 5\n"}, "test_cmd": "python test_calc.py"}  # fmt: skip
    try:
        s = Sample(index=0, prompt="fix the bug", label=json.dumps(task))
        rows = asyncio.run(ex.generate(args, s, {"max_new_tokens": 256, "temperature": 1.0}))
        assert not outputs and len(rows) >= 1, [r.metadata for r in rows]
        assert all(r.reward == 1.0 for r in rows) and rows[-1].metadata["verdict"] == "solved"
        assert rows[-1].metadata["agent_exit_code"] == 0 and rows[-1].metadata["patch_chars"] > 0
        assert sum(rows[-1].loss_mask) > 0 and len(rows[-1].loss_mask) == rows[-1].response_length
        # an agent that changes nothing scores 0 without running the tests
        outputs.append("Looks fine to me.")
        rows = asyncio.run(ex.generate(args, Sample(index=1, prompt="fix", label=json.dumps(task)), {"max_new_tokens": 64}))
        assert rows[-1].reward == 0.0 and rows[-1].metadata["verdict"] == "empty_patch"
        # rows without a usable task abort instead of raising
        bad = asyncio.run(ex.generate(args, Sample(index=2, prompt="x", label="{}"), {}))
        assert bad[0].status == Sample.Status.ABORTED and "bad_task" in bad[0].metadata["abort_reason"]
    finally:
        service = SingletonMeta._instances.pop(ex.AdapterService, None)
        if service is not None:
            service.handle.stop()

    async def wrong_patch():
        t = tasks.Task("t", "p", "python test_calc.py", files=task["files"], test_files=task["test_files"])
        return await tasks.grade(t, "diff --git a/nope.py b/nope.py\n--- a/nope.py\n+++ b/nope.py\n@@ -1 +1 @@\n-x\n+y\n", ex.sandbox_factory())

    assert asyncio.run(wrong_patch())[1]["verdict"] == "patch_does_not_apply"


def test_tau_style_tool_agent_masks_environment_turns_and_takes_the_env_reward(engine):
    from examples.tau_bench import generate_with_tau as ex
    from examples.tau_bench.envs import MockRetailEnv

    args, state, tok = engine

    def template(messages, tokenize=True, add_generation_prompt=True, tools=None):
        parts = []
        for m in messages:
            body = m.get("content") or ""
            for c in m.get("tool_calls", []):
                body += " <tool_call> " + '{"name": "' + c["function"]["name"] + '", "arguments": ' + c["function"]["arguments"].replace(" ", "") + "} </tool_call>"
            parts.append(f"<|{m['role']}|> {body}")
        return tok.encode(" ".join(parts) + (" <|assistant|>" if add_generation_prompt else ""))

    tok.apply_chat_template = template

    def script(prompt):
        if "Order cancelled" in prompt:
            return "It is cancelled . Anything else ?" if "That is all" not in prompt.split("Order cancelled")[-1] else "Goodbye !"
        if "go ahead" in prompt:
            return '<tool_call> {"name": "cancel_order", "arguments": {"order_id":"W100"}} </tool_call>'
        if '"status":' in prompt or "pending" in prompt.split("<|tool|>")[-1]:
            return "Do you confirm the cancellation ?"
        return '<tool_call> {"name": "get_order", "arguments": {"order_id":"W100"}} </tool_call>'

    state["script"] = script
    s = Sample(index=0, prompt="", label='{"env": "mock_retail", "task_index": 0}')
    out = asyncio.run(ex.generate(args, s, {"max_new_tokens": 400, "temperature": 1.0}))
    assert out.status == Sample.Status.COMPLETED and out.reward == 1.0, (out.metadata, out.response)
    assert out.metadata["tool_calls"] == 2 and out.metadata["env_done"]
    assert len(out.loss_mask) == out.response_length == len(out.rollout_log_probs)
    assert 0 < sum(out.loss_mask) < out.response_length  # the model's turns are trained on, the environment's are not
    trained = tok.decode([t for t, m in zip(out.tokens[-out.response_length:], out.loss_mask) if m])
    assert "cancel_order" in trained and "Order cancelled" not in trained and "go ahead" not in trained
    # the environment itself: a delivered order cannot be cancelled, and touching the wrong order loses the reward
    env = MockRetailEnv(0)
    env.reset()
    assert env.step({"name": "cancel_order", "arguments": {"order_id": "W300"}})[0].startswith("Error")
    env.step({"name": "cancel_order", "arguments": {"order_id": "W200"}})
    env.step({"name": "respond", "arguments": {"content": "done"}})
    assert env.step({"name": "respond", "arguments": {"content": "bye"}}) == ("###STOP###", 0.0, True)


def test_message_level_agent_keeps_the_exact_token_trajectory(engine):
    from examples.strands_sglang import generate_with_strands as ex
    from examples.strands_sglang import token_agent as ta

    args, state, tok = engine

    def template(messages, tokenize=True, add_generation_prompt=True, tools=None):
        parts = []
        for m in messages:
            body = m.get("content") or ""
            for c in m.get("tool_calls", []):
                body += " <tool_call> " + '{"name": "' + c["function"]["name"] + '", "arguments": ' + c["function"]["arguments"].replace(" ", "") + "} </tool_call>"
            parts.append(f"<|{m['role']}|> {body}")
        return tok.encode(" ".join(parts) + (" <|assistant|>" if add_generation_prompt else ""))

    tok.apply_chat_template = template
    spec = ex.execute_python_code.tool_spec["function"]
    assert spec["name"] == "execute_python_code" and spec["parameters"]["required"] == ["code"]
    assert spec["parameters"]["properties"]["code"] == {"type": "string"}

    def script(prompt):
        if "<|tool|> 42" in prompt:
            return "So the answer is \\boxed{42}"
        return '<tool_call> {"name": "execute_python_code", "arguments": {"code":"print(6*7)"}} </tool_call>'

    state["script"] = script
    out = asyncio.run(ex.generate(args, Sample(index=0, prompt="What is 6 times 7 ?", label="42"), {"max_new_tokens": 200}))
    assert out.status == Sample.Status.COMPLETED and out.metadata == {"tool_iters": 1, "tool_calls": 1}
    assert len(out.loss_mask) == out.response_length == len(out.rollout_log_probs) == len(out.tokens) - 0 - (len(out.tokens) - out.response_length)
    trained = tok.decode([t for t, m in zip(out.tokens[-out.response_length:], out.loss_mask) if m])
    assert "print(6*7)" in trained and "\\boxed{42}" in trained and "<|tool|>" not in trained
    context = tok.decode([t for t, m in zip(out.tokens[-out.response_length:], out.loss_mask) if not m])
    assert "<|tool|> 42" in context
    assert all(lp == -0.5 for lp, m in zip(out.rollout_log_probs, out.loss_mask) if m) and all(lp == 0.0 for lp, m in zip(out.rollout_log_probs, out.loss_mask) if not m)
    assert tok.decode(out.tokens[: len(out.tokens) - out.response_length]).startswith("<|system|> You are a helpful")
    # the second request carried the first turn's ids unchanged (no re-tokenisation): its prompt extends the first one
    p1, p2 = state["calls"][0][0], state["calls"][1][0]
    assert p2.startswith(p1) and p2[len(p1):].lstrip().startswith("<tool_call>")
    assert asyncio.run(ex.reward_func(args, out)) == 1.0

    # a model that keeps calling the tool is stopped by the limiter and kept as truncated, with a softened penalty
    state["script"] = lambda prompt: '<tool_call> {"name": "execute_python_code", "arguments": {"code":"print(1)"}} </tool_call>'
    args.strands_max_tool_iters = 3
    out = asyncio.run(ex.generate(args, Sample(index=1, prompt="loop", label="7"), {"max_new_tokens": 400}))
    assert out.status == Sample.Status.TRUNCATED and out.metadata["tool_iters"] == 3
    assert sum(out.loss_mask) > 0 and len(out.loss_mask) == out.response_length
    assert asyncio.run(ex.reward_func(args, out)) == pytest.approx(-0.95)
    out.metadata["tool_iters"] = 20
    assert asyncio.run(ex.reward_func(args, out)) == -0.6  # never better than -0.6

    # the token budget is what is left of max_new_tokens after everything appended so far
    state["script"] = script
    state["calls"].clear()
    out = asyncio.run(ex.generate(args, Sample(index=2, prompt="What is 6 times 7 ?", label="42"), {"max_new_tokens": 50}))
    budgets = [c[1]["max_new_tokens"] for c in state["calls"]]
    assert budgets[0] == 50 and budgets[-1] < 50 - 5  # (a retried request may repeat an entry)

    # unknown tools and failing tools come back as observations
    async def bad_tools():
        agent = ta.ToolAgent(ta.TokenTrackingModel(tok, "http://unused", {}), tools=[ex.execute_python_code])
        return await agent._run_tool({"name": "nope", "arguments": {}}), await agent._run_tool({"name": "execute_python_code", "arguments": {"bad": 1}})

    a, b = asyncio.run(bad_tools())
    assert a.startswith("Error: unknown tool") and b.startswith("Error: TypeError")


def test_multi_turn_vision_rollout_collects_images_and_masks_environment_tokens(engine, monkeypatch):
    import torch
    from PIL import Image

    from examples.geo3k_vlm_multi_turn import env_geo3k
    from examples.geo3k_vlm_multi_turn import rollout as ex

    args, state, tok = engine

    def template(messages, tools=None, tokenize=False, add_generation_prompt=True, **kw):
        parts = []
        for m in messages:
            c = m["content"]
            body = c if isinstance(c, str) else " ".join("<image>" if p["type"] == "image" else p["text"] for p in c)
            parts.append(f"<|{m['role']}|> {body}")
        return " ".join(parts) + (" <|assistant|>" if add_generation_prompt else "")

    tok.apply_chat_template = template
    tok.bos_token_id = None

    class FakeProcessor:
        """Expands every <image> word into 4 placeholder tokens and emits one 4 x 4 grid of pixel rows per image."""

        def __call__(self, text, images=None, return_tensors="pt", **kw):
            ids = []
            for w in text.split():
                ids += tok.encode("<image>") * 4 if w == "<image>" else tok.encode(w)
            out = {"input_ids": torch.tensor([ids]), "attention_mask": torch.ones(1, len(ids))}
            if images:
                out["pixel_values"] = torch.cat([torch.full((16, 8), float(im.size[0])) for im in images])
                out["image_grid_thw"] = torch.tensor([[1, 4, 4]] * len(images))
            return out

    monkeypatch.setattr(sglang_rollout, "load_processor", lambda *a, **k: FakeProcessor())
    sglang_rollout.GenerateState.clear_instances()
    args.max_turns, args.rollout_interaction_env_path, args.apply_chat_template = 3, None, True
    args.apply_chat_template_kwargs, args.rollout_max_context_len = None, 400

    replies = iter(['I think <tool_call> {"name":"calc_score","arguments":{"answer":"7"}} </tool_call>',
                    'Then <tool_call> {"name":"calc_score","arguments":{"answer":"12"}} </tool_call>',
                    "So the answer is \\boxed{12}"])
    state["script"] = lambda prompt: next(replies)
    img = Image.new("RGB", (24, 24))
    s = Sample(index=0, prompt="<|user|> <image> What is x ? <|assistant|>", label="12", multimodal_inputs={"images": [img]})
    out = asyncio.run(ex.generate(args, s, {"max_new_tokens": 64, "temperature": 1.0}))
    assert out.status == Sample.Status.COMPLETED
    assert len(out.loss_mask) == out.response_length == len(out.rollout_log_probs)
    trained = tok.decode([t for t, m in zip(out.tokens[-out.response_length:], out.loss_mask) if m])
    context = tok.decode([t for t, m in zip(out.tokens[-out.response_length:], out.loss_mask) if not m])
    assert "calc_score" in trained and "\\boxed{12}" in trained and "does not match" not in trained
    assert "does not match the reference" in context and "matches the reference" in context and "helpful assistant" not in context
    # the first image travelled with every call; its processor outputs reach the trainer; the prompt's placeholders are expanded
    assert all(len(c) == 2 for c in state["calls"]) and len(state["calls"]) == 3
    assert out.tokens.count(tok.encode("<image>")[0]) == 4
    assert out.multimodal_train_inputs["pixel_values"].shape == (16, 8) and out.multimodal_train_inputs["image_grid_thw"].tolist() == [[1, 4, 4]]
    # budget = context limit minus what is there: it shrinks from call to call
    budgets = [c[1]["max_new_tokens"] for c in state["calls"]]
    assert budgets[0] == 400 - (len(out.tokens) - out.response_length) and budgets[0] > budgets[1] > budgets[2]

    # the environment by itself
    env = env_geo3k.Geo3kEnv("12", max_turns=3)
    obs, done, info = env.step('<tool_call>{"name": "calc_score", "arguments": {"answer": "\\\\boxed{12}"}}</tool_call>')
    assert obs["tool_score"] == 1.0 and not done and info["tool_executed"]
    obs, done, info = env.step('<tool_call>{"function": {"name": "calc_geo3k_reward", "arguments": "{\\"answer\\": \\"5\\"}"}}</tool_call>')
    assert obs["tool_score"] == 0.0 and "one chance left" in obs["obs_str"] and not done
    obs, done, info = env.step('<tool_call>{"name": "other", "arguments": {}}</tool_call>')
    assert "not supported" in obs["obs_str"] and done  # third of three turns
    assert env.step("no call here")[1] is True and env_geo3k.parse_tool_call("<tool_call>{broken</tool_call>") is None
    msg = env.format_observation({"obs_str": "look", "multi_modal_data": {"image": [img]}})
    assert [p["type"] for p in msg["content"]] == ["image", "text"]
    ids, image_data, images, train = ex.encode_observation(tok, FakeProcessor(), msg, None, True, None)
    assert tok.decode(ids).startswith("<|user|> <image> <image> <image> <image> look") and len(image_data) == 1 and train["pixel_values"].shape[0] == 16


def test_token_delta_survives_templates_that_rewrite_history():
    import re

    from examples.tau_bench.token_delta import get_context_delta, get_token_delta

    class Tok:
        """Byte-level tokenizer whose template hides the reasoning of assistant turns that precede the last user turn."""

        def apply_chat_template(self, messages, *, add_generation_prompt, tokenize):
            assert tokenize is False
            last_user = max((i for i, m in enumerate(messages) if m["role"] == "user"), default=-1)
            out = []
            for i, m in enumerate(messages):
                c = re.sub(r"<think>.*?</think>", "", m["content"], flags=re.DOTALL) if m["role"] == "assistant" and i < last_user else m["content"]
                out.append(f"<{m['role']}>{c}</{m['role']}>")
            return "".join(out) + ("<assistant>" if add_generation_prompt else "")

        def encode(self, text, *, add_special_tokens):
            return list(text.encode())

        def decode(self, ids):
            return bytes(ids).decode()

    class Merging(Tok):
        """'>' followed by a newline is one token: the end of the generation prompt merges with the answer's first byte."""

        def encode(self, text, *, add_special_tokens):
            raw, out, i = text.encode(), [], 0
            while i < len(raw):
                if raw[i : i + 2] == b">\n":
                    out.append(1000)
                    i += 2
                else:
                    out.append(raw[i])
                    i += 1
            return out

    tok = Tok()
    first = [{"role": "user", "content": "first user"}, {"role": "assistant", "content": "<think>first reasoning</think>first answer"}]
    ids, mask = get_token_delta(tok, first + [{"role": "user", "content": "second user must remain complete"}])
    assert tok.decode(ids) == "<user>second user must remain complete</user>" and mask == [0] * len(ids)
    ids, mask = get_token_delta(tok, [{"role": "user", "content": "q"}, {"role": "assistant", "content": "<think>r</think>a"}])
    assert tok.decode(ids) == "<think>r</think>a</assistant>" and mask == [1] * len(ids)
    assert tok.decode(get_context_delta(tok, first + [{"role": "user", "content": "again"}])) == "<user>again</user><assistant>"
    # six turns accumulated message by message: every user span is context, every answer is trained on, every
    # generation prompt is context
    messages = [{"role": "user", "content": "user 1"}]
    ids = tok.encode(tok.apply_chat_template(messages, add_generation_prompt=True, tokenize=False), add_special_tokens=False)
    mask = [0] * len(ids)
    for turn in range(1, 7):
        messages.append({"role": "assistant", "content": f"<think>reasoning {turn}</think>answer {turn}"})
        d, m = get_token_delta(tok, messages, include_generation_prompt=turn > 1)
        ids, mask = ids + d, mask + m
        if turn < 6:
            messages.append({"role": "user", "content": f"user {turn + 1}"})
            d, m = get_token_delta(tok, messages)
            ids, mask = ids + d, mask + m
    text = tok.decode(ids)
    assert text.count("<assistant>") == 6 == text.count("</assistant>")
    for turn in range(1, 7):
        span = f"<user>user {turn}</user>"
        at = text.index(span)
        assert mask[at : at + len(span)] == [0] * len(span)
        span = f"<think>reasoning {turn}</think>answer {turn}</assistant>"
        at = text.index(span)
        assert mask[at : at + len(span)] == [1] * len(span)
        prompt_at = text.rfind("<assistant>", 0, at)
        assert mask[prompt_at:at] == [0] * (at - prompt_at)
    # a token that spans the end of the generation prompt and the start of the answer is kept whole and masked with the prompt
    mt = Merging()
    ids, mask = get_token_delta(mt, first + [{"role": "user", "content": "second user"}, {"role": "assistant", "content": "\nsecond answer"}],
                                include_generation_prompt=True)  # fmt: skip
    want = mt.encode("<assistant>\nsecond answer</assistant>", add_special_tokens=False)
    n = len(mt.encode("<assistant>", add_special_tokens=False))
    assert ids == want and 1000 in ids and mask == [0] * n + [1] * (len(want) - n)
    with pytest.raises(ValueError, match="empty conversation"):
        get_token_delta(tok, [])
