"""Rollout buffer service, the math generator and the trainer-side rollout function, wired over real HTTP on localhost."""

import asyncio
import json
import time
from argparse import Namespace

import pytest
import requests

from slime_b200.agent.aiohttp_threaded import serve_in_thread
from slime_b200.plugins.rollout_buffer import buffer as rb
from slime_b200.plugins.rollout_buffer import rollout_buffer_example as ex
from slime_b200.plugins.rollout_buffer.generator import base_generator as bg


def _traj(iid, reward, content="x", ts=None):
    return {"uid": f"u{iid}-{reward}", "instance_id": iid, "messages": [{"role": "user", "content": "q"},
            {"role": "assistant", "content": content}], "reward": reward, "extra_info": {"timestamp": str(ts or time.time())}}


def test_buffer_groups_and_meta():
    buf = rb.RolloutBuffer(group_size=2, is_valid_group_func=bg.is_valid_group)
    assert buf.read() == {"data": [], "meta_info": {}}
    buf.write(_traj(1, 1.0))
    buf.write(_traj(2, 0.0))
    assert len(buf) == 0
    buf.write(_traj(1, 0.0))
    buf.write(_traj(2, 1.0, content="  "))  # group 2 complete but one answer is blank -> not valid
    assert len(buf) == 2
    out = buf.read()
    assert [t["instance_id"] for t in out["data"]] == [1, 1]
    assert out["meta_info"]["total_samples"] == 4 and out["meta_info"]["num_groups"] == 2
    assert out["meta_info"]["avg_reward"] == 0.5
    assert buf.stats() == {"written": 4, "read": 2, "pending_groups": 1, "ready_samples": 0}


def test_normalize_group_data():
    _, items = bg.normalize_group_data((7, [{"reward": 1.0}, {"reward": 0.0}, {"reward": -2.0}]))
    assert items[0]["reward"] == pytest.approx(1.0, abs=1e-6) and items[1]["reward"] == pytest.approx(-1.0, abs=1e-6)
    assert items[2]["reward"] == -2.0 and [i["raw_reward"] for i in items] == [1.0, 0.0, -2.0]
    _, same = bg.normalize_group_data((8, [{"reward": 1.0}, {"reward": 1.0}]))
    assert [i["reward"] for i in same] == [0.0, 0.0]
    _, zeros = bg.normalize_group_data((9, [{"reward": 0.0}, {"reward": 0.0}]))
    assert [i["reward"] for i in zeros] == [0.0, 0.0]


def test_select_newest_groups():
    rows = [_traj(1, 0, ts=10), _traj(1, 0, ts=50), _traj(2, 0, ts=40), _traj(3, 0, ts=60)]
    picked = ex.select_rollout_data(Namespace(n_samples_per_prompt=1), rows, 2)
    assert [g[0]["instance_id"] for g in picked] == [3, 1] and len(picked[1]) == 2


def test_query_single_turn_resumes_after_abort(monkeypatch):
    monkeypatch.setattr(bg, "ABORT_BACKOFF_SEC", 0.0)
    calls = []

    class Client:
        def chat(self, **req):
            calls.append(req)
            if len(calls) == 1:
                return {"choices": [{"finish_reason": "abort", "message": {"content": "The ans"}}], "usage": {"completion_tokens": 3}}
            return {"choices": [{"finish_reason": "stop", "message": {"content": "wer is 4"}}], "usage": {"completion_tokens": 4}}

    msgs, finish = bg.query_single_turn(Client(), [{"role": "user", "content": "2+2?"}], {"max_tokens": 10})
    assert finish == "stop" and msgs[-1] == {"role": "assistant", "content": "The answer is 4"}
    assert calls[1]["max_tokens"] == 7 and calls[1]["extra_body"] == {"continue_final_message": True}
    assert calls[1]["messages"][-1] == {"role": "assistant", "content": "The ans"}


def test_end_to_end_over_http(tmp_path, monkeypatch):
    from aiohttp import web

    # a chat server that always answers \boxed{4}
    async def chat(request):
        body = await request.json()
        assert body["messages"][-1]["role"] == "user" and body["max_tokens"] == 16
        return web.json_response({"choices": [{"finish_reason": "stop", "message": {"role": "assistant", "content": "hm </think> so \\boxed{4}"}}],
                                  "usage": {"completion_tokens": 3}})

    engine_app = web.Application()
    engine_app.router.add_post("/v1/chat/completions", chat)
    engine = serve_in_thread(engine_app, host="127.0.0.1")
    service = rb.BufferService()
    buf = serve_in_thread(rb.build_app(service), host="127.0.0.1")
    prompts = tmp_path / "p.jsonl"
    prompts.write_text("".join(json.dumps({"prompt": [{"role": "user", "content": f"what is {i}+{4 - i}?"}], "label": "4"}) + "\n"
                               for i in range(3)))
    try:
        host, port = "127.0.0.1", engine.port
        args = Namespace(rollout_buffer_url=buf.url, rollout_task_type="math", prompt_data=str(prompts), num_epoch=1,
                         sglang_router_ip=host, sglang_router_port=port, n_samples_per_prompt=2, rollout_batch_size=2,
                         rollout_max_response_len=16, rollout_temperature=1.0, rollout_top_p=1.0, hf_checkpoint="tok",
                         fetch_trajectory_retry_times=3, loss_mask_type="qwen", use_wandb=False, use_tensorboard=False,
                         global_batch_size=4)
        orig = rb.BufferService.start_rollout

        def quick(self, payload):  # no start-up delay, one pass over the prompts
            return orig(self, {**payload, "startup_delay_sec": 0, "num_repeats": 1, "num_process": 4})

        monkeypatch.setattr(rb.BufferService, "start_rollout", quick)
        monkeypatch.setattr(ex, "POLL_SEC", 0.05)
        from test_mask_utils import ChatMLTokenizer

        monkeypatch.setattr(ex, "_tokenizer", lambda a: ChatMLTokenizer())
        ex._state["started"] = False

        class DataBuffer:
            def __init__(self):
                self.groups, self.meta = [], {}

            def get_metadata(self):
                return self.meta

            def update_metadata(self, m):
                self.meta.update(m)

            def get_buffer_length(self):
                return sum(len(g) for g in self.groups)

            def add_samples(self, groups):
                self.groups += groups

            def get_samples(self, n):
                out, self.groups = self.groups[:n], self.groups[n:]
                return out

        db = DataBuffer()
        groups = asyncio.run(ex.generate_rollout_async(args, 0, db))
        assert len(groups) == 2 and all(len(g) == 2 for g in groups)
        s = groups[0][0]
        assert s.reward == 1 and s.response_length > 0 and len(s.loss_mask) == s.response_length and sum(s.loss_mask) > 0
        assert s.status.name == "COMPLETED" and s.metadata["finish_reason"] == "stop" and "0" in db.meta
        assert requests.get(buf.url + "/stats", timeout=5).json()["written"] >= 4
        r = requests.post(buf.url + "/start_rollout", json={"task_type": "nope", "num_repeat_per_sample": 1}, timeout=5)
        assert r.status_code == 400 and "no generator" in r.json()["message"]
    finally:
        engine.stop()
        buf.stop()
