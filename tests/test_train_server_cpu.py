"""The trainer-as-a-service scorer on CPU: packing, label / sample outputs, HTTP contract, OPD post-processing."""

import asyncio

import pytest
import torch

from slime_b200.backends.train.server import LogprobService, build_app, normalize_label_token_ids, parse_sample_n


def _toy_forward(vocab=17):
    torch.manual_seed(0)
    table = torch.randn(vocab, vocab)

    def forward(ids, cu, max_len):  # logits at position t depend only on token t: easy to verify
        return table[ids]

    return forward, table


def test_service_scores_packs_and_matches_reference():
    fwd, table = _toy_forward()
    svc = LogprobService(fwd, max_tokens=12, device="cpu")
    try:
        seqs = [[1, 2, 3, 4, 5], [6, 7], [8], [9, 10, 11, 12, 13, 14, 15, 16]]
        reqs = [svc.submit(s, sample_n=2 if i == 0 else 0, label_token_ids=[[0, 1]] * (len(s) - 1) if i == 1 else None)
                for i, s in enumerate(seqs)]  # fmt: skip
        for r in reqs:
            assert r.done.wait(10) and r.error is None
        for s, r in zip(seqs, reqs):
            t = torch.tensor(s)
            ref = torch.log_softmax(table[t[:-1]], -1).gather(1, t[1:, None]).squeeze(1)
            assert torch.allclose(torch.tensor(r.result["log_probs"]), ref, atol=1e-5)
        assert len(reqs[0].result["sampled_token_ids"]) == 4 and len(reqs[0].result["sampled_token_ids"][0]) == 2
        lab = torch.tensor(reqs[1].result["label_token_log_probs"])
        assert torch.allclose(lab, torch.log_softmax(table[torch.tensor([6])], -1)[:, :2], atol=1e-5)
        assert reqs[2].result["log_probs"] == []
        assert svc.loads()["served"] == 4 and svc.wait_idle(1.0)
    finally:
        svc.stop()


def test_argument_normalisation():
    assert parse_sample_n(None) == 0 and parse_sample_n("3") == 3
    with pytest.raises(ValueError):
        parse_sample_n(-1)
    assert normalize_label_token_ids([1, 2], 2) == [[1], [2]]
    with pytest.raises(ValueError):
        normalize_label_token_ids([[1], [2, 3]], 2)
    with pytest.raises(ValueError):
        normalize_label_token_ids([[1]], 2)


def test_http_contract_and_opd_post_processing():
    from aiohttp.test_utils import TestClient, TestServer

    from slime_b200.rollout.on_policy_distillation import post_process_rewards
    from slime_b200.utils.arguments import namespace_from_dict
    from slime_b200.utils.types import Sample

    fwd, table = _toy_forward()
    svc = LogprobService(fwd, device="cpu")
    reloaded = []

    async def run():
        app = build_app(svc, {"model": "toy"}, update_from_disk=reloaded.append, max_request_length=16)
        async with TestClient(TestServer(app)) as c:
            assert (await (await c.get("/detect")).json())["server_type"] == "slime_b200_train_server"
            assert (await c.post("/generate", json={})).status == 400
            assert (await c.post("/generate", json={"input_ids": list(range(17))})).status == 413
            r = await c.post("/generate", json={"input_ids": [3, 1, 4, 1, 5]})
            body = await r.json()
            assert r.status == 200 and len(body["log_probs"]) == 4
            assert body["meta_info"]["input_token_logprobs"][0] == [None, 3]
            r2 = await c.post("/update_weights_from_disk", json={"model_path": "/tmp/x"})
            assert r2.status == 200 and reloaded == ["/tmp/x"]
            assert (await (await c.get("/get_loads")).json())["queue_size"] == 0
            return body

    try:
        body = asyncio.run(run())
    finally:
        svc.stop()
    # the response plugs straight into the on-policy-distillation reward post-processing
    s = Sample(index=0, tokens=[3, 1, 4, 1, 5], response_length=2, reward=body)
    post_process_rewards(namespace_from_dict(dict(rollout_batch_size=1, num_rollout=1)), [s])
    assert torch.allclose(s.teacher_log_probs, torch.tensor(body["log_probs"][-2:]))
