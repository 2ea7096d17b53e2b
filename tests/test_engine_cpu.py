"""Rollout engine on CPU (fp32 reference ops): scheduling, prefix cache, stop conditions, control plane."""

import numpy as np
import pytest
import torch

from slime_b200.engine.engine import Engine
from slime_b200.engine.kv_cache import PageAllocator
from slime_b200.engine.server_args import ServerArgs
from slime_b200.models.config import get_preset


def make_engine(pages=96, max_running=8, **kw):
    cfg = get_preset("tiny")
    e = Engine(cfg, ServerArgs(page_size=4, max_running_requests=max_running, context_length=128, disable_cuda_graph=True, **kw),
               device="cpu", num_pages=pages)  # fmt: skip
    e.weights.init_random(0)
    return e


def teacher_forced(e, ids, n_prompt):
    rq = e.generate([ids], [dict(max_new_tokens=0)], logprob_start_len=0)[0]
    return np.array(rq.input_logprobs[n_prompt:])


def test_decode_logprobs_match_teacher_forcing_and_prefix_cache():
    e = make_engine()
    p = [1, 2, 3, 4, 5, 6, 7, 8, 9, 10]
    reqs = e.generate([p] * 4 + [[5, 4, 3, 2, 1, 9, 9, 9, 9]], [dict(max_new_tokens=6 + i, ignore_eos=True) for i in range(5)])
    for i, r in enumerate(reqs):
        assert len(r.output_ids) == 6 + i and r.finish_reason["type"] == "length"
        ref = teacher_forced(e, r.input_ids + r.output_ids, len(r.input_ids))
        assert np.abs(ref - np.array(r.output_logprobs)).max() < 1e-5
    assert [r.num_cached_tokens for r in reqs[:4]] == [0, 8, 8, 8]  # siblings reuse the first request's full pages
    assert e.kv.allocator.stats()["hit_rate"] > 0
    assert not e.has_work() and all(s is None for s in e.slot_req)


def test_same_seed_reproduces_and_different_seed_differs():
    e = make_engine()
    p = [3, 1, 4, 1, 5, 9, 2, 6]
    a, b, c = e.generate([p, p, p], [dict(max_new_tokens=12, ignore_eos=True, sampling_seed=s) for s in (7, 7, 8)])
    assert a.output_ids == b.output_ids
    assert a.output_ids != c.output_ids


def test_eos_and_stop_token_finish_and_discard_overshoot():
    e = make_engine()
    p = [1, 2, 3, 4, 5]
    base = e.generate([p], [dict(max_new_tokens=20, ignore_eos=True, sampling_seed=1)])[0]
    stop_tok = base.output_ids[6]
    first = base.output_ids.index(stop_tok)
    r = e.generate([p], [dict(max_new_tokens=20, ignore_eos=True, sampling_seed=1, stop_token_ids=[stop_tok])])[0]
    assert r.output_ids == base.output_ids[: first + 1]
    assert r.finish_reason == {"type": "stop", "matched": stop_tok}
    e.eos_ids = {stop_tok}
    r2 = e.generate([p], [dict(max_new_tokens=20, sampling_seed=1)])[0]
    assert r2.output_ids == base.output_ids[: first + 1] and r2.finish_reason["type"] == "stop"
    r3 = e.generate([p], [dict(max_new_tokens=20, sampling_seed=1, min_new_tokens=first + 2)])[0]
    assert len(r3.output_ids) > first + 1


def test_abort_pause_flush_and_memory_tags():
    e = make_engine()
    r = e.add_request([1, 2, 3], dict(max_new_tokens=50, ignore_eos=True))
    for _ in range(5):
        e.step()
    assert not e.flush_cache()  # busy
    assert e.abort(r.rid) == 1
    assert r.finish_reason == {"type": "abort"} and 0 < len(r.output_ids) < 50
    assert len(r.output_logprobs) == len(r.output_ids)
    assert e.flush_cache()
    e.pause_generation()
    r2 = e.add_request([1, 2, 3], dict(max_new_tokens=3, ignore_eos=True))
    assert e.step() == [] and not r2.finished()
    e.continue_generation()
    while e.has_work():
        e.step()
    assert r2.finished()
    free_before = e.kv.allocator.available()
    e.release_memory_occupation(["kv_cache"])
    e.release_memory_occupation(["kv_cache"])  # idempotent
    assert e.step() == []
    e.resume_memory_occupation(["kv_cache"])
    assert e.kv.allocator.available() >= free_before - 1
    e.release_memory_occupation(["weights"])
    e.resume_memory_occupation(["weights"])
    e.weights.init_random(0)
    assert e.generate([[1, 2, 3]], [dict(max_new_tokens=2, ignore_eos=True)])[0].finished()


def test_retraction_when_cache_is_exhausted_keeps_outputs_consistent():
    e = make_engine(pages=14, max_running=4)  # 13 usable pages of 4 tokens
    prompts = [[i + 1] * 6 for i in range(4)]
    reqs = e.generate(prompts, [dict(max_new_tokens=24, ignore_eos=True, sampling_seed=i) for i in range(4)])
    assert all(len(r.output_ids) == 24 for r in reqs)
    big = make_engine(pages=200, max_running=4)
    ref = big.generate(prompts, [dict(max_new_tokens=24, ignore_eos=True, sampling_seed=i) for i in range(4)])
    for a, b in zip(reqs, ref):
        assert a.output_ids == b.output_ids  # re-prefill after retraction continues the same sequence
        assert np.abs(np.array(a.output_logprobs) - np.array(b.output_logprobs)).max() < 1e-4


def test_update_weights_changes_outputs_and_version():
    e = make_engine()
    p = [2, 7, 1, 8]
    a = e.generate([p], [dict(max_new_tokens=8, ignore_eos=True, sampling_seed=3)])[0]
    named = [("model.layers.0.mlp.down_proj.weight", torch.randn(128, 256) * 0.5)]
    assert e.update_weights(named, version="7") == []
    assert e.get_weight_version() == "7"
    b = e.generate([p], [dict(max_new_tokens=8, ignore_eos=True, sampling_seed=3)])[0]
    assert b.weight_version == "7" and b.num_cached_tokens == 0  # the prefix cache was flushed with the update
    assert a.output_logprobs != b.output_logprobs
    assert e.update_weights([("model.layers.0.nonexistent.weight", torch.zeros(1))]) == ["model.layers.0.nonexistent.weight"]


def test_top_p_returns_kept_sets_and_renormalised_logprobs():
    e = make_engine()
    sp = dict(max_new_tokens=5, ignore_eos=True, top_p=0.3, top_k=20, custom_params={"return_top_p_token_ids": True})
    r = e.generate([[1, 2, 3, 4]], [sp])[0]
    assert len(r.kept_offsets) == len(r.output_ids) + 1 and r.kept_offsets[-1] == len(r.kept_ids)
    for i, tok in enumerate(r.output_ids):
        kept = r.kept_ids[r.kept_offsets[i] : r.kept_offsets[i + 1]]
        assert tok in kept and len(kept) <= 20
    m = e.meta_info(r)
    from slime_b200.utils.misc import decode_int32_meta_array

    assert decode_int32_meta_array(m, "top_p_token_offsets").tolist() == r.kept_offsets
    plain = teacher_forced(e, r.input_ids + r.output_ids, 4)
    assert all(lp >= ref - 1e-5 for lp, ref in zip(r.output_logprobs, plain))  # renormalising can only raise log-probs


def test_page_allocator_prefix_index_and_lru():
    a = PageAllocator(8, 4)
    toks = list(range(13))
    pages = a.alloc(4)
    parent = b""
    for i in range(3):
        parent = a.commit(pages[i], parent, toks[i * 4 : (i + 1) * 4])
    a.release(pages)
    assert a.available() == 8 and len(a.lru) == 3
    got, _ = a.match_prefix(toks)
    assert got == pages[:3]
    a.release(got)
    taken = a.alloc(8)  # evicts the cached pages in LRU order
    assert len(set(taken)) == 8 and not a.index
    with pytest.raises(Exception):
        a.alloc(1)


def test_openai_compatible_endpoints():
    """/v1/chat/completions, /v1/completions and /v1/models on the CPU engine with a word-level tokenizer."""
    import requests

    from slime_b200.engine.http_server import EngineServer

    class Tok:
        def encode(self, text, add_special_tokens=False):
            return [3 + (sum(map(ord, w)) % 500) for w in text.split()]

        def decode(self, ids, skip_special_tokens=True):
            return " ".join(f"w{i}" for i in ids)

        def apply_chat_template(self, messages, tokenize=False, add_generation_prompt=True, **kw):
            text = " ".join(f"<{m['role']}> {m['content']} </s>" for m in messages)
            return text + (" <assistant> " if add_generation_prompt else "")

    e = make_engine()
    tok = Tok()
    srv = EngineServer(e, "127.0.0.1", 0, tok).start(block=False)
    try:
        url = f"http://127.0.0.1:{srv.port}"
        msgs = [{"role": "user", "content": "what is two plus two"}]
        r = requests.post(url + "/v1/chat/completions", json={"messages": msgs, "max_tokens": 5, "temperature": 0}, timeout=60).json()
        ch = r["choices"][0]
        assert r["object"] == "chat.completion" and ch["message"]["role"] == "assistant" and ch["finish_reason"] == "length"
        assert r["usage"]["completion_tokens"] == 5 and len(ch["message"]["content"].split()) == 5
        # resuming a partial answer feeds template(prompt) + partial text, so greedy decoding continues the same sequence
        head = " ".join(ch["message"]["content"].split()[:2])
        prompt_ids = tok.encode(tok.apply_chat_template(msgs))
        full = requests.post(url + "/v1/completions", json={"prompt": prompt_ids, "max_tokens": 5, "temperature": 0}, timeout=60).json()
        assert full["choices"][0]["token_ids"] == [int(w[1:]) for w in ch["message"]["content"].split()]
        r2 = requests.post(url + "/v1/chat/completions", timeout=60,
                           json={"messages": msgs + [{"role": "assistant", "content": head}], "max_tokens": 3,
                                 "temperature": 0, "continue_final_message": True}).json()
        assert r2["usage"]["prompt_tokens"] == len(prompt_ids) + 2
        assert requests.get(url + "/v1/models", timeout=10).json()["data"][0]["object"] == "model"
        assert requests.post(url + "/v1/chat/completions", json={}, timeout=10).status_code == 400
    finally:
        srv.shutdown()


@pytest.mark.parametrize("moe,family", [(False, None), (True, None), (False, "glm4"), (False, "minimax_m2"), (False, "deepseek_v3"),
                                        (False, "qwen3_next"), (False, "mtp_moe")],
                         ids=["dense", "moe_ep2", "glm4", "minimax_m2_ep2", "deepseek_v3_ep2", "qwen3_next", "speculative_moe_ep2"])  # fmt: skip
def test_tensor_parallel_engine_on_gloo_matches_single_rank(moe, family):
    """Two gloo ranks: TP weight slicing, row-parallel reductions and the vocab-parallel logits gather (host logic);
    with ``moe`` also experts sharded over the two ranks (each rank serves its own experts' routes, outputs summed)."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, ENGINE_TP_CHECK_DEVICE="cpu", MASTER_ADDR="127.0.0.1", ENGINE_TP_CHECK_MOE=str(int(moe)))
    if family:
        env["ENGINE_TP_CHECK_FAMILY"] = family
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                        "127.0.0.1", "--master-port", str(29671 + int(moe) + {None: 0, "glm4": 2, "minimax_m2": 3, "deepseek_v3": 4, "qwen3_next": 5, "mtp_moe": 6}[family]), os.path.join(root, "tests/multigpu/engine_tp_check.py")],
                       env=env, cwd=root, capture_output=True, text=True, timeout=280)  # fmt: skip
    assert r.returncode == 0 and "RESULT ok world=2" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def make_moe_engine(**kw):
    cfg = get_preset("tiny-moe")
    e = Engine(cfg, ServerArgs(page_size=4, max_running_requests=8, context_length=128, disable_cuda_graph=True, **kw),
               device="cpu", num_pages=96)  # fmt: skip
    e.weights.init_random(0, std=0.2)
    return e


def test_moe_engine_returns_routed_experts_for_every_fed_token():
    e = make_moe_engine(enable_return_routed_experts=True)
    cfg = e.cfg
    p = [1, 2, 3, 4, 5, 6, 7, 8, 9]
    a, b = e.generate([p, p[:5]], [dict(max_new_tokens=6, ignore_eos=True, sampling_seed=3)] * 2, return_routed_experts=True)
    for r in (a, b):
        routed = torch.cat(r.routed_experts)
        n = len(r.input_ids) + len(r.output_ids) - 1  # the last sampled token is never fed to the model
        assert routed.shape == (n, cfg.num_layers, cfg.moe_router_topk) and routed.dtype == torch.int32
        assert int(routed.min()) >= 0 and int(routed.max()) < cfg.num_experts
        # teacher forcing over the same tokens takes the same routes
        again = e.generate([r.input_ids + r.output_ids], [dict(max_new_tokens=0)], logprob_start_len=0, return_routed_experts=True)[0]
        assert torch.equal(torch.cat(again.routed_experts)[:n], routed)
        meta = e.meta_info(r)
        from slime_b200.utils.misc import decode_int32_meta_array

        assert decode_int32_meta_array(meta, "routed_experts").reshape(n, cfg.num_layers, -1).tolist() == routed.tolist()
    # a request that does not ask for them gets none, and an engine that does not record keeps the prefix cache
    c = e.generate([p], [dict(max_new_tokens=2, ignore_eos=True)])[0]
    assert c.routed_experts == [] and "routed_experts" not in e.meta_info(c)


def test_device_layout_skips_routes_of_other_ranks():
    from slime_b200.ops import grouped

    torch.manual_seed(0)
    T, k, E, H = 37, 2, 8, 16
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(T)])
    x, probs = torch.randn(T, H), torch.rand(T, k)
    w = torch.randn(E, H, H)
    full = grouped.DeviceLayout(idx, E)
    ref = full.combine(grouped.grouped_gemm(full.pad(x), w, full), probs, T)
    parts = []
    for r in range(4):  # four expert-parallel ranks, two experts each: their partial outputs add up to the full result
        lay = grouped.DeviceLayout(idx, E // 4, first_expert=r * 2)
        assert int((lay.slot_dest >= 0).sum()) == int(((idx >= r * 2) & (idx < r * 2 + 2)).sum())
        parts.append(lay.combine(grouped.grouped_gemm(lay.pad(x), w[r * 2 : r * 2 + 2], lay), probs, T))
    assert torch.allclose(sum(parts), ref, atol=1e-5)


def test_prefill_decode_disaggregation_hands_the_kv_over():
    """A prefill-only engine exports the prompt's KV and the first token; a second engine adopts both and decodes the
    same continuation, with the same log-probs, as one engine doing everything."""
    whole, pre, dec = make_engine(), make_engine(), make_engine()
    prompts = [[1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11], [5, 4, 3]]
    sp = dict(max_new_tokens=9, ignore_eos=True, sampling_seed=5)
    ref = whole.generate(prompts, [dict(sp)] * 2)
    staged = pre.generate(prompts, [dict(sp)] * 2, prefill_only=True)
    assert [r.finish_reason["type"] for r in staged] == ["prefill_done"] * 2 and all(len(r.output_ids) == 1 for r in staged)
    assert staged[0].kv_export[0].shape == (pre.cfg.num_layers, 11, pre.weights.hkv, pre.cfg.head_dim)
    assert not pre.has_work() and pre.kv.allocator.available() == whole.kv.allocator.available()  # pages went back
    adopted = [dec.import_request(r.input_ids, r.output_ids[0], r.output_logprobs[0], r.kv_export, dict(sp)) for r in staged]
    while dec.has_work():
        dec.step()
    for a, b in zip(adopted, ref):
        assert a.output_ids == b.output_ids and a.finish_reason == b.finish_reason
        assert np.abs(np.array(a.output_logprobs) - np.array(b.output_logprobs)).max() < 1e-5
    assert dec.stats["prefill_tokens"] == 0 and dec.stats["imported_tokens"] == 14
    with pytest.raises(ValueError, match="does not fit"):
        dec.import_request([1, 2], 3, 0.0, staged[0].kv_export, dict(sp))


def test_router_runs_prefill_and_decode_on_different_servers():
    """Router + one prefill server + one decode server over HTTP: the decode server pulls the prompt's KV from the
    prefill server and returns what a single server returns; its own prefill counter stays at zero."""
    import requests

    from slime_b200.engine.http_server import EngineServer
    from slime_b200.engine.router import Router
    from slime_b200.utils.misc import get_free_port

    engines = [make_engine() for _ in range(3)]
    servers = [EngineServer(e, "127.0.0.1", get_free_port(start_port=31200 + 17 * i)).start(block=False) for i, e in enumerate(engines)]
    router = Router("127.0.0.1", get_free_port(start_port=31300), policy="round_robin").start(block=False)
    try:
        urls = [f"http://127.0.0.1:{s.port}" for s in servers]
        router.add_worker(urls[0], "prefill")
        router.add_worker(urls[1], "decode")
        body = {"input_ids": [1, 2, 3, 4, 5, 6, 7, 8, 9], "return_logprob": True,
                "sampling_params": {"max_new_tokens": 7, "ignore_eos": True, "sampling_seed": 3}}  # fmt: skip
        via = requests.post(f"http://127.0.0.1:{router.port}/generate", json=body, timeout=120)
        assert via.status_code == 200, via.text
        via = via.json()
        ref = requests.post(urls[2] + "/generate", json=body, timeout=120).json()
        assert via["output_ids"] == ref["output_ids"] and via["meta_info"]["finish_reason"] == ref["meta_info"]["finish_reason"]
        a = [x[0] for x in via["meta_info"]["output_token_logprobs"]]
        b = [x[0] for x in ref["meta_info"]["output_token_logprobs"]]
        assert np.abs(np.array(a) - np.array(b)).max() < 1e-5
        assert engines[1].stats["prefill_tokens"] == 0 and engines[1].stats["imported_tokens"] == 9
        assert engines[0].stats["prefill_tokens"] == 9 and engines[0].stats["decode_tokens"] == 0
        assert not servers[0].kv_store  # served once, then dropped
        assert via["meta_info"]["pd_transfer_total_mb"] > 0 and via["meta_info"]["pd_transfer_speed_gb_s"] > 0
        assert "pd_transfer_total_mb" not in ref["meta_info"]
        # a request that ends with its first token never reaches the decode server
        one = requests.post(f"http://127.0.0.1:{router.port}/generate", timeout=120,
                            json=dict(body, sampling_params=dict(body["sampling_params"], max_new_tokens=1))).json()
        assert one["output_ids"] == ref["output_ids"][:1] and engines[1].stats["imported_tokens"] == 9
    finally:
        router.shutdown()
        for s in servers:
            s.shutdown()


def test_evicted_prefix_pages_come_back_from_the_host_tier():
    """Few device pages, a host tier behind them: a prompt whose pages were pushed out by other traffic is served from
    the host copy (same tokens and log-probs as a cold run), counted as cached tokens; without the tier it is recomputed."""
    from slime_b200.engine.kv_cache import HostKVTier

    cfg = get_preset("tiny")
    mk = lambda **kw: Engine(cfg, ServerArgs(page_size=4, max_running_requests=2, context_length=128, disable_cuda_graph=True, **kw),
                             device="cpu", num_pages=24)  # noqa: E731
    plain, tiered = mk(), mk(enable_hierarchical_cache=True, hicache_ratio=4.0)
    for e in (plain, tiered):
        e.weights.init_random(0, std=0.2)
    tier = tiered.kv.allocator.host_tier
    assert isinstance(tier, HostKVTier) and tier.num_pages == 96 and plain.kv.allocator.host_tier is None
    sp = dict(max_new_tokens=4, temperature=0, ignore_eos=True)
    first = list(range(1, 42))
    others = [[100 + 50 * j + i for i in range(41)] for j in range(4)]
    ref = plain.generate([first], [sp])[0]
    for e in (plain, tiered):
        e.generate([first], [sp])
        for o in others:  # enough traffic to evict every page of the first prompt
            e.generate([o], [sp])
    assert tiered.kv.allocator.stats()["host_stores"] >= 10
    again_plain, again = plain.generate([first], [sp])[0], tiered.generate([first], [sp])[0]
    assert again_plain.num_cached_tokens == 0  # gone without the tier
    assert again.num_cached_tokens == 40 and tiered.kv.allocator.stats()["host_hits"] == 10
    assert again.output_ids == ref.output_ids and np.abs(np.array(again.output_logprobs) - np.array(ref.output_logprobs)).max() < 1e-5
    # a weight update makes host copies stale too; releasing the cache keeps the host pool unless asked otherwise
    tiered.update_weights([], flush_cache=True)
    assert tiered.kv.allocator.stats()["host_cached"] == 0
    tiered.generate([first], [sp])
    for o in others:
        tiered.generate([o], [sp])
    assert tiered.kv.allocator.stats()["host_cached"] > 0
    tiered.release_memory_occupation(["kv_cache"])
    tiered.resume_memory_occupation(["kv_cache"])
    assert tiered.kv.allocator.host_tier is tier and tier.k is not None
    back = tiered.generate([first], [sp])[0]
    assert back.num_cached_tokens > 0 and back.output_ids == ref.output_ids  # the device cache was dropped, the host copies were not
    freeing = mk(enable_hierarchical_cache=True, release_hicache=True)
    freeing.release_memory_occupation(["kv_cache"])
    assert freeing.kv.allocator.host_tier.k is None and freeing.kv.allocator.host_tier.num_bytes() == 0
    freeing.resume_memory_occupation(["kv_cache"])
    assert freeing.kv.allocator.host_tier.k is not None


def test_deterministic_inference_switch_removes_batch_dependent_choices():
    from slime_b200 import ops

    try:
        assert ops._pick_splitk(8, 1024, 8192, 128) > 1
        e = Engine(get_preset("tiny"), ServerArgs(page_size=4, max_running_requests=2, context_length=64, disable_cuda_graph=True,
                                                  enable_deterministic_inference=True), device="cpu", num_pages=24)  # fmt: skip
        assert ops.BATCH_INVARIANT and ops._pick_splitk(8, 1024, 8192, 128) == 1 == ops._pick_splitk(4096, 128, 65536, 128)
        e.weights.init_random(0, std=0.2)
        sp = dict(max_new_tokens=6, temperature=1.0, ignore_eos=True, sampling_seed=7)
        alone = e.generate([[1, 2, 3, 4, 5]], [sp])[0]
        crowd = e.generate([[1, 2, 3, 4, 5], [9, 8, 7], [4, 4, 4, 4, 4, 4, 4]], [sp, dict(sp, sampling_seed=1), dict(sp, sampling_seed=2)])[0]
        # (bit equality is a property of the GPU kernels; the CPU reference matmul may differ in the last bit)
        assert alone.output_ids == crowd.output_ids and np.abs(np.array(alone.output_logprobs) - np.array(crowd.output_logprobs)).max() < 1e-5
    finally:
        ops.set_batch_invariant(False)
