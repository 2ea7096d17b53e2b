"""Speculative decoding with the model's own draft head: the token sequence, log-probs and side outputs must be those of
ordinary decoding; the draft head in the engine must compute what the trainer's draft head computes."""

import numpy as np
import pytest
import torch

from slime_b200.engine.engine import Engine
from slime_b200.engine.server_args import ServerArgs
from slime_b200.models.config import ModelConfig
from slime_b200.models.gpt import GPTModel
from slime_b200.weight_sync import convert

BASE = dict(num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=2, kv_channels=16, ffn_hidden_size=128,
            vocab_size=48, rotary_base=1e4, tie_word_embeddings=False, mtp_num_layers=1, qk_layernorm=True)  # fmt: skip
VARIANTS = {
    "dense": dict(model_arch="Qwen3ForCausalLM"),
    "mimo": dict(add_qkv_bias=True, qk_layernorm=False, model_arch="MiMoForCausalLM"),
    "moe": dict(num_experts=4, moe_ffn_hidden_size=32, moe_router_topk=2, model_arch="Qwen3MoeForCausalLM"),
    "glm4_moe": dict(add_qkv_bias=True, rotary_percent=0.5, num_experts=4, moe_ffn_hidden_size=32, moe_router_topk=2,
                     moe_layer_freq=[0, 1], moe_shared_expert_intermediate_size=32, moe_router_score_function="sigmoid",
                     moe_router_enable_expert_bias=True, moe_router_pre_softmax=True, model_arch="Glm4MoeForCausalLM"),
    "mla": dict(multi_latent_attention=True, q_lora_rank=24, kv_lora_rank=16, qk_head_dim=8, qk_pos_emb_head_dim=4, v_head_dim=8,
                rotary_interleaved=True, qk_layernorm=False, model_arch="DeepseekV3ForCausalLM"),
}  # fmt: skip


def _pair(variant, spec_kw=None, **engine_kw):
    torch.manual_seed(0)
    cfg = ModelConfig(**{**BASE, **VARIANTS[variant]})
    model = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=3)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    hf = []
    for name, p in list(model.named_parameters()) + list(model.named_buffers()):
        hf += convert.convert_to_hf(cfg, name, p.detach())
    kw = dict(page_size=4, max_running_requests=4, context_length=96, disable_cuda_graph=True, **engine_kw)
    plain = Engine(cfg, ServerArgs(**kw), device="cpu", num_pages=96)
    spec = Engine(cfg, ServerArgs(**kw, speculative_algorithm="EAGLE", **(spec_kw or dict(speculative_num_steps=3, speculative_num_draft_tokens=4))),
                  device="cpu", num_pages=96)  # fmt: skip
    assert not plain.weights.load_weights(hf) and not spec.weights.load_weights(hf)
    assert len(spec.kv.k) == len(plain.kv.k) + 1  # the draft head's slab
    return cfg, model, plain, spec


def _prompts(cfg, n, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab_size, (int(torch.randint(5, 14, (1,), generator=g)),), generator=g).tolist() for _ in range(n)]


@pytest.mark.parametrize("variant", sorted(VARIANTS))
def test_speculative_rounds_reproduce_ordinary_decoding(variant):
    cfg, _, plain, spec = _pair(variant)
    prompts = _prompts(cfg, 5)
    for sampling in (dict(max_new_tokens=24, temperature=0, ignore_eos=True),
                     dict(max_new_tokens=21, temperature=1.0, ignore_eos=True, sampling_seed=11),
                     dict(max_new_tokens=17, temperature=0.8, top_p=0.9, top_k=20, ignore_eos=True, sampling_seed=5)):
        a = plain.generate(prompts, [dict(sampling) for _ in prompts])
        b = spec.generate(prompts, [dict(sampling) for _ in prompts])
        for x, y in zip(a, b):
            assert x.output_ids == y.output_ids, (variant, sampling)
            assert np.abs(np.array(x.output_logprobs) - np.array(y.output_logprobs)).max() < 2e-4
            assert y.finish_reason == x.finish_reason
            m = spec.meta_info(y)
            assert m["spec_verify_ct"] >= 1 and m["spec_draft_token_num"] >= m["spec_accept_token_num"] >= 0
            # every round emits its accepted guesses plus one token; the first token came from the prefill
            assert m["spec_verify_ct"] + m["spec_accept_token_num"] == len(y.output_ids) - 1
    st = spec.kv.allocator.stats()
    assert st["free"] + st["cached"] == 96 - 1  # nothing leaked: every page is free or indexed (page 0 is the scratch page)
    assert not spec.running and not spec.prefilling and not spec.waiting


def test_engine_draft_head_computes_the_trainers_draft_head():
    """After the prefill and after every round, the first guess is the argmax of the trainer's draft logits at the last
    position whose successor is known."""
    cfg, model, _, spec = _pair("dense")
    ids = _prompts(cfg, 1, seed=4)[0]
    r = spec.add_request(ids, dict(max_new_tokens=12, temperature=0, ignore_eos=True))

    def trainer_guess(tokens):
        full = torch.tensor(tokens)
        with torch.enable_grad():
            model.mtp_training = True
            model(full)
            hidden, _, packed, table = model._mtp_inputs
            model._mtp_inputs = None
        with torch.no_grad():
            nxt = torch.cat([full[1:], full.new_zeros(1)])
            out, _ = model.mtp.layers[0](hidden.detach(), model.embedding.word_embeddings.weight[nxt], table, packed)
            logits = out @ model.output_weight().t()
        # row p (stream of position p, embedding of token p + 1) guesses token p + 2: the guess for the token after the
        # last known one comes from the row before it
        return int(logits[len(tokens) - 2].argmax())

    rounds = 0
    while not r.finished():
        spec.step()  # the first step is the prefill (+ first token + the draft head over the prompt)
        if not r.finished():
            assert r.spec_draft[0] == trainer_guess(ids + r.output_ids), rounds
            rounds += 1
    assert rounds >= 3


def test_a_draft_head_that_knows_the_answer_is_accepted_in_full(monkeypatch):
    """With guesses taken from the known continuation every round keeps k + 1 tokens; a wrong guess ends the run of kept
    tokens at the trunk's own sample."""
    cfg, _, plain, spec = _pair("dense")
    ids = _prompts(cfg, 1, seed=9)[0]
    want = plain.generate([ids], [dict(max_new_tokens=22, temperature=0, ignore_eos=True)])[0].output_ids
    seq = ids + want

    orig = spec.runner.draft_extend
    state = {}

    def oracle_extend(depth, hidden, next_ids, positions, *a, **k):
        state["pos"] = positions.tolist()
        return orig(depth, hidden, next_ids, positions, *a, **k)

    def oracle_logits(normed):
        # the row at position p guesses the token at position p + 2
        out = torch.full((normed.shape[0], cfg.vocab_size), -1e9)
        pos = state["pos"][-normed.shape[0]:] if normed.shape[0] <= len(state["pos"]) else state["pos"]
        rows = pos if len(pos) == normed.shape[0] else [pos[-1]] * normed.shape[0]
        for i, p in enumerate(rows):
            t = seq[p + 2] if p + 2 < len(seq) else 0
            if state.get("sabotage") and p + 2 == len(ids) + 7:
                t = (t + 1) % cfg.vocab_size
            out[i, t] = 0.0
        return out

    monkeypatch.setattr(spec.runner, "draft_extend", oracle_extend)
    monkeypatch.setattr(spec.runner, "logits_of", oracle_logits)
    r = spec.generate([ids], [dict(max_new_tokens=22, temperature=0, ignore_eos=True)])[0]
    m = spec.meta_info(r)
    assert r.output_ids == want
    assert m["spec_accept_token_num"] == m["spec_draft_token_num"]  # every guess kept
    assert m["spec_verify_ct"] == -(-(22 - 1) // 4)  # 4 tokens a round after the prefill's first token
    state["sabotage"] = True
    r = spec.generate([ids], [dict(max_new_tokens=22, temperature=0, ignore_eos=True)])[0]
    m2 = spec.meta_info(r)
    assert r.output_ids == want and m2["spec_accept_token_num"] < m2["spec_draft_token_num"]


def test_speculation_with_stops_prefix_reuse_routed_experts_and_page_pressure():
    cfg, _, plain, spec = _pair("moe", enable_return_routed_experts=True)
    prompts = _prompts(cfg, 4, seed=2)
    ref = plain.generate(prompts, [dict(max_new_tokens=20, temperature=0, ignore_eos=True)] * 4, return_routed_experts=True)
    # a stop token in the middle of a round ends the request there
    stop = ref[0].output_ids[6]
    a = plain.generate([prompts[0]], [dict(max_new_tokens=20, temperature=0, ignore_eos=True, stop_token_ids=[stop])])[0]
    b = spec.generate([prompts[0]], [dict(max_new_tokens=20, temperature=0, ignore_eos=True, stop_token_ids=[stop])])[0]
    assert a.output_ids == b.output_ids and b.finish_reason == a.finish_reason == {"type": "stop", "matched": stop}
    # routed experts: one row per fed token, the trunk's layers only
    got = spec.generate(prompts, [dict(max_new_tokens=20, temperature=0, ignore_eos=True)] * 4, return_routed_experts=True)
    for x, y in zip(ref, got):
        assert x.output_ids == y.output_ids
        assert torch.equal(torch.cat(x.routed_experts), torch.cat(y.routed_experts))
    # the same prompt again is served from the prefix cache, draft head included
    again = spec.generate([prompts[1]], [dict(max_new_tokens=20, temperature=0, ignore_eos=True)])[0]
    assert again.num_cached_tokens > 0 and again.output_ids == ref[1].output_ids
    # few pages: requests are retracted and finish all the same
    torch.manual_seed(0)
    small = Engine(cfg, ServerArgs(page_size=4, max_running_requests=4, context_length=96, disable_cuda_graph=True,
                                   speculative_algorithm="EAGLE", speculative_num_steps=2, speculative_num_draft_tokens=3),
                   device="cpu", num_pages=20)  # fmt: skip
    for (n1, t1), (n2, t2) in zip(_named(spec), _named(small)):
        t2.copy_(t1)
    out = small.generate(prompts, [dict(max_new_tokens=20, temperature=0, ignore_eos=True)] * 4)
    assert [o.output_ids for o in out] == [o.output_ids for o in ref]


def _named(engine):
    return [(i, t) for i, t in enumerate(engine.weights.tensors())]


def test_speculation_needs_a_draft_head_and_a_chain():
    cfg = ModelConfig(**{**BASE, "mtp_num_layers": 0, "model_arch": "Qwen3ForCausalLM"})
    with pytest.raises(ValueError, match="draft head"):
        Engine(cfg, ServerArgs(speculative_algorithm="EAGLE", disable_cuda_graph=True), device="cpu", num_pages=16)
    cfg = ModelConfig(**{**BASE, "model_arch": "Qwen3ForCausalLM"})
    with pytest.raises(NotImplementedError, match="chain"):
        Engine(cfg, ServerArgs(speculative_algorithm="EAGLE", speculative_eagle_topk=4, disable_cuda_graph=True), device="cpu", num_pages=16)
    with pytest.raises(ValueError, match="rows"):
        Engine(cfg, ServerArgs(speculative_algorithm="EAGLE", speculative_num_steps=3, speculative_num_draft_tokens=8,
                               disable_cuda_graph=True), device="cpu", num_pages=16)  # fmt: skip


def test_mimo_draft_head_names_round_trip():
    """MiMo keeps its draft head under model.mtp_layers.k with the joining projection's halves swapped."""
    cfg = ModelConfig(**{**BASE, **VARIANTS["mimo"]})
    model = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=3)
    named = dict(model.named_parameters())
    hf = dict(x for n, p in named.items() if n.startswith("mtp.") for x in convert.convert_to_hf(cfg, n, p.detach()))
    assert {"model.mtp_layers.0.token_layernorm.weight", "model.mtp_layers.0.hidden_layernorm.weight", "model.mtp_layers.0.input_proj.weight",
            "model.mtp_layers.0.final_layernorm.weight", "model.mtp_layers.0.self_attn.q_proj.weight",
            "model.mtp_layers.0.mlp.down_proj.weight"} <= set(hf)  # fmt: skip
    w = named["mtp.layers.0.eh_proj.weight"]
    assert torch.equal(hf["model.mtp_layers.0.input_proj.weight"], torch.cat([w[:, 64:], w[:, :64]], dim=1))
    for n, p in named.items():
        if n.startswith("mtp."):
            names, rule = convert.hf_sources_for(cfg, n)
            assert torch.equal(convert.merge_hf_sources(rule, [hf[x] for x in names], cfg), p), n
