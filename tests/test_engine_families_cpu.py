"""The rollout engine against the trainer model, family by family (CPU, fp32): weights travel trainer -> checkpoint names
-> engine, then the engine's prompt log-probs (prefill path) and its decode log-probs must equal the trainer's."""

import numpy as np
import pytest
import torch

from slime_b200.engine.engine import Engine
from slime_b200.engine.server_args import ServerArgs
from slime_b200.models.config import ModelConfig
from slime_b200.models.gpt import GPTModel
from slime_b200.weight_sync import convert

BASE = dict(num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=2, kv_channels=16, ffn_hidden_size=128,
            vocab_size=256, rotary_base=1e4, tie_word_embeddings=False)  # fmt: skip
FAMILIES = {
    "qwen2": dict(add_qkv_bias=True, model_arch="Qwen2ForCausalLM"),
    "qwen3": dict(qk_layernorm=True, model_arch="Qwen3ForCausalLM"),
    "llama31": dict(model_arch="LlamaForCausalLM", rotary_scaling_type="llama3", rotary_scaling_factor=8.0, rotary_original_max_position=16),
    "qwen3_yarn": dict(qk_layernorm=True, model_arch="Qwen3ForCausalLM", rotary_scaling_type="yarn", rotary_scaling_factor=4.0,
                       rotary_original_max_position=16),
    "qwen3_moe": dict(qk_layernorm=True, num_experts=4, moe_ffn_hidden_size=32, moe_router_topk=2, model_arch="Qwen3MoeForCausalLM"),
    "glm4": dict(add_qkv_bias=True, post_self_attn_layernorm=True, post_mlp_layernorm=True, rotary_percent=0.5,
                 rotary_interleaved=True, model_arch="Glm4ForCausalLM"),
    "glm4_moe": dict(add_qkv_bias=True, rotary_percent=0.5, num_experts=4, moe_ffn_hidden_size=32, moe_router_topk=2,
                     moe_layer_freq=[0, 1], moe_shared_expert_intermediate_size=32, moe_router_score_function="sigmoid",
                     moe_router_enable_expert_bias=True, moe_router_pre_softmax=True, moe_router_topk_scaling_factor=1.5,
                     model_arch="Glm4MoeForCausalLM"),
    "sinks": dict(softmax_sinks=True, qk_layernorm=True, model_arch="Qwen3ForCausalLM"),
    "minimax_m2": dict(qk_layernorm_full=True, rotary_percent=0.5, num_experts=4, moe_ffn_hidden_size=32, moe_router_topk=2,
                       moe_router_score_function="sigmoid", moe_router_enable_expert_bias=True, moe_router_pre_softmax=True,
                       model_arch="MiniMaxM2ForCausalLM"),
    "qwen3_next": dict(num_layers=4, full_attention_interval=4, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=8,
                       linear_value_head_dim=8, attention_output_gate=True, qk_layernorm=True, rotary_percent=0.25, num_experts=4,
                       moe_ffn_hidden_size=32, moe_router_topk=2, moe_shared_expert_intermediate_size=32, moe_shared_expert_gate=True,
                       model_arch="Qwen3NextForCausalLM"),
    "qwen3_5": dict(num_layers=4, full_attention_interval=2, linear_num_key_heads=2, linear_num_value_heads=2, linear_key_head_dim=8,
                    linear_value_head_dim=8, attention_output_gate=True, qk_layernorm=True, rotary_percent=0.25,
                    model_arch="Qwen3_5ForCausalLM"),
    "deepseek_v3": dict(multi_latent_attention=True, q_lora_rank=24, kv_lora_rank=16, qk_head_dim=8, qk_pos_emb_head_dim=4, v_head_dim=8,
                        rotary_interleaved=True, num_experts=4, moe_ffn_hidden_size=32, moe_router_topk=2, moe_layer_freq=[0, 1],
                        moe_shared_expert_intermediate_size=32, moe_router_score_function="sigmoid",
                        moe_router_enable_expert_bias=True, moe_router_topk_scaling_factor=2.5, rotary_scaling_type="yarn",
                        rotary_scaling_factor=40.0, mscale=1.0, mscale_all_dim=1.0, model_arch="DeepseekV3ForCausalLM"),
    "glm5_dsa": dict(num_layers=3, multi_latent_attention=True, q_lora_rank=24, kv_lora_rank=16, qk_head_dim=8, qk_pos_emb_head_dim=4,
                     v_head_dim=12, rotary_interleaved=True, index_topk=5, index_n_heads=8, index_head_dim=8, index_topk_freq=2,
                     index_skip_topk_offset=1, model_arch="GlmMoeDsaForCausalLM"),
    "moonlight": dict(multi_latent_attention=True, q_lora_rank=None, kv_lora_rank=16, qk_head_dim=8, qk_pos_emb_head_dim=4,
                      v_head_dim=8, rotary_interleaved=True, model_arch="DeepseekV3ForCausalLM"),
    "deepseek_routing": dict(qk_layernorm=True, num_experts=8, moe_ffn_hidden_size=32, moe_router_topk=2, moe_router_num_groups=4,
                             moe_router_group_topk=2, moe_router_score_function="sigmoid", moe_router_enable_expert_bias=True,
                             moe_shared_expert_intermediate_size=64, model_arch="Qwen3MoeForCausalLM"),
}  # fmt: skip


@pytest.mark.parametrize("family", sorted(FAMILIES))
def test_engine_reproduces_the_trainers_log_probs(family):
    torch.manual_seed(0)
    cfg = ModelConfig(**{**BASE, **FAMILIES[family]})
    model = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=3)
    with torch.no_grad():  # make biases and norm weights non-trivial so that a dropped one shows
        for n, p in model.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * (1.0 if "softmax_offset" in n else 0.1))
        for n, b in model.named_buffers():
            if "expert_bias" in n:
                b.copy_(torch.randn_like(b) * 0.5)
    e = Engine(cfg, ServerArgs(page_size=4, max_running_requests=4, context_length=64, disable_cuda_graph=True), device="cpu", num_pages=64)
    hf = []
    for name, p in list(model.named_parameters()) + list(model.named_buffers()):
        hf += convert.convert_to_hf(cfg, name, p.detach())
    missing = e.weights.load_weights(hf)
    assert not missing, missing
    ids = torch.randint(0, cfg.vocab_size, (17,), generator=torch.Generator().manual_seed(1)).tolist()
    with torch.no_grad():
        logits = model(torch.tensor(ids))[0]
    ref = logits.log_softmax(-1)[:-1].gather(-1, torch.tensor(ids[1:])[:, None]).squeeze(-1).numpy()
    got = e.generate([ids], [dict(max_new_tokens=0)], logprob_start_len=0)[0].input_logprobs[1:]
    assert np.abs(np.array(got) - ref).max() < 2e-4, float(np.abs(np.array(got) - ref).max())
    # decode path: continue greedily from a prefix and score the continuation with the trainer
    r = e.generate([ids[:9]], [dict(max_new_tokens=6, temperature=0, ignore_eos=True)])[0]
    full = ids[:9] + r.output_ids
    with torch.no_grad():
        lp = model(torch.tensor(full))[0].log_softmax(-1)
    want = [float(lp[8 + i, t]) for i, t in enumerate(r.output_ids)]
    assert np.abs(np.array(r.output_logprobs) - np.array(want)).max() < 2e-4


def test_hf_checkpoint_round_trip_keeps_the_router_bias(tmp_path):
    """Trainer -> Hugging Face directory -> trainer for a sigmoid-router MoE: the score-correction bias (a buffer, not a
    parameter) is written and read back."""
    from argparse import Namespace

    from slime_b200.checkpoint import hf_loader, hf_saver

    cfg = ModelConfig(**{**BASE, **FAMILIES["glm4_moe"]})
    a = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=1)
    with torch.no_grad():
        for n, b in a.named_buffers():
            if n.endswith("expert_bias"):
                b.copy_(torch.arange(b.numel(), dtype=b.dtype) * 0.25)
    tensors = {}
    for name, p in list(a.named_parameters()) + [(n, b) for n, b in a.named_buffers() if n.endswith("expert_bias")]:
        tensors.update(dict(convert.convert_to_hf(cfg, name, p.detach().clone())))
    from safetensors.torch import save_file

    import json

    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_hf_dict()))
    b = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=2)
    wrap = Namespace(cfg=cfg, named_parameters=b.named_parameters, named_buffers=b.named_buffers)
    missing = hf_loader.load_hf_weights(str(tmp_path), wrap)
    assert not missing, missing
    for (n, x), (_, y) in zip(list(a.named_parameters()) + list(a.named_buffers()), list(b.named_parameters()) + list(b.named_buffers())):
        assert torch.equal(x, y), n


def test_hybrid_engine_carries_recurrent_state_through_chunked_prefill_and_batched_decode():
    """Qwen3.5-style hybrid: prompts prefilled in small chunks (the delta-net state and the convolution history travel from
    chunk to chunk), then decoded together in one batch; every request's log-probs equal the trainer's."""
    torch.manual_seed(0)
    cfg = ModelConfig(**{**BASE, **FAMILIES["qwen3_5"]})
    model = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=3)
    e = Engine(cfg, ServerArgs(page_size=4, max_running_requests=4, context_length=64, disable_cuda_graph=True, chunked_prefill_size=5,
                               max_prefill_tokens=7), device="cpu", num_pages=64)  # fmt: skip
    hf = [x for n, p in model.named_parameters() for x in convert.convert_to_hf(cfg, n, p.detach())]
    assert not e.weights.load_weights(hf)
    assert e.kv.num_layers == 2 and e.runner.has_gdn  # two of the four layers keep keys and values
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (13, 3, 9)]
    reqs = e.generate(prompts, [dict(max_new_tokens=5 + i, temperature=0, ignore_eos=True) for i in range(3)])
    assert e.stats["steps"] > 6  # the prompts really went through several prefill passes
    for p, r in zip(prompts, reqs):
        full = p + r.output_ids
        with torch.no_grad():
            lp = model(torch.tensor(full))[0].log_softmax(-1)
        want = [float(lp[len(p) - 1 + i, t]) for i, t in enumerate(r.output_ids)]
        assert np.abs(np.array(r.output_logprobs) - np.array(want)).max() < 2e-4
        assert r.num_cached_tokens == 0  # hybrids do not reuse prefixes
    # the same prompt again: still no prefix reuse, same answer
    again = e.generate([prompts[0]], [dict(max_new_tokens=5, temperature=0, ignore_eos=True)])[0]
    assert again.output_ids == reqs[0].output_ids and again.num_cached_tokens == 0


def test_latent_attention_engine_reuses_prefixes_and_prefills_in_chunks():
    """DeepSeek-style model: the latent cache serves a cached prefix and chunked prefill (queries of a later chunk attend
    the latent vectors of earlier ones), and sibling requests share pages; log-probs equal the trainer's."""
    torch.manual_seed(0)
    cfg = ModelConfig(**{**BASE, **FAMILIES["deepseek_v3"]})
    model = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=3)
    e = Engine(cfg, ServerArgs(page_size=4, max_running_requests=4, context_length=64, disable_cuda_graph=True, chunked_prefill_size=6,
                               max_prefill_tokens=10), device="cpu", num_pages=64)  # fmt: skip
    hf = [x for n, p in list(model.named_parameters()) + list(model.named_buffers()) for x in convert.convert_to_hf(cfg, n, p.detach())]
    assert not e.weights.load_weights(hf)
    assert e.kv.k[0].shape[1:] == (1, cfg.kv_lora_rank + cfg.qk_pos_emb_head_dim) and e.kv.v[0].shape[-1] == 0
    g = torch.Generator().manual_seed(5)
    p = torch.randint(0, cfg.vocab_size, (14,), generator=g).tolist()
    reqs = e.generate([p, p, p[:9] + [1, 2]], [dict(max_new_tokens=5, temperature=0, ignore_eos=True)] * 3)
    assert reqs[1].num_cached_tokens >= 4 and reqs[2].num_cached_tokens >= 4  # pages of the first request's prompt were reused
    for r in reqs:
        full = r.input_ids + r.output_ids
        with torch.no_grad():
            lp = model(torch.tensor(full))[0].log_softmax(-1)
        want = [float(lp[len(r.input_ids) - 1 + i, t]) for i, t in enumerate(r.output_ids)]
        assert np.abs(np.array(r.output_logprobs) - np.array(want)).max() < 2e-4
    assert reqs[0].output_ids == reqs[1].output_ids
