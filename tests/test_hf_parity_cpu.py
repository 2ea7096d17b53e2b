"""Whole-model parity with the Transformers implementations, family by family, on random weights (CPU, fp32): the
library builds a tiny model, its config goes through ``ModelConfig.from_hf``, its tensors through the checkpoint-name
rules of ``weight_sync/convert.py`` into the trainer model, and the logits of a random prompt must agree. A wrong default
in ``from_hf``, a misnamed tensor, a transposed projection, another rotary convention or routing rule shows up here.
(The library is the oracle in this file only; nothing in the package imports these model classes.)"""

import importlib

import pytest
import torch

from slime_b200.models.config import ModelConfig
from slime_b200.models.gpt import GPTModel
from slime_b200.weight_sync import convert

BASE = dict(vocab_size=200, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
            max_position_embeddings=256, tie_word_embeddings=False)  # fmt: skip
MLA = dict(num_key_value_heads=4, kv_lora_rank=16, q_lora_rank=24, qk_rope_head_dim=4, v_head_dim=12, qk_nope_head_dim=8)
DS_MOE = dict(moe_intermediate_size=32, n_shared_experts=1, num_experts_per_tok=2, first_k_dense_replace=1, norm_topk_prob=True)
# module, config class, model class, architecture string, config arguments
CASES = {
    "qwen2": ("qwen2", "Qwen2Config", "Qwen2ForCausalLM", dict(BASE)),
    "qwen3": ("qwen3", "Qwen3Config", "Qwen3ForCausalLM", dict(BASE, head_dim=16)),
    "llama": ("llama", "LlamaConfig", "LlamaForCausalLM", dict(BASE)),
    "llama31": ("llama", "LlamaConfig", "LlamaForCausalLM",
                dict(BASE, max_position_embeddings=512, rope_parameters=dict(rope_type="llama3", rope_theta=10000.0, factor=8.0, low_freq_factor=1.0,
                                                                             high_freq_factor=4.0, original_max_position_embeddings=64))),
    "qwen3_moe": ("qwen3_moe", "Qwen3MoeConfig", "Qwen3MoeForCausalLM",
                  dict(BASE, head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, norm_topk_prob=True,
                       decoder_sparse_step=1, mlp_only_layers=[])),
    "glm4": ("glm4", "Glm4Config", "Glm4ForCausalLM", dict(BASE, pad_token_id=0, head_dim=16, partial_rotary_factor=0.5, attention_bias=True)),
    "glm4_moe": ("glm4_moe", "Glm4MoeConfig", "Glm4MoeForCausalLM",
                 dict(BASE, **DS_MOE, head_dim=16, partial_rotary_factor=0.5, attention_bias=True, n_routed_experts=4, n_group=1,
                      topk_group=1, routed_scaling_factor=1.5, use_qk_norm=True)),
    "glm4_moe_lite": ("glm4_moe_lite", "Glm4MoeLiteConfig", "Glm4MoeLiteForCausalLM",
                      dict(BASE, **MLA, **DS_MOE, n_routed_experts=4, n_group=1, topk_group=1, routed_scaling_factor=1.8)),
    "deepseek_v3": ("deepseek_v3", "DeepseekV3Config", "DeepseekV3ForCausalLM",
                    dict(BASE, **MLA, **DS_MOE, n_routed_experts=8, n_group=4, topk_group=2, routed_scaling_factor=2.5)),
    "deepseek_v3_yarn": ("deepseek_v3", "DeepseekV3Config", "DeepseekV3ForCausalLM",
                         dict(BASE, **{**MLA, "q_lora_rank": None, "qk_rope_head_dim": 8}, **DS_MOE, n_routed_experts=8, n_group=4,
                              topk_group=2, routed_scaling_factor=2.5,
                              rope_parameters=dict(rope_type="yarn", rope_theta=10000.0, factor=4.0, original_max_position_embeddings=64,
                                                   beta_fast=32, beta_slow=1, mscale=1.0, mscale_all_dim=0.707))),
    "glm_moe_dsa": ("glm_moe_dsa", "GlmMoeDsaConfig", "GlmMoeDsaForCausalLM",
                    dict(BASE, **MLA, **DS_MOE, n_routed_experts=4, n_group=2, topk_group=1, routed_scaling_factor=1.5, index_topk=5,
                         index_n_heads=8, index_head_dim=8, rms_norm_eps=1e-5, mlp_layer_types=["dense", "sparse", "sparse"])),
    "minimax_m2": ("minimax_m2", "MiniMaxM2Config", "MiniMaxM2ForCausalLM",
                   dict(BASE, head_dim=16, num_local_experts=4, num_experts_per_tok=2, use_qk_norm=True,
                        rope_parameters=dict(rope_type="default", rope_theta=10000.0, partial_rotary_factor=0.5))),
    "qwen3_next": ("qwen3_next", "Qwen3NextConfig", "Qwen3NextForCausalLM",
                   dict(BASE, num_hidden_layers=4, head_dim=16, partial_rotary_factor=0.25, linear_conv_kernel_dim=4, linear_key_head_dim=8,
                        linear_value_head_dim=8, linear_num_key_heads=2, linear_num_value_heads=4, full_attention_interval=2,
                        num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=32,
                        norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[], layer_types=["linear_attention", "full_attention"] * 2)),
}  # fmt: skip


def _checkpoint_names(module: str, sd: dict) -> dict:
    """The library keeps a layer's experts in two fused tensors and uses its own module names; checkpoints (and every
    consumer of checkpoint names here) name each expert, MiniMax-M2 under ``block_sparse_moe`` as w1 / w3 / w2."""
    out = {}
    for k, v in sd.items():
        if k.endswith("mlp.experts.gate_up_proj"):
            for e in range(v.shape[0]):
                g, u = v[e].chunk(2, 0)
                out[k.replace("gate_up_proj", f"{e}.gate_proj.weight")], out[k.replace("gate_up_proj", f"{e}.up_proj.weight")] = g, u
        elif k.endswith("mlp.experts.down_proj"):
            for e in range(v.shape[0]):
                out[k.replace("down_proj", f"{e}.down_proj.weight")] = v[e]
        else:
            out[k] = v
    if module == "minimax_m2":
        ren = {}
        for k, v in out.items():
            k = k.replace(".mlp.e_score_correction_bias", ".block_sparse_moe.e_score_correction_bias").replace(".mlp.gate.weight", ".block_sparse_moe.gate.weight")
            k = k.replace(".mlp.experts.", ".block_sparse_moe.experts.").replace("gate_proj.weight", "w1.weight").replace("up_proj.weight", "w3.weight")
            ren[k.replace("down_proj.weight", "w2.weight") if ".block_sparse_moe." in k else k] = v
        out = ren
    return out


@pytest.mark.parametrize("family", sorted(CASES))
def test_trainer_model_matches_the_library_model(family):
    module, config_cls, model_cls, kw = CASES[family]
    cfg = getattr(importlib.import_module(f"transformers.models.{module}.configuration_{module}"), config_cls)(**kw)
    cfg._attn_implementation = "eager"  # an explicit causal mask on every path (the sparse-attention model needs one)
    torch.manual_seed(0)
    hf = getattr(importlib.import_module(f"transformers.models.{module}.modeling_{module}"), model_cls)(cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():  # norms start at 1 and biases at 0: make every tensor matter
            p.add_(torch.randn_like(p) * 0.05)
        for n, b in hf.named_buffers():
            if "e_score_correction_bias" in n:
                b.copy_(torch.randn_like(b) * 0.3)
    d = cfg.to_dict()
    d["architectures"] = [model_cls]
    mc = ModelConfig.from_hf(d)
    if family == "glm_moe_dsa":
        # The library rotates half-split pairs in this family; the training and serving stacks this framework follows
        # rotate (2i, 2i + 1) pairs, which stays the default. The flag is the only difference.
        assert mc.rotary_interleaved
        mc.rotary_interleaved = False
    ours = GPTModel(mc, dtype=torch.float32, device="cpu", seed=1)
    sd = _checkpoint_names(module, hf.state_dict())
    used = set()
    with torch.no_grad():
        for name, p in list(ours.named_parameters()) + list(ours.named_buffers()):
            names, rule = convert.hf_sources_for(mc, name)
            assert all(n in sd for n in names), (name, names)
            used.update(names)
            p.copy_(convert.merge_hf_sources(rule, [sd[n] for n in names], mc))
    assert not [k for k in sd if k not in used and "rotary_emb" not in k], sorted(set(sd) - used)[:6]
    # and back: the trainer's tensors under checkpoint names are the library's tensors
    back = dict(x for n, p in list(ours.named_parameters()) + list(ours.named_buffers()) for x in convert.convert_to_hf(mc, n, p.detach()))
    assert set(back) == used and all(torch.allclose(back[k], sd[k], atol=1e-6) for k in used)
    ids = torch.randint(0, cfg.vocab_size, (1, 23), generator=torch.Generator().manual_seed(3))
    with torch.no_grad():
        want, got = hf(input_ids=ids).logits[0], ours(ids)[0]
    assert (got - want).abs().max() < 3e-4, float((got - want).abs().max())
