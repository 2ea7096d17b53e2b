"""Architecture presets for the model families the launch recipes name, and a CLI that prints them as flags.

    python -m slime_b200.models.presets --list
    python -m slime_b200.models.presets qwen3-4B            # -> "--num-layers 36 --hidden-size 2560 ..." (one line)
    MODEL_ARGS=($(python -m slime_b200.models.presets qwen3-30B-A3B))   # in a launch script

Every entry is the constructor arguments of ``ModelConfig``; ``--hf-checkpoint preset:<name>`` builds a random-weight
model from it, and a real checkpoint's ``config.json`` overrides nothing here (it is read instead). Families with attention variants, latent
attention, sparse latent attention or gated delta-net layers build their layers from ``models/mixers.py``; what is not
implemented is listed in ``UNSUPPORTED`` with the missing piece, so asking for it fails with a reason instead of a
silently wrong model. Parity: scripts/models/*.sh (39 flag sets).
"""

from __future__ import annotations

import argparse
import dataclasses
import sys


def _dense(layers, hidden, ffn, heads, groups, vocab, *, kv=None, rope=1e6, eps=1e-6, tied=False, bias=False, qk=False,
           arch="Qwen2ForCausalLM", **extra) -> dict:  # fmt: skip
    d = dict(num_layers=layers, hidden_size=hidden, ffn_hidden_size=ffn, num_attention_heads=heads, num_query_groups=groups,
             vocab_size=vocab, kv_channels=kv or hidden // heads, rotary_base=rope, norm_epsilon=eps,
             tie_word_embeddings=tied, add_qkv_bias=bias, qk_layernorm=qk, model_arch=arch)  # fmt: skip
    d.update(extra)
    return d


def _moe(dense_layers: int, moe_layers: int, **kw) -> dict:
    kw["moe_layer_freq"] = [0] * dense_layers + [1] * moe_layers
    return kw


MORE_PRESETS: dict[str, dict] = {
    "qwen2.5-1.5b": _dense(28, 1536, 8960, 12, 2, 151936, rope=1e4, tied=True, bias=True),
    "qwen2.5-3b": _dense(36, 2048, 11008, 16, 2, 151936, tied=True, bias=True),
    "qwen2.5-7b": _dense(28, 3584, 18944, 28, 4, 152064, bias=True),
    "qwen2.5-32b": _dense(64, 5120, 27648, 40, 8, 152064, eps=1e-5, bias=True),
    "qwen3-1.7b": _dense(28, 2048, 6144, 16, 8, 151936, kv=128, tied=True, qk=True, arch="Qwen3ForCausalLM"),
    "qwen3-14b": _dense(40, 5120, 17408, 40, 8, 151936, kv=128, qk=True, arch="Qwen3ForCausalLM"),
    "qwen3-4b-instruct-2507": _dense(36, 2560, 9728, 32, 8, 151936, kv=128, rope=5e6, tied=True, qk=True,
                                     arch="Qwen3ForCausalLM"),
    "llama3.1-8b-instruct": _dense(32, 4096, 14336, 32, 8, 128256, kv=128, rope=5e5, eps=1e-5, arch="LlamaForCausalLM",
                                   rotary_scaling_factor=8.0, rotary_scaling_type="llama3", rotary_original_max_position=8192,
                                   max_position_embeddings=131072),
    "llama3.2-3b-instruct": _dense(28, 3072, 8192, 24, 8, 128256, kv=128, rope=5e5, eps=1e-5, tied=True,
                                   arch="LlamaForCausalLM", rotary_scaling_factor=32.0, rotary_scaling_type="llama3",
                                   rotary_original_max_position=8192, max_position_embeddings=131072),
    "mimo-7b-rl": _dense(36, 4096, 11008, 32, 8, 151680, rope=6.4e5, eps=1e-5, bias=True, mtp_num_layers=1,
                         arch="MiMoForCausalLM"),
    "qwen3-235b-a22b": _moe(0, 94, **_dense(94, 4096, 12288, 64, 4, 151936, kv=128, qk=True, arch="Qwen3MoeForCausalLM",
                                            num_experts=128, moe_ffn_hidden_size=1536, moe_router_topk=8)),
}  # fmt: skip

def _mla(q_lora, kv_lora=512, nope=128, rope=64, v=128) -> dict:
    return dict(multi_latent_attention=True, q_lora_rank=q_lora, kv_lora_rank=kv_lora, qk_head_dim=nope,
                qk_pos_emb_head_dim=rope, v_head_dim=v, rotary_interleaved=True)  # fmt: skip


def _sigmoid_router(scale, groups=None, group_topk=None) -> dict:
    return dict(moe_router_score_function="sigmoid", moe_router_pre_softmax=True, moe_router_enable_expert_bias=True,
                moe_router_topk_scaling_factor=scale, moe_router_num_groups=groups, moe_router_group_topk=group_topk)  # fmt: skip


def _gdn(key_heads, value_heads, key_dim=128, value_dim=128) -> dict:
    # Head counts of the linear-attention layers come from the checkpoint's config.json (linear_num_key_heads, ...);
    # a preset only needs them for random-weight runs.
    return dict(full_attention_interval=4, linear_num_key_heads=key_heads, linear_num_value_heads=value_heads,
                linear_key_head_dim=key_dim, linear_value_head_dim=value_dim, linear_conv_kernel_dim=4,
                attention_output_gate=True, rotary_percent=0.25)  # fmt: skip


def _deepseek_v3(layers: int) -> dict:
    return _moe(min(3, layers), max(layers - 3, 0), **_dense(
        layers, 7168, 18432, 128, 128, 129280, kv=128, rope=1e4, arch="DeepseekV3ForCausalLM", rotary_scaling_factor=40.0,
        rotary_scaling_type="yarn", mscale=1.0, mscale_all_dim=1.0,
        num_experts=256, moe_ffn_hidden_size=2048, moe_router_topk=8, moe_shared_expert_intermediate_size=2048,
        **_mla(1536), **_sigmoid_router(2.5, 8, 4)))  # fmt: skip


def _kimi_k2(eps: float, scaling: float) -> dict:
    return _moe(1, 60, **_dense(61, 7168, 18432, 64, 64, 163840, kv=64, rope=5e4, eps=eps, arch="DeepseekV3ForCausalLM",
                                rotary_scaling_factor=scaling, rotary_scaling_type="yarn", mscale=1.0, mscale_all_dim=1.0,
                                num_experts=384, moe_ffn_hidden_size=2048, moe_router_topk=8,
                                moe_shared_expert_intermediate_size=2048, **_mla(1536), **_sigmoid_router(2.827)))  # fmt: skip


def _glm5(rope: float) -> dict:
    # indexer sizes follow the DeepSeek-V3.2 layout this family adopted; a checkpoint's config.json overrides them
    return _moe(3, 75, **_dense(78, 6144, 12288, 64, 64, 154880, kv=192, rope=rope, arch="GlmMoeDsaForCausalLM",
                                num_experts=256, moe_ffn_hidden_size=2048, moe_router_topk=8,
                                moe_shared_expert_intermediate_size=2048, index_topk=2048, index_n_heads=32, index_head_dim=128,
                                **_mla(2048, nope=192, v=256), **_sigmoid_router(2.5)))  # fmt: skip


def _glm45(dense, moe, hidden, ffn, experts, moe_ffn, scale=None) -> dict:
    return _moe(dense, moe, **_dense(dense + moe, hidden, ffn, 96, 8, 151552, kv=128, bias=True, arch="Glm4MoeForCausalLM",
                                     rotary_percent=0.5, num_experts=experts, moe_ffn_hidden_size=moe_ffn, moe_router_topk=8,
                                     moe_shared_expert_intermediate_size=moe_ffn, **_sigmoid_router(scale)))  # fmt: skip


MORE_PRESETS.update({
    "glm4-9b": _dense(40, 4096, 13696, 32, 2, 151552, rope=1e4, eps=1e-5, bias=True, arch="Glm4ForCausalLM",
                      post_self_attn_layernorm=True, post_mlp_layernorm=True, rotary_interleaved=True, rotary_percent=0.5),
    "glm4-32b": _dense(64, 6144, 23040, 48, 8, 151552, rope=1e4, eps=1e-5, arch="Glm4ForCausalLM",
                       post_self_attn_layernorm=True, post_mlp_layernorm=True, rotary_interleaved=True, rotary_percent=0.5),
    "glm4.5-106b-a12b": _glm45(1, 45, 4096, 10944, 128, 1408),
    "glm4.5-355b-a32b": _glm45(3, 89, 5120, 12288, 160, 1536, 2.5),
    "glm4.7-30b-a3b": _moe(1, 46, **_dense(47, 2048, 10240, 20, 20, 154880, kv=192, bias=True, arch="Glm4MoeLiteForCausalLM",
                                           num_experts=64, moe_ffn_hidden_size=1536, moe_router_topk=4,
                                           moe_shared_expert_intermediate_size=1536, **_mla(768, nope=192, v=256),
                                           **_sigmoid_router(1.8))),
    "deepseek-v3": _deepseek_v3(61), "deepseek-v3-5layer": _deepseek_v3(5), "deepseek-v3-20layer": _deepseek_v3(20),
    "kimi-k2": _kimi_k2(1e-6, 32.0), "kimi-k2-thinking": _kimi_k2(1e-5, 64.0),
    "moonlight": _moe(1, 26, **_dense(27, 2048, 11264, 16, 16, 163840, kv=128, rope=5e4, eps=1e-5, arch="DeepseekV3ForCausalLM",
                                      num_experts=64, moe_ffn_hidden_size=1408, moe_router_topk=6,
                                      moe_shared_expert_intermediate_size=2816, **_mla(None), **_sigmoid_router(2.446))),
    "glm5-744b-a40b": _glm5(1e6), "glm5.2-744b-a40b": _glm5(8e6),
    "minimax-m2": _dense(62, 3072, 1536, 48, 8, 200064, kv=128, rope=5e6, arch="MiniMaxM2ForCausalLM", rotary_percent=0.5,
                         qk_layernorm_full=True, num_experts=256, moe_ffn_hidden_size=1536, moe_router_topk=8,
                         moe_router_score_function="sigmoid", moe_router_pre_softmax=True, moe_router_enable_expert_bias=True),
    "qwen3-next-80b-a3b": _dense(48, 2048, 5120, 16, 2, 151936, kv=256, rope=1e7, qk=True, arch="Qwen3NextForCausalLM",
                                 num_experts=512, moe_ffn_hidden_size=512, moe_router_topk=10,
                                 moe_shared_expert_intermediate_size=512, moe_shared_expert_gate=True, **_gdn(16, 32)),
    "qwen3.5-0.8b": _dense(24, 1024, 3584, 8, 2, 248320, kv=256, rope=1e7, tied=True, qk=True, arch="Qwen3_5ForCausalLM", **_gdn(16, 16)),
    "qwen3.5-4b": _dense(32, 2560, 9216, 16, 4, 248320, kv=256, rope=1e7, tied=True, qk=True, arch="Qwen3_5ForCausalLM", **_gdn(16, 32)),
    "qwen3.5-9b": _dense(32, 4096, 12288, 16, 4, 248320, kv=256, rope=1e7, qk=True, arch="Qwen3_5ForCausalLM", **_gdn(16, 32)),
    "qwen3.5-27b": _dense(64, 5120, 17408, 24, 4, 248320, kv=256, rope=1e7, qk=True, arch="Qwen3_5ForCausalLM", **_gdn(16, 48)),
    "qwen3.5-35b-a3b": _dense(40, 2048, 512, 16, 2, 248320, kv=256, rope=1e7, qk=True, arch="Qwen3_5MoeForCausalLM",
                              num_experts=256, moe_ffn_hidden_size=512, moe_router_topk=8,
                              moe_shared_expert_intermediate_size=512, moe_shared_expert_gate=True, **_gdn(16, 32)),
})  # fmt: skip
# the same language model with its image / video encoder (27 blocks of width 1152, 16 x 16 pixel patches joined 2 x 2) and
# three-stream rotary positions; the placeholder token ids are the tokenizer's (a real config.json overrides them)
MORE_PRESETS["qwen3.5-35b-a3b-vl"] = dict(
    MORE_PRESETS["qwen3.5-35b-a3b"], model_arch="Qwen3_5MoeForConditionalGeneration", mrope_section=[11, 11, 10], mrope_interleaved=True,
    image_token_id=248056, video_token_id=248057,
    vision=dict(depth=27, hidden_size=1152, num_heads=16, intermediate_size=4304, in_channels=3, patch_size=16, temporal_patch_size=2,
                spatial_merge_size=2, out_hidden_size=2048, num_position_embeddings=2304, hidden_act="gelu_pytorch_tanh"))  # fmt: skip

# Qwen3-VL-8B: the Qwen3-8B language model (rotary base 5e6) with the same kind of encoder, three of whose blocks (8, 16,
# 24) also feed the first three language layers through mergers of their own
MORE_PRESETS["qwen3-vl-8b"] = dict(
    num_layers=36, hidden_size=4096, num_attention_heads=32, num_query_groups=8, kv_channels=128, ffn_hidden_size=12288,
    vocab_size=151936, tie_word_embeddings=False, qk_layernorm=True,
    model_arch="Qwen3VLForConditionalGeneration", rotary_base=5e6, mrope_section=[24, 20, 20], mrope_interleaved=True,
    image_token_id=151655, video_token_id=151656,
    vision=dict(depth=27, hidden_size=1152, num_heads=16, intermediate_size=4304, in_channels=3, patch_size=16, temporal_patch_size=2,
                spatial_merge_size=2, out_hidden_size=4096, num_position_embeddings=2304, hidden_act="gelu_pytorch_tanh",
                deepstack_visual_indexes=[8, 16, 24]))  # fmt: skip

# name -> what is missing. The numbers of these families are in the recipes they come from; they are not repeated here
# because a preset that cannot be instantiated correctly is worse than none.
UNSUPPORTED: dict[str, str] = {}

ALIASES = {"qwen2.5-0.5b": "qwen2.5-0.5b", "llama3.2-3b-instruct-amd": "llama3.2-3b-instruct"}


def to_flags(cfg) -> list[str]:
    """The preset as the command-line flags ``slime_b200.utils.arguments`` parses (Megatron names)."""
    from slime_b200.models.config import VISION_FIELDS, ModelConfig

    base = {f.name: f.default for f in dataclasses.fields(ModelConfig)}
    out: list[str] = ["--swiglu", "--normalization", "RMSNorm", "--use-rotary-position-embeddings", "--disable-bias-linear"]
    for f in dataclasses.fields(cfg):
        v = getattr(cfg, f.name)
        if f.name in ("model_arch", "padded_vocab_size", "init_method_std", "tie_word_embeddings") or v is None:
            continue
        if cfg.num_experts is None and (f.name.startswith("moe_") or f.name == "norm_topk_prob"):
            continue
        if f.name in ("rotary_scaling_factor", "mtp_num_layers", "norm_topk_prob", "rotary_percent", "linear_conv_kernel_dim",
                      "index_topk_freq", "index_skip_topk_offset", "rotary_scaling_type", "rotary_original_max_position",
                      "yarn_beta_fast", "yarn_beta_slow", "mscale", "mscale_all_dim", "rope_low_freq_factor", "rope_high_freq_factor", "index_rotary_interleaved") and v == base[f.name]:  # fmt: skip
            continue
        if f.name in VISION_FIELDS:
            continue  # no flags: the trainer reads the image encoder's description from --hf-checkpoint
        flag = "--" + f.name.replace("_", "-")
        if isinstance(v, bool):
            if v:
                out.append(flag)
        elif isinstance(v, (list, tuple)):
            out += [flag, "[" + ",".join(str(int(x)) for x in v) + "]"]
        else:
            out += [flag, str(int(v)) if isinstance(v, float) and v == int(v) else str(v)]
    if cfg.num_query_groups != cfg.num_attention_heads:
        out.append("--group-query-attention")
    if not cfg.tie_word_embeddings:
        out.append("--untie-embeddings-and-output-weights")
    return out


def main(argv=None) -> int:
    from slime_b200.models.config import PRESETS, _register_more_presets, get_preset

    _register_more_presets()
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("name", nargs="?")
    ap.add_argument("--list", action="store_true")
    a = ap.parse_args(argv)
    if a.list or not a.name:
        for n in sorted(PRESETS):
            print(f"{n:<28} {get_preset(n).num_params() / 1e9:8.2f} B parameters")
        for n, why in sorted(UNSUPPORTED.items()):
            print(f"{n:<28} unsupported: {why}")
        return 0
    try:
        print(" ".join(to_flags(get_preset(a.name))))
    except KeyError as e:
        print(str(e.args[0]), file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
