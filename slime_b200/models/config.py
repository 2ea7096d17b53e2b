"""Model architecture description shared by the trainer and the rollout engine.

Built from CLI args (Megatron flag names, cf. scripts/models/*.sh of the
reference), from a Hugging Face ``config.json``, or from a named preset.
"""

from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass


VISION_FIELDS = ("vision", "image_token_id", "video_token_id", "mrope_section", "mrope_interleaved")


@dataclass
class ModelConfig:
    num_layers: int
    hidden_size: int
    num_attention_heads: int
    num_query_groups: int
    ffn_hidden_size: int
    vocab_size: int
    kv_channels: int | None = None  # head dim
    norm_epsilon: float = 1e-6
    rotary_base: float = 10000.0
    rotary_scaling_factor: float = 1.0
    rotary_scaling_type: str = "linear"  # linear (positions divided by the factor) | llama3 | yarn
    rope_low_freq_factor: float = 1.0  # llama3: bands with a wavelength above original / low are slowed by the factor ...
    rope_high_freq_factor: float = 4.0  # ... bands below original / high are kept, the rest blend
    rotary_original_max_position: int = 4096  # yarn: the context length the frequencies were trained at
    yarn_beta_fast: float = 32.0
    yarn_beta_slow: float = 1.0
    mscale: float = 1.0
    mscale_all_dim: float = 0.0
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = True
    add_qkv_bias: bool = False
    qk_layernorm: bool = False
    post_self_attn_layernorm: bool = False  # GLM-4 sandwich norms
    post_mlp_layernorm: bool = False
    # MoE
    num_experts: int | None = None
    moe_ffn_hidden_size: int | None = None
    moe_router_topk: int = 2
    moe_router_score_function: str = "softmax"  # softmax | sigmoid
    moe_router_pre_softmax: bool = False
    moe_router_enable_expert_bias: bool = False
    moe_router_topk_scaling_factor: float | None = None
    moe_shared_expert_intermediate_size: int | None = None
    moe_shared_expert_gate: bool = False  # Qwen3-Next: the shared expert's output is scaled by sigmoid(w_g . x)
    moe_router_num_groups: int | None = None  # DeepSeek-V3: experts in groups, only the best groups are eligible
    moe_router_group_topk: int | None = None
    moe_layer_freq: int | list | None = None
    moe_aux_loss_coeff: float = 0.0
    norm_topk_prob: bool = True
    # attention variants (models/mixers.py)
    rotary_percent: float = 1.0  # fraction of the head dim that is rotated (GLM-4 family: 0.5)
    rotary_interleaved: bool = False  # rotate (2i, 2i+1) pairs instead of (i, i + d/2)
    attention_output_gate: bool = False  # Qwen3-Next: q projection carries a sigmoid gate for the attention output
    qk_layernorm_full: bool = False  # MiniMax-M2: RMSNorm over all heads of q (and of k) at once instead of per head
    softmax_sinks: bool = False  # learnable per-head sink logit in the softmax denominator
    # rotary convention of the sparse-attention indexer: None = the attention's own (``rotary_interleaved``), as the
    # reference's trainer does; DeepSeek-V3.2's released inference code rotates the indexer half-split (False)
    index_rotary_interleaved: bool | None = None
    # vision inputs (models/vision.py): the encoder's own config, the placeholder token ids, and multi-axis rotary positions
    vision: dict | None = None
    image_token_id: int | None = None
    video_token_id: int | None = None
    mrope_section: list | None = None  # rotary frequency bands per position stream (temporal, height, width)
    mrope_interleaved: bool = True  # bands of the three streams interleaved (Qwen3-VL / Qwen3.5) or one after another (Qwen2-VL)
    # gated delta-net linear attention (Qwen3-Next / Qwen3.5): layers with (i + 1) % full_attention_interval != 0
    full_attention_interval: int | None = None
    linear_num_key_heads: int | None = None
    linear_num_value_heads: int | None = None
    linear_key_head_dim: int | None = None
    linear_value_head_dim: int | None = None
    linear_conv_kernel_dim: int = 4
    # multi-head latent attention (DeepSeek-V3 / Kimi-K2 / Moonlight / GLM-5)
    multi_latent_attention: bool = False
    q_lora_rank: int | None = None
    kv_lora_rank: int | None = None
    qk_head_dim: int | None = None  # the part of a query / key head without position information
    qk_pos_emb_head_dim: int | None = None  # the rotated part, one key shared by all heads
    v_head_dim: int | None = None
    # sparse attention with a lightning indexer over MLA (GLM-5, DeepSeek-V3.2)
    index_topk: int | None = None
    index_n_heads: int | None = None
    index_head_dim: int | None = None
    index_topk_freq: int = 1  # a layer computes its own top-k when max(layer - offset, 0) % freq == 0, else reuses
    index_skip_topk_offset: int = 0
    # multi-token prediction (draft head)
    mtp_num_layers: int | None = None
    model_arch: str = "qwen2"
    padded_vocab_size: int | None = None
    init_method_std: float = 0.02

    def __post_init__(self):
        if self.kv_channels is None:
            self.kv_channels = self.hidden_size // self.num_attention_heads
        if self.padded_vocab_size is None:
            self.padded_vocab_size = self.vocab_size

    @property
    def head_dim(self) -> int:
        return self.kv_channels

    def is_moe_layer(self, layer: int) -> bool:
        if self.num_experts is None:
            return False
        f = self.moe_layer_freq
        if f is None:
            return True
        if isinstance(f, (list, tuple)):
            return bool(f[min(layer, len(f) - 1)])  # draft depths (layer >= num_layers) follow the last layer
        return layer % f == 0

    def mixer(self, layer: int) -> str:
        """Token mixer of a layer: ``attention`` (the fused kernel path), ``general_attention`` (attention variants
        composed from separate ops), ``gated_delta_net``, ``mla`` or ``dsa``."""
        if self.full_attention_interval and (layer + 1) % self.full_attention_interval != 0:
            return "gated_delta_net"
        if self.multi_latent_attention:
            return "dsa" if self.index_topk else "mla"
        if (self.rotary_percent < 1.0 or self.rotary_interleaved or self.attention_output_gate or self.qk_layernorm_full
                or self.softmax_sinks or self.mrope_section):  # fmt: skip
            return "general_attention"
        return "attention"

    def mixer_params(self, layer: int) -> int:
        h, d = self.hidden_size, self.head_dim
        kind = self.mixer(layer)
        if kind == "gated_delta_net":
            kd, vd = self.linear_num_key_heads * self.linear_key_head_dim, self.linear_num_value_heads * self.linear_value_head_dim
            return (h * (2 * kd + 2 * vd) + h * 2 * self.linear_num_value_heads + (2 * kd + vd) * self.linear_conv_kernel_dim
                    + 2 * self.linear_num_value_heads + self.linear_value_head_dim + vd * h)  # fmt: skip
        if kind in ("mla", "dsa"):
            hq, dn, dr, dv = self.num_attention_heads, self.qk_head_dim, self.qk_pos_emb_head_dim, self.v_head_dim
            q = (h * self.q_lora_rank + self.q_lora_rank + self.q_lora_rank * hq * (dn + dr)) if self.q_lora_rank else h * hq * (dn + dr)
            n = q + h * (self.kv_lora_rank + dr) + self.kv_lora_rank + self.kv_lora_rank * hq * (dn + dv) + hq * dv * h
            if kind == "dsa":
                n += self.index_n_heads * self.index_head_dim * self.q_lora_rank + self.index_head_dim * (h + 2) + self.index_n_heads * h
            return n
        n = h * d * ((2 if self.attention_output_gate else 1) * self.num_attention_heads + 2 * self.num_query_groups)
        n += self.num_attention_heads * d * h
        if self.add_qkv_bias:
            n += d * (self.num_attention_heads + 2 * self.num_query_groups)
        return n

    def num_params(self) -> int:
        h = self.hidden_size
        total = 0
        for i in range(self.num_layers):
            total += self.mixer_params(i) + 2 * h
            if self.is_moe_layer(i):
                total += self.num_experts * 3 * h * self.moe_ffn_hidden_size + self.num_experts * h
                if self.moe_shared_expert_intermediate_size:
                    total += 3 * h * self.moe_shared_expert_intermediate_size
            else:
                total += 3 * h * self.ffn_hidden_size
        total += self.vocab_size * h * (1 if self.tie_word_embeddings else 2) + h
        if self.vision:
            v = self.vision
            d, inter, big = v["hidden_size"], v["intermediate_size"], v["hidden_size"] * v.get("spatial_merge_size", 2) ** 2
            patch = v.get("in_channels", 3) * v.get("temporal_patch_size", 2) * v["patch_size"] ** 2
            total += d * patch + d + v.get("num_position_embeddings", 0) * d  # patch embedding, learned positions
            total += v["depth"] * (4 * d + 4 * d * d + 4 * d + 2 * d * inter + inter + d)  # norms, qkv + proj, mlp
            total += 2 * d + big * big + big + v.get("out_hidden_size", h) * big + v.get("out_hidden_size", h)  # merger
            # deepstack mergers: the same two linears behind a norm over the joined patches
            total += len(v.get("deepstack_visual_indexes") or []) * (2 * big + big * big + big + v.get("out_hidden_size", h) * (big + 1))
        return total

    # -- constructors ---------------------------------------------------------
    @classmethod
    def from_args(cls, args) -> "ModelConfig":
        names = {f.name for f in dataclasses.fields(cls)}
        kw = {k: getattr(args, k) for k in names if getattr(args, k, None) is not None}
        kw["tie_word_embeddings"] = not getattr(args, "untie_embeddings_and_output_weights", False)
        kw.setdefault("model_arch", getattr(args, "model_arch", None) or "qwen2")
        for req in ("num_layers", "hidden_size", "num_attention_heads", "vocab_size"):
            if req not in kw:
                raise ValueError(f"--{req.replace('_', '-')} is required (or give --hf-checkpoint with a config.json)")
        kw.setdefault("num_query_groups", kw["num_attention_heads"])
        kw.setdefault("ffn_hidden_size", 4 * kw["hidden_size"])
        # the image encoder has no flags of its own: it is described by the checkpoint's config (or the preset)
        hf = getattr(args, "hf_checkpoint", None)
        if "vision" not in kw and isinstance(hf, str) and (hf.startswith("preset:") or os.path.exists(os.path.join(hf, "config.json"))):
            try:
                src = cls.from_hf(hf)
            except (KeyError, ValueError, OSError):
                src = None
            if src is not None and src.vision is not None:
                kw.update({f: getattr(src, f) for f in VISION_FIELDS})
        return cls(**kw)

    @classmethod
    def from_hf(cls, path_or_dict) -> "ModelConfig":
        if isinstance(path_or_dict, dict):
            c = path_or_dict
        elif isinstance(path_or_dict, str) and path_or_dict.startswith("preset:"):
            return get_preset(path_or_dict[len("preset:") :])  # random-weight runs with no checkpoint directory
        else:
            with open(os.path.join(path_or_dict, "config.json")) as f:
                c = json.load(f)
        top = c
        c = c.get("text_config", c)
        arch = (c.get("architectures") or top.get("architectures") or [c.get("model_type", "qwen2")])[0]
        rp = c.get("rope_parameters") or {}
        if rp:  # newer configs keep every rotary setting in one dict
            c = {**c, **{k: v for k, v in rp.items() if k in ("rope_theta", "partial_rotary_factor")}}
        a = arch.lower()
        kw = dict(
            num_layers=c["num_hidden_layers"],
            hidden_size=c["hidden_size"],
            num_attention_heads=c["num_attention_heads"],
            num_query_groups=c.get("num_key_value_heads", c["num_attention_heads"]),
            ffn_hidden_size=c.get("intermediate_size", 4 * c["hidden_size"]),
            vocab_size=c["vocab_size"],
            kv_channels=c.get("head_dim"),
            norm_epsilon=c.get("rms_norm_eps", 1e-6),
            rotary_base=c.get("rope_theta", 10000.0),
            max_position_embeddings=c.get("max_position_embeddings", 32768),
            # a nested configuration: the output layer belongs to the outer model, whose setting decides
            tie_word_embeddings=top.get("tie_word_embeddings", c.get("tie_word_embeddings", False)) if "text_config" in top
            else c.get("tie_word_embeddings", False),
            add_qkv_bias=c.get("attention_bias", a.startswith("qwen2")),
            qk_layernorm=a.startswith("qwen3"),
            model_arch=arch,
        )
        n_experts = c.get("num_experts") or c.get("n_routed_experts") or c.get("num_local_experts")
        if n_experts:
            kw.update(
                num_experts=n_experts,
                moe_ffn_hidden_size=c.get("moe_intermediate_size") or c.get("intermediate_size"),
                moe_router_topk=c.get("num_experts_per_tok", 2),
                norm_topk_prob=c.get("norm_topk_prob", True),
            )
            if c.get("shared_expert_intermediate_size"):
                kw["moe_shared_expert_intermediate_size"] = c["shared_expert_intermediate_size"]
            if c.get("n_shared_experts"):  # DeepSeek-style: shared experts of the routed experts' width
                kw["moe_shared_expert_intermediate_size"] = c["n_shared_experts"] * c["moe_intermediate_size"]
            if c.get("first_k_dense_replace"):
                k0 = c["first_k_dense_replace"]
                kw["moe_layer_freq"] = [0] * k0 + [1] * (c["num_hidden_layers"] - k0)
            # GLM-4.5 / 4.7 / 5, DeepSeek-V3 and MiniMax-M2 always score with a sigmoid and a correction bias; configs
            # written by older tools say so (scoring_func / topk_method), newer ones leave it to the architecture
            fixed = (a.startswith("glm") and "moe" in a) or a.startswith("deepseekv3") or "minimaxm2" in a
            if c.get("scoring_func", "sigmoid" if fixed else None) == "sigmoid":
                kw.update(moe_router_score_function="sigmoid", moe_router_pre_softmax=True,
                          moe_router_enable_expert_bias=(fixed and "topk_method" not in c) or c.get("topk_method") == "noaux_tc"
                          or bool(c.get("use_routing_bias")))  # fmt: skip
            if c.get("routed_scaling_factor"):
                kw["moe_router_topk_scaling_factor"] = c["routed_scaling_factor"]
            if c.get("n_group") and c.get("topk_group") and c["n_group"] > 1:
                kw.update(moe_router_num_groups=c["n_group"], moe_router_group_topk=c["topk_group"])
            if "qwen3next" in a or "qwen3_5" in a or "qwen3_next" in a:
                kw["moe_shared_expert_gate"] = True
        if c.get("partial_rotary_factor") and c["partial_rotary_factor"] < 1.0:
            kw["rotary_percent"] = c["partial_rotary_factor"]
        elif c.get("rotary_dim") and c.get("head_dim") and c["rotary_dim"] < c["head_dim"]:
            kw["rotary_percent"] = c["rotary_dim"] / c["head_dim"]
        if a.startswith("glm4") or a.startswith("glm"):
            kw["rotary_interleaved"] = not a.startswith("glm4moe") and "moe" not in a
            kw["post_self_attn_layernorm"] = kw["post_mlp_layernorm"] = a.startswith("glm4for")
            kw["qk_layernorm"] = bool(c.get("use_qk_norm", False))
        if c.get("full_attention_interval"):  # Qwen3-Next / Qwen3.5 hybrids
            kw.update(full_attention_interval=c["full_attention_interval"], linear_num_key_heads=c["linear_num_key_heads"],
                      linear_num_value_heads=c["linear_num_value_heads"], linear_key_head_dim=c["linear_key_head_dim"],
                      linear_value_head_dim=c["linear_value_head_dim"], linear_conv_kernel_dim=c.get("linear_conv_kernel_dim", 4),
                      attention_output_gate=True, qk_layernorm=True)  # fmt: skip
        if c.get("kv_lora_rank"):
            kw.update(multi_latent_attention=True, q_lora_rank=c.get("q_lora_rank"), kv_lora_rank=c["kv_lora_rank"],
                      qk_head_dim=c["qk_nope_head_dim"], qk_pos_emb_head_dim=c["qk_rope_head_dim"], v_head_dim=c["v_head_dim"],
                      qk_layernorm=False)  # fmt: skip
            if c.get("index_topk"):
                kw.update(index_topk=c["index_topk"], index_n_heads=c["index_n_heads"], index_head_dim=c["index_head_dim"])
                if c.get("index_rope_interleave") is not None:
                    kw["index_rotary_interleaved"] = bool(c["index_rope_interleave"])
            # DeepSeek-style checkpoints rotate (2i, 2i + 1) pairs of the rotary part unless the config says otherwise
            kw["rotary_interleaved"] = bool(c.get("rope_interleave", True))
        rs = c.get("rope_scaling") or (rp if rp.get("rope_type", rp.get("type")) not in (None, "default") else {})
        if rs.get("type", rs.get("rope_type")) == "yarn":
            kw.update(rotary_scaling_type="yarn", rotary_scaling_factor=float(rs["factor"]),
                      rotary_original_max_position=int(rs.get("original_max_position_embeddings", 4096)),
                      yarn_beta_fast=float(rs.get("beta_fast", 32)), yarn_beta_slow=float(rs.get("beta_slow", 1)),
                      mscale=float(rs.get("mscale", 1.0)), mscale_all_dim=float(rs.get("mscale_all_dim", 0.0)))  # fmt: skip
        elif rs.get("type", rs.get("rope_type")) == "linear":
            kw["rotary_scaling_factor"] = float(rs["factor"])
        elif rs.get("type", rs.get("rope_type")) == "llama3":
            kw.update(rotary_scaling_type="llama3", rotary_scaling_factor=float(rs["factor"]),
                      rotary_original_max_position=int(rs.get("original_max_position_embeddings", 8192)),
                      rope_low_freq_factor=float(rs.get("low_freq_factor", 1.0)), rope_high_freq_factor=float(rs.get("high_freq_factor", 4.0)))  # fmt: skip
        if "minimax" in a:
            kw.update(qk_layernorm=False, qk_layernorm_full=bool(c.get("use_qk_norm", True)))
        section = rp.get("mrope_section") or rs.get("mrope_section")
        if top.get("vision_config") is not None:
            kw.update(vision=dict(top["vision_config"]), image_token_id=top.get("image_token_id"), video_token_id=top.get("video_token_id"))
            if section:
                kw.update(mrope_section=list(section), mrope_interleaved=bool(rp.get("mrope_interleaved", rs.get("mrope_interleaved", "qwen2" not in a))))
        return cls(**kw)

    def to_hf_dict(self) -> dict:
        moe = self.num_experts is not None
        arch = self.model_arch if self.model_arch.endswith("ForCausalLM") else {
            "qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM", "qwen3_moe": "Qwen3MoeForCausalLM",
            "llama": "LlamaForCausalLM",
        }.get(self.model_arch, "Qwen2ForCausalLM")  # fmt: skip
        d = {
            "architectures": [arch],
            "model_type": {"Qwen2ForCausalLM": "qwen2", "Qwen3ForCausalLM": "qwen3", "Qwen3MoeForCausalLM": "qwen3_moe",
                           "LlamaForCausalLM": "llama"}.get(arch, "qwen2"),
            "num_hidden_layers": self.num_layers,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_query_groups,
            "intermediate_size": self.ffn_hidden_size,
            "vocab_size": self.vocab_size,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.norm_epsilon,
            "rope_theta": self.rotary_base,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.add_qkv_bias,
            "hidden_act": "silu",
            "torch_dtype": "bfloat16",
        }  # fmt: skip
        if moe:
            d.update(num_experts=self.num_experts, moe_intermediate_size=self.moe_ffn_hidden_size,
                     num_experts_per_tok=self.moe_router_topk, norm_topk_prob=self.norm_topk_prob)  # fmt: skip
        return d


PRESETS: dict[str, dict] = {
    # Qwen2.5-0.5B: 24L, hidden 896, 14 Q / 2 KV heads x 64, FFN 4864, tied, qkv bias
    "qwen2.5-0.5b": dict(num_layers=24, hidden_size=896, num_attention_heads=14, num_query_groups=2, kv_channels=64,
                         ffn_hidden_size=4864, vocab_size=151936, rotary_base=1e6, norm_epsilon=1e-6,
                         tie_word_embeddings=True, add_qkv_bias=True, model_arch="Qwen2ForCausalLM"),
    "qwen3-0.6b": dict(num_layers=28, hidden_size=1024, num_attention_heads=16, num_query_groups=8, kv_channels=128,
                       ffn_hidden_size=3072, vocab_size=151936, rotary_base=1e6, tie_word_embeddings=True,
                       qk_layernorm=True, model_arch="Qwen3ForCausalLM"),
    "qwen3-4b": dict(num_layers=36, hidden_size=2560, num_attention_heads=32, num_query_groups=8, kv_channels=128,
                     ffn_hidden_size=9728, vocab_size=151936, rotary_base=1e6, tie_word_embeddings=True,
                     qk_layernorm=True, model_arch="Qwen3ForCausalLM"),
    "qwen3-8b": dict(num_layers=36, hidden_size=4096, num_attention_heads=32, num_query_groups=8, kv_channels=128,
                     ffn_hidden_size=12288, vocab_size=151936, rotary_base=1e6, tie_word_embeddings=False,
                     qk_layernorm=True, model_arch="Qwen3ForCausalLM"),
    "qwen3-32b": dict(num_layers=64, hidden_size=5120, num_attention_heads=64, num_query_groups=8, kv_channels=128,
                      ffn_hidden_size=25600, vocab_size=151936, rotary_base=1e6, tie_word_embeddings=False,
                      qk_layernorm=True, model_arch="Qwen3ForCausalLM"),
    "qwen3-30b-a3b": dict(num_layers=48, hidden_size=2048, num_attention_heads=32, num_query_groups=4, kv_channels=128,
                          ffn_hidden_size=6144, vocab_size=151936, rotary_base=1e6, tie_word_embeddings=False,
                          qk_layernorm=True, num_experts=128, moe_ffn_hidden_size=768, moe_router_topk=8,
                          model_arch="Qwen3MoeForCausalLM"),
    "llama-3.2-1b": dict(num_layers=16, hidden_size=2048, num_attention_heads=32, num_query_groups=8, kv_channels=64,
                         ffn_hidden_size=8192, vocab_size=128256, rotary_base=5e5, tie_word_embeddings=True,
                         model_arch="LlamaForCausalLM"),
    "glm4-9b": dict(num_layers=40, hidden_size=4096, num_attention_heads=32, num_query_groups=2, kv_channels=128,
                    ffn_hidden_size=13696, vocab_size=151552, rotary_base=1e4, tie_word_embeddings=False,
                    add_qkv_bias=True, post_self_attn_layernorm=True, post_mlp_layernorm=True, norm_epsilon=1e-5,
                    rotary_percent=0.5, rotary_interleaved=True, model_arch="Glm4ForCausalLM"),
    "tiny": dict(num_layers=2, hidden_size=128, num_attention_heads=4, num_query_groups=2, kv_channels=64,
                 ffn_hidden_size=256, vocab_size=512, rotary_base=1e4, tie_word_embeddings=True, add_qkv_bias=True,
                 model_arch="Qwen2ForCausalLM"),
    "tiny-moe": dict(num_layers=2, hidden_size=128, num_attention_heads=4, num_query_groups=2, kv_channels=64,
                     ffn_hidden_size=256, vocab_size=512, rotary_base=1e4, tie_word_embeddings=False,
                     qk_layernorm=True, num_experts=8, moe_ffn_hidden_size=64, moe_router_topk=2,
                     model_arch="Qwen3MoeForCausalLM"),
}  # fmt: skip


def _register_more_presets() -> None:
    from slime_b200.models import presets as more

    for k, v in more.MORE_PRESETS.items():
        PRESETS.setdefault(k, v)


def get_preset(name: str) -> ModelConfig:
    from slime_b200.models import presets as more

    _register_more_presets()
    key = name.lower()
    key = more.ALIASES.get(key, key)
    if key in more.UNSUPPORTED:
        raise KeyError(f"model preset {name!r} is not supported: {more.UNSUPPORTED[key]}")
    if key not in PRESETS:
        raise KeyError(f"unknown model preset {name!r}; known: {sorted(PRESETS)}")
    return ModelConfig(**PRESETS[key])


def apply_to_args(cfg: ModelConfig, args) -> None:
    """Copy the architecture into an args namespace under the Megatron flag names."""
    for f in dataclasses.fields(cfg):
        setattr(args, f.name, getattr(cfg, f.name))
    args.untie_embeddings_and_output_weights = not cfg.tie_word_embeddings
    args.swiglu = True
