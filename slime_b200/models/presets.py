"""Architecture presets for the model families the launch recipes name, and a CLI that prints them as flags.

    python -m slime_b200.models.presets --list
    python -m slime_b200.models.presets qwen3-4B            # -> "--num-layers 36 --hidden-size 2560 ..." (one line)
    MODEL_ARGS=($(python -m slime_b200.models.presets qwen3-30B-A3B))   # in a launch script

Every entry is the constructor arguments of ``ModelConfig``; ``--hf-checkpoint preset:<name>`` builds a random-weight
model from it, and a real checkpoint's ``config.json`` overrides nothing here (it is read instead). Families whose layers
this framework does not implement yet (multi-head latent attention, gated delta-net hybrids, sparse-attention
indexers) are listed in ``UNSUPPORTED`` with the missing piece, so asking for one fails with a reason instead of a
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
                                   rotary_scaling_factor=8.0, max_position_embeddings=131072),
    "llama3.2-3b-instruct": _dense(28, 3072, 8192, 24, 8, 128256, kv=128, rope=5e5, eps=1e-5, tied=True,
                                   arch="LlamaForCausalLM", rotary_scaling_factor=32.0, max_position_embeddings=131072),
    "mimo-7b-rl": _dense(36, 4096, 11008, 32, 8, 151680, rope=6.4e5, eps=1e-5, bias=True, mtp_num_layers=1,
                         arch="MiMoForCausalLM"),
    "qwen3-235b-a22b": _moe(0, 94, **_dense(94, 4096, 12288, 64, 4, 151936, kv=128, qk=True, arch="Qwen3MoeForCausalLM",
                                            num_experts=128, moe_ffn_hidden_size=1536, moe_router_topk=8)),
}  # fmt: skip

# name -> what is missing. The numbers of these families are in the recipes they come from; they are not repeated here
# because a preset that cannot be instantiated correctly is worse than none.
UNSUPPORTED: dict[str, str] = {
    "glm4-32b": "partial rotary (rotary_percent 0.5, interleaved) is not implemented in the rope kernel",
    "glm4.5-106b-a12b": "partial rotary (rotary_percent 0.5) and sequence-level aux loss are not implemented",
    "glm4.5-355b-a32b": "partial rotary (rotary_percent 0.5) and sequence-level aux loss are not implemented",
    "glm4.7-30b-a3b": "partial rotary (rotary_percent 0.5) and sequence-level aux loss are not implemented",
    "deepseek-v3": "multi-head latent attention (MLA) is not implemented",
    "deepseek-v3-5layer": "multi-head latent attention (MLA) is not implemented",
    "deepseek-v3-20layer": "multi-head latent attention (MLA) is not implemented",
    "kimi-k2": "multi-head latent attention (MLA) is not implemented",
    "kimi-k2-thinking": "multi-head latent attention (MLA) is not implemented",
    "moonlight": "multi-head latent attention (MLA) is not implemented",
    "glm5-744b-a40b": "sparse attention with a lightning indexer (DSA) over MLA is not implemented",
    "glm5.2-744b-a40b": "sparse attention with a lightning indexer (DSA) over MLA is not implemented",
    "minimax-m2": "per-layer qk-norm over the full projection and its router variant are not implemented",
    "qwen3-next-80b-a3b": "gated delta-net linear-attention layers are not implemented",
    "qwen3.5-0.8b": "gated delta-net linear-attention layers are not implemented",
    "qwen3.5-4b": "gated delta-net linear-attention layers are not implemented",
    "qwen3.5-9b": "gated delta-net linear-attention layers are not implemented",
    "qwen3.5-27b": "gated delta-net linear-attention layers are not implemented",
    "qwen3.5-35b-a3b": "gated delta-net linear-attention layers are not implemented",
    "qwen3.5-35b-a3b-vl": "gated delta-net layers and the vision tower are not implemented",
}

ALIASES = {"qwen2.5-0.5b": "qwen2.5-0.5b", "llama3.2-3b-instruct-amd": "llama3.2-3b-instruct"}


def to_flags(cfg) -> list[str]:
    """The preset as the command-line flags ``slime_b200.utils.arguments`` parses (Megatron names)."""
    from slime_b200.models.config import ModelConfig

    base = {f.name: f.default for f in dataclasses.fields(ModelConfig)}
    out: list[str] = ["--swiglu", "--normalization", "RMSNorm", "--use-rotary-position-embeddings", "--disable-bias-linear"]
    for f in dataclasses.fields(cfg):
        v = getattr(cfg, f.name)
        if f.name in ("model_arch", "padded_vocab_size", "init_method_std", "tie_word_embeddings") or v is None:
            continue
        if cfg.num_experts is None and (f.name.startswith("moe_") or f.name == "norm_topk_prob"):
            continue
        if f.name in ("rotary_scaling_factor", "mtp_num_layers", "norm_topk_prob") and v == base[f.name]:
            continue
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
