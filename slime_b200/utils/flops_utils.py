"""Analytic forward-FLOPs model used for TFLOPs logging and FLOPs-balanced packing.

Parity: slime/utils/flops_utils.py:74-135 (dense + MoE layer mix, LM head).
The attention term is the full (non-causal) ``4*s^2*h*d`` count, as in the
reference, so logged TFLOPs are comparable.
"""

from __future__ import annotations


def _head_dim(args) -> int:
    kv = getattr(args, "kv_channels", None)
    return kv if kv else args.hidden_size // args.num_attention_heads


def attention_block_flops(args, s: int) -> int:
    h, nq = args.hidden_size, args.num_attention_heads
    nkv = getattr(args, "num_query_groups", None) or nq
    d = _head_dim(args)
    qkv = 2 * s * h * d * (nq + 2 * nkv)
    scores_and_mix = 4 * s * s * nq * d
    out = 2 * s * nq * d * h
    return qkv + scores_and_mix + out


def mlp_flops(s: int, h: int, ffn: int) -> int:
    return 6 * s * h * ffn  # gate, up, down


def lm_head_flops(s: int, h: int, vocab: int) -> int:
    return 2 * s * h * vocab


def layer_mix(args) -> tuple[int, int]:
    """(dense layers, moe layers) according to ``num_experts`` / ``moe_layer_freq``."""
    L = args.num_layers
    if getattr(args, "num_experts", None) is None:
        return L, 0
    freq = getattr(args, "moe_layer_freq", None)
    if freq is None:
        return 0, L
    if isinstance(freq, (list, tuple)):
        moe = sum(1 for f in freq if f > 0)
        return len(freq) - moe, moe
    moe = sum(1 for i in range(L) if i % freq == 0)
    return L - moe, moe


def calculate_fwd_flops(seqlens, args) -> int:
    dense_layers, moe_layers = layer_mix(args)
    h = args.hidden_size
    moe_ffn = 0
    if moe_layers:
        shared = getattr(args, "moe_shared_expert_intermediate_size", None) or 0
        moe_ffn = args.moe_ffn_hidden_size * args.moe_router_topk + shared
    total = 0
    for s in seqlens:
        attn = attention_block_flops(args, s)
        if dense_layers:
            total += dense_layers * (attn + mlp_flops(s, h, args.ffn_hidden_size))
        if moe_layers:
            total += moe_layers * (attn + mlp_flops(s, h, moe_ffn))
        total += lm_head_flops(s, h, args.vocab_size)
    return total


def calculate_fwd_bwd_flops(seqlens, args) -> int:
    return 3 * calculate_fwd_flops(seqlens, args)
