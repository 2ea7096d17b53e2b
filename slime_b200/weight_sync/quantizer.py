"""Quantise HF-named tensors on their way to the rollout engine.

FP8: 128x128 (``weight_block_size``) block-scaled e4m3 with fp32 ``<w>_scale_inv`` (optionally
power-of-two scales for the UE8M0 GEMM format), per-tensor otherwise; applied only to attention /
MLP / expert / MLA / indexer projections. INT4: compressed-tensors W4A16 packing of a fake-quantised
weight. Parity: slime/backends/megatron_utils/megatron_to_hf/processors/quantizer_fp8.py:10-118,
quantizer_compressed_tensors.py:21-297, padding_remover.py.
"""

from __future__ import annotations

import re

import torch

from slime_b200 import ops

_QUANT_TARGETS = re.compile(
    r"(self_attn\.(q_proj|k_proj|v_proj|o_proj|qkv_proj|q_a_proj|q_b_proj|kv_a_proj_with_mqa|kv_b_proj|wq_b|wk)|"
    r"mlp\.(gate_proj|up_proj|down_proj|gate_up_proj)|"
    r"mlp\.experts\.\d+\.(gate_proj|up_proj|down_proj)|mlp\.shared_experts?\.(gate_proj|up_proj|down_proj)|"
    r"indexer\.(wq_b|wk))\.weight$"
)


def should_quantize(hf_name: str) -> bool:
    return _QUANT_TARGETS.search(hf_name) is not None


def quantize_param_fp8(name: str, weight: torch.Tensor, block_size, pow2_scale: bool = False):
    assert name.endswith(".weight"), name
    if block_size is not None:
        q, s = ops.block_fp8_quant(weight.to(torch.bfloat16), tuple(block_size), pow2_scale)
        return [(name, q), (name.replace(".weight", ".weight_scale_inv"), s)]
    amax = weight.abs().max().clamp(min=1e-12).float()
    scale = amax / 448.0
    q = (weight.float() / scale).clamp(-448, 448).to(torch.float8_e4m3fn)
    return [(name, q), (name.replace(".weight", ".weight_scale"), scale.view(1))]


def pack_int4(q: torch.Tensor) -> torch.Tensor:
    """Pack int4 code values (int8 tensor in [-8, 7], last dim % 8 == 0) into int32, 8 per word,
    compressed-tensors order (element i at bits [4i, 4i+4) with an offset of 8)."""
    u = (q.to(torch.int32) + 8) & 0xF
    u = u.reshape(*q.shape[:-1], q.shape[-1] // 8, 8)
    shifts = torch.arange(0, 32, 4, device=q.device, dtype=torch.int32)
    return (u << shifts).sum(-1).to(torch.int32)


def quantize_param_int4(name: str, weight: torch.Tensor, group_size: int = 32):
    y, s, _z = ops.fake_int4_quant(weight.to(torch.bfloat16).contiguous(), (1, group_size), True)
    codes = torch.round(y.float().view(weight.shape[0], -1, group_size) / s[..., None]).clamp(-8, 7).to(torch.int8)
    packed = pack_int4(codes.view(weight.shape))
    base = name[: -len(".weight")]
    return [(f"{base}.weight_packed", packed), (f"{base}.weight_scale", s.to(torch.bfloat16)),
            (f"{base}.weight_shape", torch.tensor(list(weight.shape), dtype=torch.int64))]  # fmt: skip


def remove_padding(name: str, t: torch.Tensor, vocab_size: int) -> torch.Tensor:
    if name in ("model.embed_tokens.weight", "lm_head.weight"):
        return t[:vocab_size]
    return t


def quantize_params(args, trainer_name: str, pairs, quantization_config):
    if not quantization_config:
        return pairs
    method = quantization_config.get("quant_method")
    out = []
    for name, t in pairs:
        if not should_quantize(name):
            out.append((name, t))
        elif method == "fp8":
            fmt = quantization_config.get("scale_fmt") == "ue8m0"
            out += quantize_param_fp8(name, t, quantization_config.get("weight_block_size"), pow2_scale=fmt)
        elif method == "compressed-tensors":
            groups = quantization_config.get("config_groups", {}).get("group_0", {}).get("weights", {})
            out += quantize_param_int4(name, t, groups.get("group_size", 32))
        else:
            raise ValueError(f"unsupported quant_method {method!r}")
    return out
