"""Block-fp8 rollout engine (CPU reference ops): resident e4m3 buffers, online and pre-quantised loading, expert stacks."""

import numpy as np
import pytest
import torch

from slime_b200.engine.engine import Engine
from slime_b200.engine.quant import Fp8Weight
from slime_b200.engine.server_args import ServerArgs
from slime_b200.models.config import ModelConfig, get_preset
from slime_b200.weight_sync.quantizer import quantize_param_fp8, should_quantize


def hf_weights(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    mat = lambda *s, std=0.05: (torch.randn(*s, generator=g) * std).to(torch.bfloat16).float()  # noqa: E731
    h, d, nq, nkv, f = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_query_groups, cfg.ffn_hidden_size
    out = [("model.embed_tokens.weight", mat(cfg.vocab_size, h, std=0.5)), ("model.norm.weight", 1 + mat(h)),
           ("lm_head.weight", mat(cfg.vocab_size, h, std=0.5))]  # fmt: skip
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        out += [(p + "input_layernorm.weight", 1 + mat(h)), (p + "post_attention_layernorm.weight", 1 + mat(h)),
                (p + "self_attn.q_proj.weight", mat(nq * d, h)), (p + "self_attn.k_proj.weight", mat(nkv * d, h)),
                (p + "self_attn.v_proj.weight", mat(nkv * d, h)), (p + "self_attn.o_proj.weight", mat(h, nq * d))]  # fmt: skip
        if cfg.is_moe_layer(i):
            fe = cfg.moe_ffn_hidden_size
            out.append((p + "mlp.gate.weight", mat(cfg.num_experts, h, std=0.5)))
            for e in range(cfg.num_experts):
                out += [(p + f"mlp.experts.{e}.gate_proj.weight", mat(fe, h)), (p + f"mlp.experts.{e}.up_proj.weight", mat(fe, h)),
                        (p + f"mlp.experts.{e}.down_proj.weight", mat(h, fe))]  # fmt: skip
        else:
            out += [(p + "mlp.gate_proj.weight", mat(f, h)), (p + "mlp.up_proj.weight", mat(f, h)), (p + "mlp.down_proj.weight", mat(h, f))]
    return out


CFG = ModelConfig(num_layers=2, hidden_size=128, num_attention_heads=4, num_query_groups=2, kv_channels=64, ffn_hidden_size=256,
                  vocab_size=512, rotary_base=1e4, tie_word_embeddings=False)  # fmt: skip
MOE = ModelConfig(num_layers=2, hidden_size=128, num_attention_heads=4, num_query_groups=2, kv_channels=64, ffn_hidden_size=256,
                  vocab_size=512, rotary_base=1e4, tie_word_embeddings=False, num_experts=4, moe_ffn_hidden_size=128,
                  moe_router_topk=2)  # fmt: skip


def engine(cfg, quantization):
    return Engine(cfg, ServerArgs(page_size=4, max_running_requests=4, context_length=64, disable_cuda_graph=True,
                                  quantization=quantization), device="cpu", num_pages=64)  # fmt: skip


def score(e, ids, n_prompt):
    rq = e.generate([ids], [dict(max_new_tokens=0)], logprob_start_len=0)[0]
    return np.array(rq.input_logprobs[n_prompt:])


@pytest.mark.parametrize("cfg", [CFG, MOE], ids=["dense", "moe"])
def test_fp8_engine_tracks_the_bf16_engine_and_accepts_prequantised_weights(cfg):
    weights = hf_weights(cfg)
    full, q8 = engine(cfg, None), engine(cfg, "fp8")
    assert not full.weights.load_weights(weights) and not q8.weights.load_weights(weights)
    L = q8.weights.layers[0]
    assert all(isinstance(L[k], Fp8Weight) for k in ("qkv", "o")) and isinstance(L.get("gate_up", L.get("w13")), Fp8Weight)
    assert q8.weights.num_bytes() < full.weights.num_bytes()  # matrices at one byte per element plus scales
    # the quantised buffers reproduce the weights to e4m3 accuracy (3 mantissa bits: 2^-4 relative per element, block-scaled)
    ref_qkv = torch.cat([dict(weights)[f"model.layers.0.self_attn.{n}_proj.weight"] for n in "qkv"])
    assert (L["qkv"].dequant(torch.float32) - ref_qkv).abs().max() <= ref_qkv.abs().max() / 16 + 1e-6
    r = full.generate([[1, 2, 3, 4, 5, 6]], [dict(max_new_tokens=8, ignore_eos=True, temperature=0)])[0]
    ids = r.input_ids + r.output_ids
    a, b = score(full, ids, 6), score(q8, ids, 6)
    # W8A8 on random weights with a wide embedding: a few tenths of a nat at worst, no systematic shift
    assert np.abs(a - b).max() < 0.5 and np.abs(a - b).mean() < 0.15 and abs((a - b).mean()) < 0.1, (a, b)
    # the sender quantises (fp8 weight sync): bytes and scales arrive under the checkpoint names, in any order
    sent = []
    for name, t in weights:
        sent += quantize_param_fp8(name, t, (128, 128)) if should_quantize(name) else [(name, t)]
    sent = sent[::-1]
    q8b = engine(cfg, "fp8")
    assert not q8b.weights.load_weights(sent)
    for La, Lb in zip(q8.weights.layers, q8b.weights.layers):
        for k, v in La.items():
            if isinstance(v, Fp8Weight):
                assert torch.equal(v.q.view(torch.uint8), Lb[k].q.view(torch.uint8)) and torch.equal(v.scale, Lb[k].scale), k
    assert np.array_equal(score(q8b, ids, 6), b)
    # quantised tensors sent to an engine that keeps bf16 are refused, not misread
    with pytest.raises(ValueError, match="block-fp8 weights were sent"):
        engine(cfg, None).weights.load_weights(sent)


def test_unaligned_shapes_stay_in_bf16():
    cfg = get_preset("tiny-moe")  # expert width 64: gate / up halves would share a scale block
    e = engine(cfg, "fp8")
    L = e.weights.layers[0]
    assert isinstance(L["w13"], torch.Tensor) and isinstance(L["w2"], torch.Tensor) and isinstance(L["qkv"], Fp8Weight)
    e.weights.init_random(0, std=0.2)
    r = e.generate([[1, 2, 3]], [dict(max_new_tokens=4, ignore_eos=True)])[0]
    assert len(r.output_ids) == 4
