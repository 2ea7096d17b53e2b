"""Token mixers (models/mixers.py) on CPU: each against an independent, slower statement of its definition."""

import math

import pytest
import torch
import torch.nn.functional as F

from slime_b200.models import mixers
from slime_b200.models.config import ModelConfig
from slime_b200.models.gpt import GPTModel, PackedSeqParams


def packed_for(lens, pad_to=None):
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens])
    if pad_to and T % pad_to:
        pad = pad_to - T % pad_to
        cu.append(T + pad)
        pos = torch.cat([pos, torch.arange(pad, dtype=torch.int32)])
    p = PackedSeqParams(torch.tensor(cu, dtype=torch.int32), max(lens), pos)
    return p, pos.numel()


def test_chunked_gated_delta_rule_matches_the_recurrence_with_gradients():
    torch.manual_seed(0)
    lens, H, Dk, Dv = [70, 5, 129], 3, 8, 12
    T = sum(lens)
    cu = torch.tensor([0, 70, 75, 204], dtype=torch.int32)
    mk = lambda *s: torch.randn(*s, dtype=torch.float64).float().requires_grad_()  # noqa: E731
    q, k, v = mk(T, H, Dk), mk(T, H, Dk), mk(T, H, Dv)
    g = (-torch.rand(T, H) * 0.5).requires_grad_()
    beta = torch.rand(T, H).requires_grad_()
    ref = mixers.gated_delta_rule_recurrent(q, k, v, g, beta, cu)
    for chunk in (16, 64):
        out = mixers.gated_delta_rule_chunked(q, k, v, g, beta, cu, chunk=chunk)
        assert torch.allclose(out, ref, atol=2e-5, rtol=1e-4), float((out - ref).abs().max())
    w = torch.randn_like(ref)
    grads_ref = torch.autograd.grad((ref * w).sum(), [q, k, v, g, beta])
    grads = torch.autograd.grad((mixers.gated_delta_rule_chunked(q, k, v, g, beta, cu, chunk=32) * w).sum(), [q, k, v, g, beta])
    for a, b in zip(grads, grads_ref):
        assert torch.allclose(a, b, atol=5e-4, rtol=1e-3), float((a - b).abs().max())


def test_short_conv_restarts_at_every_sequence():
    torch.manual_seed(1)
    lens, C, K = [5, 1, 7], 6, 4
    p, T = packed_for(lens)
    x, w = torch.randn(T, C), torch.randn(C, K)
    got = mixers.causal_short_conv(x, w, p.position_ids)
    off = 0
    for n in lens:
        seq = x[off : off + n].t()[None]  # [1, C, n]
        ref = F.silu(F.conv1d(F.pad(seq, (K - 1, 0)), w[:, None, :], groups=C))[0].t()
        assert torch.allclose(got[off : off + n], ref, atol=1e-6)
        off += n


def test_partial_and_interleaved_rotary():
    from slime_b200 import ops

    T, H, D, rot = 9, 2, 16, 8
    x = torch.randn(T, H, D)
    pos = torch.arange(T)
    table = ops.rope_cos_sin(32, rot, 1e4)
    cos, sin = mixers.rotary_cos_sin(table, pos)
    y = mixers.apply_rotary(x, cos, sin)
    assert torch.equal(y[..., rot:], x[..., rot:])  # pass-through part
    inv = 1.0 / (1e4 ** (torch.arange(0, rot, 2).float() / rot))
    ang = pos[:, None].float() * inv[None]
    x1, x2 = x[..., : rot // 2], x[..., rot // 2 : rot]
    assert torch.allclose(y[..., : rot // 2], x1 * ang.cos()[:, None] - x2 * ang.sin()[:, None], atol=1e-5)
    yi = mixers.apply_rotary(x, cos, sin, interleaved=True)
    a, b = x[..., 0:rot:2], x[..., 1:rot:2]
    assert torch.allclose(yi[..., 0:rot:2], a * ang.cos()[:, None] - b * ang.sin()[:, None], atol=1e-5)
    assert torch.allclose(yi[..., 1:rot:2], b * ang.cos()[:, None] + a * ang.sin()[:, None], atol=1e-5)
    # norms are preserved by a rotation
    assert torch.allclose(yi.norm(dim=-1), x.norm(dim=-1), atol=1e-5)


def test_softmax_sinks_match_an_explicit_extra_column_and_train():
    from slime_b200.ops import attention

    torch.manual_seed(2)
    T, Hq, Hkv, D = 11, 4, 2, 8
    q, k, v = torch.randn(T, Hq, D), torch.randn(T, Hkv, D), torch.randn(T, Hkv, D)
    sinks = torch.randn(Hq, requires_grad=True)
    seg = attention.segments_from_cu_seqlens(torch.tensor([0, 4, 11], dtype=torch.int32))
    out = attention.segment_attention(q, k, v, seg, 0.3, sinks=sinks)
    # explicit: a zero-valued key whose logit is the sink
    ref = torch.zeros_like(out)
    for a, b in ((0, 4), (4, 11)):
        for h in range(Hq):
            s = (q[a:b, h] @ k[a:b, h // 2].t()) * 0.3
            s = s.masked_fill(~torch.ones(b - a, b - a, dtype=torch.bool).tril(), float("-inf"))
            p = torch.cat([s, sinks[h].expand(b - a, 1)], -1).softmax(-1)
            ref[a:b, h] = p[:, :-1] @ v[a:b, h // 2]
    assert torch.allclose(out, ref, atol=1e-5)
    # the gate form used on the GPU path: plain attention times sigmoid(lse - sink)
    plain = attention.segment_attention(q, k, v, seg, 0.3)
    lse = torch.stack([torch.cat([torch.logsumexp(((q[a:b, h] @ k[a:b, h // 2].t()) * 0.3).masked_fill(
        ~torch.ones(b - a, b - a, dtype=torch.bool).tril(), float("-inf")), -1) for a, b in ((0, 4), (4, 11))]) for h in range(Hq)])
    assert torch.allclose(out, plain * torch.sigmoid(lse - sinks[:, None]).t()[:, :, None], atol=1e-5)
    out.sum().backward()
    assert sinks.grad is not None and float(sinks.grad.abs().sum()) > 0


def _tiny(**kw):
    base = dict(num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=2, kv_channels=16, ffn_hidden_size=128,
                vocab_size=256, rotary_base=1e4, tie_word_embeddings=False)  # fmt: skip
    base.update(kw)
    return ModelConfig(**base)


@pytest.mark.parametrize("kw,kinds", [
    (dict(rotary_percent=0.5, rotary_interleaved=True, post_self_attn_layernorm=True, post_mlp_layernorm=True), ["general_attention"] * 2),
    (dict(qk_layernorm_full=True, softmax_sinks=True), ["general_attention"] * 2),
    (dict(num_layers=4, full_attention_interval=4, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=8,
          linear_value_head_dim=8, attention_output_gate=True, qk_layernorm=True, rotary_percent=0.25),
     ["gated_delta_net"] * 3 + ["general_attention"]),
    (dict(multi_latent_attention=True, q_lora_rank=24, kv_lora_rank=16, qk_head_dim=8, qk_pos_emb_head_dim=4, v_head_dim=8), ["mla"] * 2),
    (dict(num_layers=3, multi_latent_attention=True, q_lora_rank=24, kv_lora_rank=16, qk_head_dim=8, qk_pos_emb_head_dim=4,
          v_head_dim=8, index_topk=4, index_n_heads=2, index_head_dim=8, index_topk_freq=2, index_skip_topk_offset=1), ["dsa"] * 3),
], ids=["glm4_partial_rotary", "minimax_full_norm_sinks", "qwen3_next_hybrid", "mla", "dsa_shared_topk"])  # fmt: skip
def test_models_with_each_mixer_are_causal_packed_and_trainable(kw, kinds):
    """Whole model per family: the layer kinds are as configured; logits of a token do not depend on later tokens or on
    the other sequences of the pack; every parameter receives a gradient (indexer weights excepted: the choice they
    make is discrete)."""
    torch.manual_seed(0)
    cfg = _tiny(**kw)
    assert [cfg.mixer(i) for i in range(cfg.num_layers)] == kinds
    model = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=1)
    lens = [9, 6]
    ids = torch.randint(0, cfg.vocab_size, (sum(lens),))
    p, T = packed_for(lens)
    logits = model(ids, position_ids=p.position_ids, packed_seq_params=p)[0]
    assert logits.shape == (T, cfg.vocab_size) and torch.isfinite(logits).all()
    # sequence 1 alone gives the same logits; changing its last token leaves earlier rows alone
    p1, _ = packed_for([9])
    alone = model(ids[:9], position_ids=p1.position_ids, packed_seq_params=p1)[0]
    assert torch.allclose(alone, logits[:9], atol=1e-4), float((alone - logits[:9]).abs().max())
    ids2 = ids.clone()
    ids2[8] = (ids2[8] + 1) % cfg.vocab_size
    p, _ = packed_for(lens)
    moved = model(ids2, position_ids=p.position_ids, packed_seq_params=p)[0]
    assert torch.allclose(moved[:8], logits[:8], atol=1e-5) and torch.allclose(moved[9:], logits[9:], atol=1e-5)
    assert not torch.allclose(moved[8], logits[8], atol=1e-5)
    p, _ = packed_for(lens)
    model(ids, position_ids=p.position_ids, packed_seq_params=p)[0].logsumexp(-1).sum().backward()
    missing = [n for n, q in model.named_parameters() if q.grad is None or float(q.grad.abs().sum()) == 0]
    assert all(any(t in n for t in ("wq_b", "wk.", "k_norm", "weights_proj")) for n in missing), missing


def test_dsa_restricts_attention_to_the_indexers_choice():
    torch.manual_seed(3)
    cfg = _tiny(num_layers=1, multi_latent_attention=True, q_lora_rank=24, kv_lora_rank=16, qk_head_dim=8, qk_pos_emb_head_dim=4,
                v_head_dim=8, index_topk=3, index_n_heads=2, index_head_dim=8)  # fmt: skip
    layer = mixers.DSASelfAttention(cfg, 0, torch.float32, "cpu", False)
    p, T = packed_for([10, 4])
    x = torch.randn(T, cfg.hidden_size)
    out, _ = layer(x, None, None, p)
    allowed = getattr(p, layer._HOLDER)[0]
    assert allowed.shape == (T, 10)
    counts = allowed.sum(-1)
    # rows with at most top-k visible keys keep all of them, the others exactly top-k, never a future key
    assert counts[:3].tolist() == [1, 2, 3] and (counts[3:10] == 3).all() and counts[10:].tolist() == [1, 2, 3, 3]
    assert not allowed[:10].triu(1).any()
    # with top-k >= sequence length the layer is plain latent attention
    cfg_all = ModelConfig(**{**cfg.__dict__, "index_topk": 64})
    dense = mixers.MLASelfAttention(cfg_all, 0, torch.float32, "cpu", False)
    sparse = mixers.DSASelfAttention(cfg_all, 0, torch.float32, "cpu", False)
    sparse.load_state_dict(dense.state_dict(), strict=False)
    p1, _ = packed_for([10, 4])
    p2, _ = packed_for([10, 4])
    assert torch.allclose(dense(x, None, None, p1)[0], sparse(x, None, None, p2)[0], atol=1e-6)


def test_indexer_logits_definition():
    q, k, w = torch.randn(5, 3, 4), torch.randn(7, 4), torch.randn(5, 3)
    ref = torch.zeros(5, 7)
    for t in range(5):
        for s in range(7):
            ref[t, s] = sum(float(w[t, h]) * max(float(q[t, h] @ k[s]), 0.0) for h in range(3))
    assert torch.allclose(mixers.indexer_logits(q, k, w), ref, atol=1e-5)
    assert math.isfinite(float(ref.sum()))


@pytest.mark.parametrize("kw,arch", [
    (dict(rotary_percent=0.5, rotary_interleaved=True, post_self_attn_layernorm=True, post_mlp_layernorm=True), "Glm4ForCausalLM"),
    (dict(qk_layernorm_full=True, softmax_sinks=True), "MiniMaxM2ForCausalLM"),
    (dict(num_layers=4, full_attention_interval=4, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=8,
          linear_value_head_dim=8, attention_output_gate=True, qk_layernorm=True, rotary_percent=0.25, num_experts=4,
          moe_ffn_hidden_size=32, moe_router_topk=2, moe_shared_expert_intermediate_size=32, moe_shared_expert_gate=True),
     "Qwen3NextForCausalLM"),
    (dict(num_layers=4, full_attention_interval=2, linear_num_key_heads=2, linear_num_value_heads=2, linear_key_head_dim=8,
          linear_value_head_dim=8, attention_output_gate=True, qk_layernorm=True, rotary_percent=0.25), "Qwen3_5ForCausalLM"),
    (dict(multi_latent_attention=True, q_lora_rank=24, kv_lora_rank=16, qk_head_dim=8, qk_pos_emb_head_dim=4, v_head_dim=8,
          num_experts=4, moe_ffn_hidden_size=32, moe_router_topk=2, moe_layer_freq=[0, 1], moe_shared_expert_intermediate_size=32,
          moe_router_score_function="sigmoid", moe_router_enable_expert_bias=True), "DeepseekV3ForCausalLM"),
    (dict(multi_latent_attention=True, q_lora_rank=24, kv_lora_rank=16, qk_head_dim=8, qk_pos_emb_head_dim=4, v_head_dim=8,
          index_topk=4, index_n_heads=2, index_head_dim=8), "GlmMoeDsaForCausalLM"),
], ids=["glm4", "minimax_m2", "qwen3_next", "qwen3_5", "deepseek_v3", "glm5_dsa"])  # fmt: skip
def test_checkpoint_names_round_trip_for_each_family(kw, arch):
    """Every trainer parameter maps to checkpoint names and back to the same tensor (names follow the public
    checkpoints of each family; zero-centred norms and the per-head (query, gate) rows are translated)."""
    from slime_b200.weight_sync import convert

    torch.manual_seed(0)
    cfg = _tiny(model_arch=arch, **kw)
    model = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=3)
    hf = {}
    for name, p in model.named_parameters():
        for hf_name, t in convert.convert_to_hf(cfg, name, p.detach().clone()):
            assert hf_name not in hf, hf_name
            hf[hf_name] = t
    # spot checks of the public naming
    names = set(hf)
    if arch == "Qwen3NextForCausalLM":
        assert "model.layers.0.linear_attn.in_proj_qkvz.weight" in names and hf["model.layers.0.linear_attn.conv1d.weight"].dim() == 3
        assert hf["model.layers.3.self_attn.q_proj.weight"].shape[0] == 2 * cfg.num_attention_heads * cfg.head_dim
        ln = dict(model.named_parameters())["decoder.layers.0.self_attention.input_layernorm.weight"]
        assert torch.allclose(hf["model.layers.0.input_layernorm.weight"], ln - 1)  # stored zero-centred
        assert torch.allclose(hf["model.layers.0.linear_attn.norm.weight"], torch.ones(8))  # the gated norm is not
    if arch == "Qwen3_5ForCausalLM":
        assert {"model.layers.0.linear_attn.in_proj_qkv.weight", "model.layers.0.linear_attn.in_proj_z.weight",
                "model.layers.0.linear_attn.in_proj_a.weight"} <= names  # fmt: skip
    if arch == "DeepseekV3ForCausalLM":
        assert {"model.layers.0.self_attn.q_a_proj.weight", "model.layers.0.self_attn.q_a_layernorm.weight",
                "model.layers.0.self_attn.kv_a_proj_with_mqa.weight", "model.layers.1.mlp.shared_experts.down_proj.weight",
                "model.layers.1.mlp.experts.3.up_proj.weight"} <= names  # fmt: skip
    if arch == "GlmMoeDsaForCausalLM":
        assert "model.layers.0.self_attn.indexer.wq_b.weight" in names and "model.layers.1.self_attn.indexer.k_norm.bias" in names
    if arch == "MiniMaxM2ForCausalLM":
        assert hf["model.layers.0.self_attn.q_norm.weight"].numel() == cfg.num_attention_heads * cfg.head_dim
        assert "model.layers.0.self_attn.sinks" in names
    for name, p in model.named_parameters():
        sources, rule = convert.hf_sources_for(cfg, name)
        back = convert.merge_hf_sources(rule, [hf[s] for s in sources], cfg)
        assert back.shape == p.shape and torch.allclose(back, p.detach(), atol=1e-6), name


def test_gated_qkv_shards_merge_and_split():
    from slime_b200.weight_sync import convert

    cfg = _tiny(attention_output_gate=True, rotary_percent=0.25, qk_layernorm=True)
    rows = (2 * cfg.num_attention_heads + 2 * cfg.num_query_groups) * cfg.head_dim
    full = torch.arange(rows * 3, dtype=torch.float32).view(rows, 3)
    shards = [convert.shard_for_tp(cfg, "decoder.layers.0.self_attention.linear_qkv.weight", full, 0, 1, 2, r) for r in range(2)]
    assert shards[0].shape[0] == rows // 2
    assert torch.equal(convert.merge_tp_shards(cfg, "decoder.layers.0.self_attention.linear_qkv.weight", shards, 0, 1), full)


def test_hugging_face_style_module_runs_as_a_layer():
    """A custom builder swaps the mixer of chosen layers for a wrapped external module; the rest keep the built-in one."""
    import torch.nn as nn

    class Toy(nn.Module):  # "attention" that mixes nothing: enough to see the plumbing
        def __init__(self, h):
            super().__init__()
            self.proj = nn.Linear(h, h, bias=False)

        def forward(self, hidden_states, position_ids=None, cu_seqlens=None):
            assert hidden_states.dim() == 3 and position_ids.shape[1] == hidden_states.shape[1] and cu_seqlens is not None
            return (self.proj(hidden_states),)

    cfg = _tiny()
    mixers.set_custom_builder(lambda c, i, dt, dev, sp: mixers.HuggingfaceAttention(c, i, dt, dev, sp, Toy(c.hidden_size)) if i == 1 else None)
    try:
        model = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=1)
    finally:
        mixers.set_custom_builder(None)
    kinds = [type(layer.self_attention).__name__ for layer in model.decoder.layers]
    assert kinds == ["SelfAttention", "HuggingfaceAttention"]
    p, T = packed_for([7, 5])
    ids = torch.randint(0, cfg.vocab_size, (T,))
    model(ids, position_ids=p.position_ids, packed_seq_params=p)[0].sum().backward()
    w = model.decoder.layers[1].self_attention.hf_module.proj.weight
    assert w.grad is not None and float(w.grad.abs().sum()) > 0 and w.tensor_model_parallel is False


def test_mtp_loss_shifts_inputs_targets_and_masks_per_sequence():
    """Depth-1 draft head: position i sees the trunk's hidden state of i and the embedding of token i + 1 and is
    scored on token i + 2; nothing crosses a sequence boundary; the loss trains the head only."""
    from slime_b200 import ops
    from slime_b200.weight_sync import convert

    torch.manual_seed(0)
    cfg = _tiny(mtp_num_layers=1)
    model = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=1)
    model.mtp_training = True
    lens = [7, 5]
    ids = torch.randint(0, cfg.vocab_size, (sum(lens),))
    full_mask = torch.tensor([0, 0, 1, 1, 1, 1, 0] + [0, 1, 1, 1, 0], dtype=torch.float32)

    def run(tokens, ls, mask):
        p, _ = packed_for(ls)
        model(tokens, position_ids=p.position_ids, packed_seq_params=p)
        return model.mtp_loss(mask)

    both = run(ids, lens, full_mask)
    # per sequence: sums of per-token terms add up (the packed loss is a mean over all valid positions)
    def terms(tokens, n, mask):
        p, _ = packed_for([n])
        model(tokens, position_ids=p.position_ids, packed_seq_params=p)
        hidden, _, packed, table = model._mtp_inputs
        model._mtp_inputs = None
        nxt = torch.cat([tokens[1:], tokens.new_zeros(1)])
        emb = ops.embedding(nxt, model.embedding.word_embeddings.weight, 0)
        out, _ = model.mtp.layers[0](hidden, emb, table, packed)
        logp = (out.float() @ model.output_weight().float().t()).log_softmax(-1)
        tot, cnt = 0.0, 0
        for i in range(n - 2):
            if mask[i + 1] > 0:
                tot, cnt = tot - logp[i, tokens[i + 2]], cnt + 1
        return tot, cnt

    t1, c1 = terms(ids[:7], 7, full_mask[:7])
    t2, c2 = terms(ids[7:], 5, full_mask[7:])
    assert c1 == 4 and c2 == 3  # targets whose own predicting position is trained, inside the sequence
    assert torch.allclose(both, (t1 + t2) / (c1 + c2), atol=1e-5)
    run(ids, lens, full_mask).backward()
    named = dict(model.named_parameters())
    assert float(named["mtp.layers.0.eh_proj.weight"].grad.abs().sum()) > 0
    # the policy is not touched by the draft loss: trunk, embedding table and output head get no gradient from it
    for n in ("decoder.layers.0.mlp.linear_fc1.weight", "embedding.word_embeddings.weight", "output_layer.weight"):
        assert named[n].grad is None or float(named[n].grad.abs().sum()) == 0, n
    # checkpoint names: the draft depth is stored as one more layer with its own norms and projection
    hf = dict(x for n, p in model.named_parameters() if n.startswith("mtp.") for x in convert.convert_to_hf(cfg, n, p.detach()))
    assert {"model.layers.2.enorm.weight", "model.layers.2.eh_proj.weight", "model.layers.2.shared_head.norm.weight",
            "model.layers.2.self_attn.q_proj.weight", "model.layers.2.mlp.down_proj.weight"} <= set(hf)
    for n, p in model.named_parameters():
        if n.startswith("mtp."):
            src, rule = convert.hf_sources_for(cfg, n)
            assert torch.equal(convert.merge_hf_sources(rule, [hf[s] for s in src], cfg), p.detach()), n


def test_grpo_step_trains_the_draft_head_end_to_end():
    """Colocated GRPO on CPU with --enable-mtp-training: the draft layer's matrices move with the step, and the rollout
    engine (which does not run the draft depth) accepts the synced weights."""
    from slime_b200.api import ColocatedGRPO
    from slime_b200.models.config import apply_to_args
    from slime_b200.utils.arguments import namespace_from_dict

    cfg = _tiny(mtp_num_layers=1)
    args = namespace_from_dict(dict(
        rollout_batch_size=2, n_samples_per_prompt=4, num_rollout=1, global_batch_size=8, colocate=True, use_dynamic_batch_size=True,
        max_tokens_per_gpu=256, lr=1e-3, eps_clip=0.2, eps_clip_high=0.28, rollout_ignore_eos=True, rollout_max_context_len=64,
        custom_rm_path="slime_b200.rollout.synthetic.mod7_reward", actor_num_nodes=1, actor_num_gpus_per_node=1, rollout_num_gpus=1,
        sglang_max_running_requests=8, sglang_disable_cuda_graph=True, untie_embeddings_and_output_weights=True,
        data_pad_size_multiplier=8, enable_mtp_training=True, mtp_num_layers=1))  # fmt: skip
    apply_to_args(cfg, args)
    r = ColocatedGRPO(args, device="cpu", engine_pages=64)
    before = {n: p.detach().clone() for n, p in r.actor.model.named_parameters() if n.startswith("mtp.") and p.dim() == 2}
    assert "mtp.layers.0.eh_proj.weight" in before
    out = r.step(torch.randint(0, cfg.vocab_size, (2, 8), generator=torch.Generator().manual_seed(0)).tolist(), 12)
    assert math.isfinite(float(out["metrics"]["train/loss"]))
    after = dict(r.actor.model.named_parameters())
    assert all(not torch.equal(after[n].detach(), w) for n, w in before.items())


def test_yarn_frequencies_keep_fast_dimensions_and_interpolate_slow_ones():
    from slime_b200.ops import reference

    dim, base, factor, orig = 64, 1e4, 40.0, 4096
    plain = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
    inv = reference.yarn_inv_freq(dim, base, factor, orig)
    assert torch.allclose(inv[:4], plain[:4])  # many turns inside the original context: untouched
    assert torch.allclose(inv[-4:], plain[-4:] / factor)  # less than one turn: positions interpolated by the factor
    mid = (inv / plain)[4:-4]
    assert ((mid <= 1 + 1e-12) & (mid >= 1 / factor - 1e-12)).all() and (mid[1:] <= mid[:-1] + 1e-12).all()  # monotone blend
    assert torch.allclose(reference.yarn_inv_freq(dim, base, 1.0, orig), plain)
    assert reference.yarn_mscale(1.0) == 1.0 and abs(reference.yarn_mscale(40.0, 1.0) - (0.1 * math.log(40.0) + 1)) < 1e-12
    table = reference.rope_cos_sin_yarn(16, dim, base, factor, orig, mscale=1.0, mscale_all_dim=1.0)
    assert table.shape == (16, dim) and torch.allclose(table[0, : dim // 2], torch.ones(dim // 2))
    # the latent-attention layer picks the table and the attention temperature up from the config
    cfg = _tiny(multi_latent_attention=True, q_lora_rank=24, kv_lora_rank=16, qk_head_dim=8, qk_pos_emb_head_dim=8, v_head_dim=8,
                rotary_scaling_type="yarn", rotary_scaling_factor=40.0, mscale=1.0, mscale_all_dim=1.0)  # fmt: skip
    layer = mixers.MLASelfAttention(cfg, 0, torch.float32, "cpu", False)
    assert abs(layer.scale - 16**-0.5 * reference.yarn_mscale(40.0, 1.0) ** 2) < 1e-9
    assert torch.allclose(layer._table("cpu", 8)[:8], reference.rope_cos_sin_yarn(4096, 8, 1e4, 40.0, 4096, mscale=1.0, mscale_all_dim=1.0)[:8])


def test_delta_rule_and_conv_continue_from_saved_state():
    """Prefill in two pieces, and decode one token at a time, equal one pass over the whole sequence."""
    torch.manual_seed(0)
    T, H, Dk, Dv, C, K = 23, 2, 4, 6, 5, 4
    q, k, v = torch.randn(T, H, Dk), torch.randn(T, H, Dk), torch.randn(T, H, Dv)
    g, beta = -torch.rand(T, H) * 0.4, torch.rand(T, H)
    cu = torch.tensor([0, T], dtype=torch.int32)
    whole, final = mixers.gated_delta_rule_chunked(q, k, v, g, beta, cu, chunk=8, return_final_states=True)
    cut = 13
    first, st = mixers.gated_delta_rule_chunked(q[:cut], k[:cut], v[:cut], g[:cut], beta[:cut], torch.tensor([0, cut], dtype=torch.int32),
                                                chunk=8, return_final_states=True)  # fmt: skip
    second, st2 = mixers.gated_delta_rule_chunked(q[cut:], k[cut:], v[cut:], g[cut:], beta[cut:], torch.tensor([0, T - cut], dtype=torch.int32),
                                                  chunk=8, initial_states=st, return_final_states=True)  # fmt: skip
    assert torch.allclose(torch.cat([first, second]), whole, atol=1e-5) and torch.allclose(st2[0], final[0], atol=1e-5)
    S = st[0].clone()[None]
    for t in range(cut, T):
        o = mixers.gated_delta_rule_step(q[t][None], k[t][None], v[t][None], g[t][None], beta[t][None], S)
        assert torch.allclose(o[0], whole[t], atol=1e-5), t
    assert torch.allclose(S[0], final[0], atol=1e-5)
    # convolution: history of the last K-1 inputs
    x, w = torch.randn(T, C), torch.randn(C, K)
    pos = torch.arange(T, dtype=torch.int32)
    ref = mixers.causal_short_conv(x, w, pos)
    hist = x[cut - (K - 1) : cut]
    tail = mixers.causal_short_conv(x[cut:], w, torch.arange(T - cut, dtype=torch.int32), history=[hist],
                                    cu_seqlens=torch.tensor([0, T - cut], dtype=torch.int32))  # fmt: skip
    assert torch.allclose(tail, ref[cut:], atol=1e-6)
    state = hist.clone()[None]
    for t in range(cut, T):
        assert torch.allclose(mixers.short_conv_step(x[t][None], w, state)[0], ref[t], atol=1e-6), t


def test_qwen_family_draft_block_names_round_trip():
    from slime_b200.weight_sync import convert

    """Qwen3-Next / Qwen3.5 keep the draft head in a top-level ``mtp`` block: norms minus one, Qwen3-Next's joining
    projection with swapped halves, the inner layer under mtp.layers.k."""
    for arch, swapped in (("Qwen3NextForCausalLM", True), ("Qwen3_5ForCausalLM", False)):
        cfg = _tiny(mtp_num_layers=1, model_arch=arch, qk_layernorm=True)
        model = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=2)
        named = {n: p for n, p in model.named_parameters() if n.startswith("mtp.")}
        hf = dict(x for n, p in named.items() for x in convert.convert_to_hf(cfg, n, p.detach()))
        assert {"mtp.pre_fc_norm_embedding.weight", "mtp.pre_fc_norm_hidden.weight", "mtp.norm.weight", "mtp.fc.weight",
                "mtp.layers.0.self_attn.q_proj.weight", "mtp.layers.0.input_layernorm.weight"} <= set(hf), sorted(hf)  # fmt: skip
        assert torch.equal(hf["mtp.norm.weight"], named["mtp.layers.0.final_layernorm.weight"] - 1)
        w = named["mtp.layers.0.eh_proj.weight"]
        h = w.shape[1] // 2
        assert torch.equal(hf["mtp.fc.weight"], torch.cat([w[:, h:], w[:, :h]], dim=1) if swapped else w)
        for n, p in named.items():
            names, rule = convert.hf_sources_for(cfg, n)
            assert torch.allclose(convert.merge_hf_sources(rule, [hf[x] for x in names], cfg), p), n
