"""End-to-end GPU checks: trainer model vs fp32 reference, engine/trainer log-prob agreement, one GRPO step."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _tiny_args(**kw):
    from slime_b200.models.config import ModelConfig, apply_to_args
    from slime_b200.utils.arguments import namespace_from_dict

    cfg = ModelConfig(num_layers=2, hidden_size=256, num_attention_heads=4, num_query_groups=2, kv_channels=64,
                      ffn_hidden_size=512, vocab_size=4096, rotary_base=1e6, tie_word_embeddings=True, add_qkv_bias=True)  # fmt: skip
    base = dict(rollout_batch_size=4, n_samples_per_prompt=4, num_rollout=1, global_batch_size=16, colocate=True,
                use_dynamic_batch_size=True, max_tokens_per_gpu=2048, lr=1e-5, eps_clip=0.2, eps_clip_high=0.28,
                rollout_ignore_eos=True, rollout_max_context_len=256, custom_rm_path="slime_b200.rollout.synthetic.mod7_reward",
                actor_num_nodes=1, actor_num_gpus_per_node=1, rollout_num_gpus=1, sglang_max_running_requests=16)  # fmt: skip
    base.update(kw)
    args = namespace_from_dict(base)
    apply_to_args(cfg, args)
    return args, cfg


def test_trainer_forward_backward_matches_fp32_reference(kernels):
    """bf16 kernel path vs the same model evaluated with the fp32 PyTorch reference ops on CPU."""
    from slime_b200.models.gpt import GPTModel, PackedSeqParams

    args, cfg = _tiny_args()
    torch.manual_seed(0)
    m = GPTModel(cfg, dtype=torch.bfloat16, device="cuda", seed=3)
    ref = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=3)
    ref.load_state_dict({k: v.float().cpu() for k, v in m.state_dict().items()})
    ids = torch.randint(0, cfg.vocab_size, (300,))
    cu = torch.tensor([0, 100, 230, 300], dtype=torch.int32)
    out = m(ids.cuda(), packed_seq_params=PackedSeqParams(cu.cuda(), 130))
    out_ref = ref(ids, packed_seq_params=PackedSeqParams(cu, 130))
    lp = torch.log_softmax(out.float(), -1).cpu()
    lp_ref = torch.log_softmax(out_ref.float(), -1)
    assert (lp - lp_ref).abs().max().item() < 0.15
    assert (lp - lp_ref).abs().mean().item() < 0.03  # the bound above is for the worst of 300 x V entries
    tgt = torch.randint(0, cfg.vocab_size, (300,))
    loss = -torch.log_softmax(out.float(), -1)[0].gather(-1, tgt.cuda()[:, None]).mean()
    loss_ref = -lp_ref[0].gather(-1, tgt[:, None]).mean()
    assert abs(loss.item() - loss_ref.item()) < 2e-2
    loss.backward()
    loss_ref.backward()
    for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
        g, gr = p.grad.float().cpu(), q.grad
        denom = gr.abs().max().item() + 1e-6
        assert (g - gr).abs().max().item() / denom < 0.12, n
        assert (g - gr).abs().mean().item() / denom < 0.02, n  # the typical entry is much closer than the worst one


def test_engine_matches_trainer_logprobs(kernels):
    """Rollout log-probs (decode path, CUDA graphs) equal the trainer's log-probs for the same weights."""
    from slime_b200.api import ColocatedGRPO

    args, cfg = _tiny_args()
    runner = ColocatedGRPO(args, engine_pages=512)
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(0, cfg.vocab_size, (4, 40), generator=g).tolist()
    samples = runner.generate(prompts, [20 + i for i in range(16)])
    assert runner.engine.stats["cached_tokens"] > 0, "siblings of a prompt should hit the prefix cache"
    out = runner.train_on(runner.reward(samples))
    diff = out[-1]["train/train_rollout_logprob_abs_diff"]
    assert diff < 2e-2, diff
    assert abs(out[-1]["train/ppo_kl"]) < 1e-6
    assert out[-1]["train/grad_norm"] > 0


def test_grpo_step_changes_weights_and_syncs(kernels):
    from slime_b200.api import ColocatedGRPO
    from slime_b200.ops import _lib

    args, cfg = _tiny_args(lr=1e-3)
    runner = ColocatedGRPO(args, engine_pages=512)
    before = runner.engine.weights.layers[0]["qkv"].clone()
    g = torch.Generator().manual_seed(2)
    prompts = torch.randint(0, cfg.vocab_size, (4, 33), generator=g).tolist()
    res = runner.step(prompts, [16] * 16)
    torch.cuda.synchronize()
    _lib.check_status("cuda")
    after = runner.engine.weights.layers[0]["qkv"]
    assert (after.float() - before.float()).abs().max().item() > 0
    p = dict(runner.actor.model.named_parameters())["decoder.layers.0.self_attention.linear_qkv.weight"]
    assert torch.equal(after, p.data)
    assert res["metrics"]["train/loss"] == res["metrics"]["train/loss"]
    assert runner.engine.get_weight_version() == "2"


def test_general_loss_path_agrees_with_fused_path(kernels):
    """The [T, V]-logits path (all options) and the fused chunked path give the same step metrics."""
    from slime_b200.api import ColocatedGRPO

    vals = {}
    for fused in (True, False):
        args, cfg = _tiny_args(lr=0.0)
        args.fused_loss = fused
        runner = ColocatedGRPO(args, engine_pages=512)
        g = torch.Generator().manual_seed(5)
        prompts = torch.randint(0, cfg.vocab_size, (4, 24), generator=g).tolist()
        res = runner.step(prompts, [12] * 16)
        vals[fused] = res["metrics"]
    for k in ("train/entropy_loss", "train/grad_norm", "train/pg_loss"):
        a, b = vals[True][k], vals[False][k]
        assert abs(a - b) <= 3e-2 * max(1.0, abs(b)), (k, a, b)
