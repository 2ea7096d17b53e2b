"""Run under torchrun (gloo ranks on CPU, or NCCL ranks with DEVICE=cuda): colocated GRPO steps with the trainer and
the rollout engine both tensor-parallel over the same group (TP2, optionally x DP2).

Checks: the ranks of a tensor-parallel group generate identical samples (the engine ranks step in lockstep), the
engine's weights equal the trainer's shard after the sync, the loss is finite and equal across the group, and the
rollout log-probs agree with the trainer's recomputation.
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    import faulthandler

    faulthandler.dump_traceback_later(240, exit=True)  # a stuck job prints where every thread is and ends itself
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    cuda = os.environ.get("DEVICE", "cpu") == "cuda"
    if cuda:
        local = int(os.environ["LOCAL_RANK"])
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        dist.init_process_group("gloo")
    from slime_b200.api import ColocatedGRPO
    from slime_b200.models.config import ModelConfig, apply_to_args
    from slime_b200.parallel import state as mpu
    from slime_b200.utils.arguments import namespace_from_dict

    tp = 2
    mpu.initialize_model_parallel(tensor_model_parallel_size=tp, **({} if cuda else {"backend": "gloo"}))
    dp = world // tp
    cfg = ModelConfig(num_layers=2, hidden_size=256, num_attention_heads=4, num_query_groups=2, kv_channels=64,
                      ffn_hidden_size=512, vocab_size=1024, rotary_base=1e4, tie_word_embeddings=False, qk_layernorm=True)
    G, n = 3, 4
    args = namespace_from_dict(dict(
        rollout_batch_size=G * dp, n_samples_per_prompt=n, num_rollout=4, global_batch_size=G * n * dp, colocate=True,
        use_dynamic_batch_size=True, max_tokens_per_gpu=512, lr=1e-4, eps_clip=0.2, eps_clip_high=0.28,
        rollout_ignore_eos=True, rollout_max_context_len=128, custom_rm_path="slime_b200.rollout.synthetic.mod7_reward",
        actor_num_nodes=1, actor_num_gpus_per_node=world, rollout_num_gpus=world, rollout_num_gpus_per_engine=tp,
        sglang_max_running_requests=G * n, tensor_model_parallel_size=tp, sequence_parallel=True, bf16=cuda,
        untie_embeddings_and_output_weights=True, sglang_disable_cuda_graph=not cuda, data_pad_size_multiplier=8 if not cuda else 128,
        get_mismatch_metrics=False,
    ))  # fmt: skip
    apply_to_args(cfg, args)
    runner = ColocatedGRPO(args, engine_pages=256)
    g = torch.Generator().manual_seed(7 + mpu.get_data_parallel_rank())
    tpg = mpu.get_tensor_model_parallel_group()
    for step in range(2):
        prompts = torch.randint(0, cfg.vocab_size, (G, 16), generator=g).tolist()
        lens = torch.randint(8, 24, (G * n,), generator=g).tolist()
        samples = runner.generate(prompts, lens)
        flat = torch.tensor([t for s in samples for t in s.tokens], dtype=torch.int64, device=runner.device)
        both = [torch.empty_like(flat) for _ in range(tp)]
        dist.all_gather(both, flat, group=tpg)
        assert all(torch.equal(both[0], b) for b in both), "tensor-parallel engine ranks generated different tokens"
        runner.reward(samples)
        metrics = runner.train_on(samples)[-1]
        runner.actor.update_weights()
        runner.rollout_id += 1
        loss = torch.tensor([float(metrics["train/loss"])], device=runner.device)
        assert torch.isfinite(loss).all()
        ls = [torch.empty_like(loss) for _ in range(tp)]
        dist.all_gather(ls, loss, group=tpg)
        assert abs(float(ls[0]) - float(ls[1])) < 1e-6, ls
        diff = float(metrics.get("train/train_rollout_logprob_abs_diff", 0.0))
        assert diff < (0.05 if cuda else 1e-4), diff
        # engine shard == trainer shard after the sync
        w = runner.engine.weights
        for name, p in runner.actor.model.named_parameters():
            if name.endswith("layers.0.self_attention.linear_qkv.weight"):
                assert torch.equal(w.layers[0]["qkv"].float().cpu(), p.detach().float().cpu().to(w.layers[0]["qkv"].dtype).float())
    if cuda:
        from slime_b200.ops import _lib

        torch.cuda.synchronize()
        _lib.check_status(runner.device)
    dist.barrier()
    if rank == 0:
        print(f"RESULT ok world={world} tp={tp} dp={dp} device={'cuda' if cuda else 'cpu'} fused_tp={runner.engine.runner._fused_tp is not None}"
              f" logprob_diff={diff:.2e}", flush=True)
    from slime_b200.utils.distributed_utils import shutdown_distributed

    shutdown_distributed([runner.engine])


if __name__ == "__main__":
    main()
