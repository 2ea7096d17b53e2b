"""Run under torchrun on 2 gloo ranks (CPU) or 2 GPUs (DEVICE=cuda): colocated GRPO on a small MoE model with the
trainer's experts sharded over the two ranks (EP2 = DP2), one rollout engine per rank that keeps its projections in
block fp8, and rollout routing replay (the trainer's routers reuse the experts the engine picked).

Checks: the engine's quantised buffers follow the trainer's weights after every sync, samples carry one routed-expert
row per fed token and layer, the trainer's routers were served exactly those rows, the loss is finite, and the rollout
log-probs stay within W8A8 error of the trainer's recomputation.
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    import faulthandler

    faulthandler.dump_traceback_later(280, exit=True)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    cuda = os.environ.get("DEVICE", "cpu") == "cuda"
    if cuda:
        local = int(os.environ["LOCAL_RANK"])
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        dist.init_process_group("gloo")
    from slime_b200.api import ColocatedGRPO
    from slime_b200.engine.quant import Fp8Weight
    from slime_b200.models.config import ModelConfig, apply_to_args
    from slime_b200.parallel import state as mpu
    from slime_b200.utils import routing_replay
    from slime_b200.utils.arguments import namespace_from_dict

    mpu.initialize_model_parallel(expert_model_parallel_size=world, **({} if cuda else {"backend": "gloo"}))
    cfg = ModelConfig(num_layers=3, hidden_size=256, num_attention_heads=4, num_query_groups=2, kv_channels=64,
                      ffn_hidden_size=512, vocab_size=1024, rotary_base=1e4, tie_word_embeddings=False, qk_layernorm=True,
                      num_experts=4, moe_ffn_hidden_size=128, moe_router_topk=2, moe_layer_freq=[0, 1, 1])  # fmt: skip
    G, n = 3, 4
    args = namespace_from_dict(dict(
        rollout_batch_size=G * world, n_samples_per_prompt=n, num_rollout=4, global_batch_size=G * n * world, colocate=True,
        use_dynamic_batch_size=True, max_tokens_per_gpu=512, lr=1e-4, eps_clip=0.2, eps_clip_high=0.28,
        rollout_ignore_eos=True, rollout_max_context_len=128, custom_rm_path="slime_b200.rollout.synthetic.mod7_reward",
        actor_num_nodes=1, actor_num_gpus_per_node=world, rollout_num_gpus=world, rollout_num_gpus_per_engine=1,
        sglang_max_running_requests=G * n, expert_model_parallel_size=world, bf16=cuda, untie_embeddings_and_output_weights=True,
        sglang_disable_cuda_graph=not cuda, data_pad_size_multiplier=8 if not cuda else 128, get_mismatch_metrics=True,
        sglang_quantization="fp8", use_rollout_routing_replay=True, use_routing_replay=True, recompute_granularity="full",
    ))  # fmt: skip
    apply_to_args(cfg, args)
    runner = ColocatedGRPO(args, engine_pages=256)
    L = runner.engine.weights.layers
    assert isinstance(L[0]["gate_up"], Fp8Weight) and isinstance(L[1]["w13"], Fp8Weight) and isinstance(L[2]["w2"], Fp8Weight)
    served = []
    original = routing_replay.RoutingReplay.compute_topk

    def spy(self, scores, k):
        idx = original(self, scores, k)
        served.append((self.layer_number, os.environ.get("ROUTING_REPLAY_STAGE"), idx.detach().cpu()))
        return idx

    routing_replay.RoutingReplay.compute_topk = spy
    g = torch.Generator().manual_seed(11 + rank)
    for step in range(2):
        prompts = torch.randint(0, cfg.vocab_size, (G, 16), generator=g).tolist()
        lens = torch.randint(8, 24, (G * n,), generator=g).tolist()
        samples = runner.generate(prompts, lens)
        for s in samples:
            r = torch.as_tensor(s.rollout_routed_experts)
            assert r.shape == (len(s.tokens) - 1, cfg.num_layers, cfg.moe_router_topk), r.shape
            assert int(r[:, 0].abs().max()) == 0 and int(r.max()) < cfg.num_experts  # layer 0 is dense
        runner.reward(samples)
        served.clear()
        metrics = runner.train_on(samples)[-1]
        # every router call of the step ran in a replay stage and returned rows the engine had recorded
        assert served and all(stage == "replay_forward" for _, stage, _ in served), {st for _, st, _ in served}
        routed_all = torch.cat([torch.as_tensor(s.rollout_routed_experts) for s in samples])
        pool = {tuple(row) for row in routed_all[:, 1].tolist()} | {(0, 0)}
        lay1 = [idx for layer, _, idx in served if layer == 1]
        assert all(tuple(row) in pool for idx in lay1 for row in idx.tolist())
        runner.actor.update_weights()
        runner.rollout_id += 1
        loss = float(metrics["train/loss"])
        assert loss == loss and abs(loss) < 1e4, loss
        diff = float(metrics.get("train/train_rollout_logprob_abs_diff", 0.0))
        assert diff < 0.3, diff  # fp8 engine against the trainer's bf16 / fp32 recomputation
        # the engine's fp8 bytes follow the trainer: a dense fc2 shard and a local expert, dequantised
        params = dict(runner.actor.model.named_parameters())
        ref = params["decoder.layers.0.mlp.linear_fc2.weight"].detach().float().cpu()
        got = L[0]["down"].dequant(torch.float32).cpu()
        assert (got - ref).abs().max() <= ref.abs().max() / 14, float((got - ref).abs().max() / ref.abs().max())
        e_local = params["decoder.layers.1.mlp.experts.linear_fc2.weight0"].detach().float().cpu()
        first = rank * (cfg.num_experts // world)
        got = L[1]["w2"][first].dequant(torch.float32).cpu()
        assert (got - e_local).abs().max() <= e_local.abs().max() / 14
    if cuda:
        from slime_b200.ops import _lib

        torch.cuda.synchronize()
        _lib.check_status(runner.device)
    dist.barrier()
    if rank == 0:
        print(f"RESULT ok world={world} ep={world} device={'cuda' if cuda else 'cpu'} engine=fp8 routing_replay=rollout "
              f"logprob_diff={diff:.3f}", flush=True)
    from slime_b200.utils.distributed_utils import shutdown_distributed

    shutdown_distributed([runner.engine])


if __name__ == "__main__":
    main()
