"""Run under torchrun with gloo ranks on CPU: invariants of the distributed training paths.

    MODE=cp   context parallel (zig-zag): per-rank reducers add up to the single-rank value; gather/slice round trip
    MODE=dp   ZeRO-1 data parallel: reduce-scatter + sharded Adam + all-gather equals one rank holding summed gradients
    MODE=tp   vocab-parallel log-prob / entropy (values and gradients) equals the full-vocabulary computation
"""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def check_cp(rank, world):
    from slime_b200.backends.train import cp_utils
    from slime_b200.parallel import state as mpu

    mpu.initialize_model_parallel(context_parallel_size=world, backend="gloo")
    g = torch.Generator().manual_seed(3)
    totals, resps = [23, 64, 10, 130], [11, 40, 9, 77]  # every sample has at least one prompt token
    full_vals = [torch.randn(r, generator=g) for r in resps]
    masks = [(torch.rand(r, generator=g) > 0.3).float() for r in resps]
    for per_token in (False, True):
        local_vals = torch.cat([cp_utils.slice_log_prob_with_cp(v, t, r) for v, t, r in zip(full_vals, totals, resps)])
        reducer = cp_utils.get_sum_of_sample_mean(totals, resps, masks, None, per_token)
        part = reducer(local_vals).reshape(1).clone()
        dist.all_reduce(part, group=mpu.get_context_parallel_group())
        if per_token:
            want = sum((v * m).sum() for v, m in zip(full_vals, masks))
        else:
            want = sum((v * m).sum() / m.sum().clamp_min(1) for v, m in zip(full_vals, masks))
        torch.testing.assert_close(part[0], want, rtol=1e-5, atol=1e-6)
    # gather(slice(x)) == x, and the gradient of the gather lands on the local slice only
    for v, t, r in zip(full_vals, totals, resps):
        loc = cp_utils.slice_log_prob_with_cp(v, t, r).clone().requires_grad_()
        full = cp_utils.all_gather_with_cp(loc, t, r)
        torch.testing.assert_close(full.detach(), v)
        (full * torch.arange(1, r + 1, dtype=torch.float32)).sum().backward()
        want = cp_utils.slice_log_prob_with_cp(torch.arange(1, r + 1, dtype=torch.float32), t, r)
        torch.testing.assert_close(loc.grad, want * world)  # every rank back-propagates the same full loss
    # token slicing pads to 2 * cp chunks and keeps chunks (r, 2cp-1-r)
    toks = torch.arange(37)
    mine = cp_utils.slice_with_cp(toks, 0)
    cs = -(-37 // (2 * world))
    padded = torch.cat([toks, torch.zeros(2 * world * cs - 37, dtype=toks.dtype)])
    want = torch.cat([padded[rank * cs : (rank + 1) * cs], padded[(2 * world - rank - 1) * cs : (2 * world - rank) * cs]])
    assert torch.equal(mine, want)


def check_dp(rank, world):
    from slime_b200.backends.train.buffers import FlatBuffer
    from slime_b200.backends.train.optimizer import DistributedOptimizer

    shapes = [(64, 48), (48,), (130, 7), (5, 3)]

    def make(group, size, r):
        torch.manual_seed(1)
        params = [torch.nn.Parameter(torch.randn(*s).to(torch.bfloat16)) for s in shapes]
        buf = FlatBuffer(params, [f"p{i}" for i in range(len(params))], group, size, r, torch.device("cpu"))
        return params, buf, DistributedOptimizer([buf], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1, clip_grad=1.0)

    p_dp, b_dp, o_dp = make(dist.group.WORLD, world, rank)
    # oracle: AdamW with global-norm clipping on fp32 masters, written out directly
    lr, b1, b2, eps, wd, clip, scale = 1e-2, 0.9, 0.95, 1e-8, 0.1, 1.0, 0.5
    torch.manual_seed(1)
    masters = [torch.randn(*s).to(torch.bfloat16).float() for s in shapes]
    ms, vs = [torch.zeros(s) for s in shapes], [torch.zeros(s) for s in shapes]
    for step in range(1, 4):
        grads = []
        for r in range(world):  # every rank can reproduce every rank's gradient
            g = torch.Generator().manual_seed(100 * step + r)
            grads.append([torch.randn(s, generator=g) for s in shapes])
        for p, gr in zip(p_dp, grads[rank]):
            p.main_grad.copy_(gr)
        b_dp.reduce_scatter_grads()
        n_dp = o_dp.step(grad_scale=scale)
        summed = [sum(grads[r][i] for r in range(world)) * scale for i in range(len(shapes))]
        norm = torch.sqrt(sum(g.pow(2).sum() for g in summed))
        torch.testing.assert_close(n_dp.reshape(()), norm, rtol=1e-5, atol=1e-6)
        coef = min(1.0, clip / (float(norm) + 1e-6))
        for i, g in enumerate(summed):
            g = g * coef
            ms[i] = b1 * ms[i] + (1 - b1) * g
            vs[i] = b2 * vs[i] + (1 - b2) * g * g
            masters[i] = masters[i] * (1 - lr * wd) - lr * (ms[i] / (1 - b1**step)) / ((vs[i] / (1 - b2**step)).sqrt() + eps)
        for a, m in zip(p_dp, masters):  # every rank holds every updated parameter (bf16 rounding of the fp32 master)
            torch.testing.assert_close(a.data.float(), m.to(torch.bfloat16).float(), rtol=0, atol=1e-6)
        b_dp.zero_grad()


def check_tp(rank, world):
    from slime_b200.parallel import state as mpu
    from slime_b200.utils.ppo_utils import calculate_log_probs_and_entropy

    mpu.initialize_model_parallel(tensor_model_parallel_size=world, backend="gloo")
    g = torch.Generator().manual_seed(9)
    T, V = 19, 64 * world
    full = torch.randn(T, V, generator=g) * 2
    tokens = torch.randint(0, V, (T,), generator=g)
    ref_logits = full.clone().requires_grad_()
    lsm = torch.log_softmax(ref_logits, -1)
    ref_lp = lsm.gather(-1, tokens[:, None]).squeeze(-1)
    ref_ent = -(lsm.exp() * lsm).sum(-1)
    w = torch.randn(T, generator=g)
    ((ref_lp * w).sum() + 0.3 * ref_ent.sum()).backward()
    vl = V // world
    local = full[:, rank * vl : (rank + 1) * vl].clone().requires_grad_()
    for chunk in (-1, 7):
        local.grad = None
        lp, ent = calculate_log_probs_and_entropy(local, tokens, mpu.get_tensor_model_parallel_group(), with_entropy=True,
                                                  chunk_size=chunk)
        torch.testing.assert_close(lp, ref_lp.detach(), rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(ent, ref_ent.detach(), rtol=1e-5, atol=1e-5)
        ((lp * w).sum() + 0.3 * ent.sum()).backward()
        torch.testing.assert_close(local.grad, ref_logits.grad[:, rank * vl : (rank + 1) * vl], rtol=1e-4, atol=1e-5)


def check_reload(rank, world):
    """Communicators are destroyed and rebuilt: topology queries survive, collectives work again on the new groups,
    a buffer that was handed a group getter follows, and repeated cycles do not collide in the rendezvous store."""
    from slime_b200.backends.train.buffers import FlatBuffer
    from slime_b200.parallel import state as mpu

    tp = 2
    mpu.initialize_model_parallel(tensor_model_parallel_size=tp, backend="gloo")
    dp = world // tp
    p = torch.nn.Parameter(torch.zeros(256, dtype=torch.bfloat16))
    buf = FlatBuffer([p], ["p"], mpu.get_data_parallel_group, dp, mpu.get_data_parallel_rank(), torch.device("cpu"))

    def exercise(tag):
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, group=mpu.get_tensor_model_parallel_group())
        base = (rank // tp) * tp
        assert float(t) == sum(base + i + 1 for i in range(tp)), (tag, float(t))
        buf.grad_data.fill_(1.0)
        buf.all_reduce_grads()
        assert float(buf.grad_data[0]) == dp, (tag, float(buf.grad_data[0]))

    exercise("before")
    for cycle in range(2):
        assert mpu.release_communicators()
        assert mpu.communicators_released() and mpu.get_tensor_model_parallel_group() is None
        assert mpu.get_tensor_model_parallel_world_size() == tp and mpu.get_data_parallel_world_size() == dp
        assert mpu.get_tensor_model_parallel_rank() == rank % tp
        t = torch.ones(1)
        dist.all_reduce(t)  # the temporary host-side WORLD
        assert float(t) == world
        assert not mpu.release_communicators()  # idempotent
        assert mpu.reload_communicators()
        exercise(f"cycle {cycle}")
    assert not mpu.reload_communicators()


def check_expert_route(rank, world):
    """An expert-parallel trainer model (EP = world) ships each routed expert to the rank whose engine shard hosts it
    (here the shards are rotated by one rank, so every tensor crosses)."""
    from slime_b200.backends.train.model import TrainModel
    from slime_b200.models.config import ModelConfig, apply_to_args
    from slime_b200.parallel import state as mpu
    from slime_b200.utils.arguments import namespace_from_dict
    from slime_b200.weight_sync import expert_routing as er

    mpu.initialize_model_parallel(expert_model_parallel_size=world, expert_tensor_parallel_size=1, backend="gloo")
    cfg = ModelConfig(num_layers=2, hidden_size=32, num_attention_heads=2, num_query_groups=2, kv_channels=16, ffn_hidden_size=64,
                      vocab_size=64, num_experts=4, moe_ffn_hidden_size=16, moe_router_topk=2, tie_word_embeddings=False)
    args = namespace_from_dict(dict(expert_model_parallel_size=world, bf16=False, seed=rank + 5, untie_embeddings_and_output_weights=True))
    apply_to_args(cfg, args)
    model = TrainModel(args, device=torch.device("cpu"), with_optimizer=False)
    tensors = er.collect_expert_tensors(model)
    assert len(tensors) == 2 * 4 * 2  # layers x experts x (fc1, fc2), each listed once with its global expert id
    targets = [((s + 1) % world,) for s in range(world)]  # engine shard s lives on rank s + 1
    rounds = er.plan_expert_transfers(tensors, cfg.num_experts, targets, buffer_size=1 << 20)
    from slime_b200.backends.train.checkpoint import global_param_name

    local = {global_param_name(n, p): p.detach() for n, p in model.named_parameters() if getattr(p, "is_expert", False)}
    received = {}
    for rnd in rounds:
        er.run_round(rnd, rank, local.__getitem__, received.__setitem__)
    per = cfg.num_experts // world
    mine = [t for t in tensors if targets[t.layer_expert[1] // per][0] == rank]
    assert sorted(received) == sorted(t.name for t in mine)
    # values: the sender's tensors were drawn from a rank-dependent seed; compare checksums through an all-gather
    sums = {n: float(v.double().sum()) for n, v in local.items()}
    everyone = [None] * world
    dist.all_gather_object(everyone, sums)
    truth = {k: v for part in everyone for k, v in part.items()}
    for n, v in received.items():
        assert abs(float(v.double().sum()) - truth[n]) < 1e-9, n


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    mode = os.environ.get("MODE", "cp")
    {"cp": check_cp, "dp": check_dp, "tp": check_tp, "reload": check_reload, "expert_route": check_expert_route}[mode](rank, world)
    dist.barrier()
    if rank == 0:
        print(f"RESULT ok mode={mode} world={world}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
