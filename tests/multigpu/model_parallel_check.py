"""Run under torchrun: the trainer model under a parallel layout equals a single-rank plain-PyTorch model.

    MODE=tp | tp_sp | pp | pp_vpp | ep | dp | tp_dp | cp | tp_sp_moe | tp_ep_moe   DEVICE=cpu (gloo, fp32) | cuda (nccl, bf16)

Every rank builds the same full set of weights from one seed (Megatron names, full shapes), keeps the shard its
coordinates own, and runs forward + backward of a weighted next-token log-likelihood over a few packed micro-batches
through the pipeline schedule and ``finalize_grads``. The oracle is a plain fp32 PyTorch transformer written out in
this file (it shares no code with ``GPTModel``) run on the full weights and all micro-batches. Compared: the loss, the
global gradient norm, and every local gradient shard against the oracle's gradient of the same parameter slice.
The counterpart in the reference is tests/test_qwen3_0.6B_parallel_check.py:12-21,103-128.
"""

import os
import sys
from argparse import Namespace

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

LAYOUTS = {  # mode -> (tp, pp, vpp, ep, sequence_parallel); "cp" is context parallel over the whole world
    "tp": (2, 1, None, 1, False), "tp_sp": (2, 1, None, 1, True), "pp": (1, 2, None, 1, False),
    "pp_vpp": (1, 2, 2, 1, False), "ep": (1, 1, None, 2, False), "dp": (1, 1, None, 1, False),
    "tp_dp": (2, 1, None, 1, True), "cp": (1, 1, None, 1, False), "tp_sp_moe": (2, 1, None, 1, True),
    "tp_ep_moe": (2, 1, None, 2, True),
}  # fmt: skip


def full_weights(cfg, seed):
    """name -> full fp32 tensor, in the trainer's in-memory layouts at tp = 1 (qkv rows [q | k | v], fc1 rows [gate; up])."""
    g = torch.Generator().manual_seed(seed)
    h, d, hq, hkv, f, V = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_query_groups, cfg.ffn_hidden_size, cfg.padded_vocab_size

    def mat(*shape, std=0.05):
        return torch.randn(*shape, generator=g) * std

    w = {"embedding.word_embeddings.weight": mat(V, h), "decoder.final_layernorm.weight": 1 + mat(h),
         "output_layer.weight": mat(V, h)}  # fmt: skip
    for i in range(cfg.num_layers):
        p = f"decoder.layers.{i}."
        w[p + "self_attention.linear_qkv.weight"] = mat((hq + 2 * hkv) * d, h)
        w[p + "self_attention.linear_qkv.layer_norm_weight"] = 1 + mat(h)
        w[p + "self_attention.q_layernorm.weight"] = 1 + mat(d)
        w[p + "self_attention.k_layernorm.weight"] = 1 + mat(d)
        w[p + "self_attention.linear_proj.weight"] = mat(h, hq * d)
        if cfg.num_experts:
            w[p + "mlp.pre_mlp_layernorm.weight"] = 1 + mat(h)
            w[p + "mlp.router.weight"] = mat(cfg.num_experts, h, std=0.5)
            for e in range(cfg.num_experts):
                w[p + f"mlp.experts.linear_fc1.weight{e}"] = mat(2 * cfg.moe_ffn_hidden_size, h)
                w[p + f"mlp.experts.linear_fc2.weight{e}"] = mat(h, cfg.moe_ffn_hidden_size)
        else:
            w[p + "mlp.linear_fc1.weight"] = mat(2 * f, h)
            w[p + "mlp.linear_fc1.layer_norm_weight"] = 1 + mat(h)
            w[p + "mlp.linear_fc2.weight"] = mat(h, f)
    return w


def oracle_loss(cfg, w, samples, weights):
    """Plain fp32 transformer over each sample separately; returns sum_t weight_t * log p(token_{t+1} | prefix)."""
    h, d, hq, hkv = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_query_groups

    def norm(x, g):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.norm_epsilon) * g

    def rope(x, pos):  # x [T, H, d], rotate-half
        inv = 1.0 / (cfg.rotary_base ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
        ang = pos.double()[:, None] * inv[None]
        c, s = ang.cos().float()[:, None], ang.sin().float()[:, None]
        lo, hi = x[..., : d // 2], x[..., d // 2 :]
        return torch.cat([lo * c - hi * s, hi * c + lo * s], -1)

    total = 0.0
    for ids, wt in zip(samples, weights):
        T = ids.numel()
        pos = torch.arange(T)
        x = w["embedding.word_embeddings.weight"][ids]
        for i in range(cfg.num_layers):
            p = f"decoder.layers.{i}."
            a = norm(x, w[p + "self_attention.linear_qkv.layer_norm_weight"]) @ w[p + "self_attention.linear_qkv.weight"].t()
            q, k, v = a.split([hq * d, hkv * d, hkv * d], -1)
            q = rope(norm(q.view(T, hq, d), w[p + "self_attention.q_layernorm.weight"]), pos)
            k = rope(norm(k.view(T, hkv, d), w[p + "self_attention.k_layernorm.weight"]), pos)
            v = v.view(T, hkv, d)
            k, v = k.repeat_interleave(hq // hkv, 1), v.repeat_interleave(hq // hkv, 1)
            att = torch.einsum("thd,shd->hts", q, k) / d**0.5
            att = att.masked_fill(~torch.ones(T, T, dtype=torch.bool).tril(), float("-inf")).softmax(-1)
            ctx = torch.einsum("hts,shd->thd", att, v).reshape(T, hq * d)
            x = x + ctx @ w[p + "self_attention.linear_proj.weight"].t()
            if cfg.num_experts:
                n = norm(x, w[p + "mlp.pre_mlp_layernorm.weight"])
                logits = n @ w[p + "mlp.router.weight"].t()
                top, idx = logits.topk(cfg.moe_router_topk, -1)
                probs = top.softmax(-1)
                out = torch.zeros_like(x)
                for e in range(cfg.num_experts):
                    sel = (idx == e)
                    rows = sel.any(-1)
                    if rows.any():
                        gu = n[rows] @ w[p + f"mlp.experts.linear_fc1.weight{e}"].t()
                        g_, u_ = gu.chunk(2, -1)
                        y = (torch.nn.functional.silu(g_) * u_) @ w[p + f"mlp.experts.linear_fc2.weight{e}"].t()
                        out[rows] = out[rows] + y * (probs * sel)[rows].sum(-1, keepdim=True)
                x = x + out
            else:
                n = norm(x, w[p + "mlp.linear_fc1.layer_norm_weight"])
                g_, u_ = (n @ w[p + "mlp.linear_fc1.weight"].t()).chunk(2, -1)
                x = x + (torch.nn.functional.silu(g_) * u_) @ w[p + "mlp.linear_fc2.weight"].t()
        hfin = norm(x, w["decoder.final_layernorm.weight"])
        lsm = torch.log_softmax(hfin @ w["output_layer.weight"].t(), -1)
        lp = lsm[:-1].gather(-1, ids[1:, None]).squeeze(-1)
        total = total + (lp * wt[1:]).sum()
    return total


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    mode = os.environ.get("MODE", "tp")
    cuda = os.environ.get("DEVICE", "cpu") == "cuda"
    if cuda:
        local = int(os.environ["LOCAL_RANK"])
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        dev = torch.device("cuda", local)
    else:
        dist.init_process_group("gloo")
        dev = torch.device("cpu")
    from slime_b200.backends.train.data import DataIterator
    from slime_b200.backends.train.model import TrainModel
    from slime_b200.models.config import ModelConfig, apply_to_args
    from slime_b200.parallel import pipeline, state as mpu
    from slime_b200.utils.arguments import namespace_from_dict
    from slime_b200.weight_sync import convert

    tp, pp, vpp, ep, sp = LAYOUTS[mode]
    cp = world if mode == "cp" else 1
    mpu.initialize_model_parallel(tp, pp, vpp, cp, ep, 1, **({} if cuda else {"backend": "gloo"}))
    moe = mode in ("ep", "tp_sp_moe", "tp_ep_moe")
    cfg = ModelConfig(num_layers=4, hidden_size=128, num_attention_heads=4, num_query_groups=2, kv_channels=64,
                      ffn_hidden_size=256, vocab_size=512, rotary_base=1e4, tie_word_embeddings=False, qk_layernorm=True,
                      num_experts=4 if moe else None, moe_ffn_hidden_size=128 if moe else None, moe_router_topk=2)  # fmt: skip
    args = namespace_from_dict(dict(
        tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp, virtual_pipeline_model_parallel_size=vpp,
        expert_model_parallel_size=ep, sequence_parallel=sp, bf16=cuda, seed=11, lr=1e-3, fused_dp_step=False,
        untie_embeddings_and_output_weights=True, data_pad_size_multiplier=8 if not cuda else 128,
    ))  # fmt: skip
    apply_to_args(cfg, args)
    model = TrainModel(args, device=dev, with_optimizer=False)

    # ---- weights: the same full set everywhere, each parameter keeps its shard
    W = full_weights(cfg, 5)
    tpr, epr = mpu.get_tensor_model_parallel_rank(), mpu.get_expert_model_parallel_rank()
    from slime_b200.backends.train.checkpoint import global_param_name

    local_slices = {}  # local name -> the oracle-side view of this shard (for the gradient comparison)
    with torch.no_grad():
        for name, p in model.named_parameters():
            gname = global_param_name(name, p)
            full = W[gname]
            if getattr(p, "tensor_model_parallel", False) and not getattr(p, "is_expert", False):
                if gname in ("embedding.word_embeddings.weight", "output_layer.weight"):
                    shard = full.chunk(tp, 0)[tpr]
                else:
                    shard = convert.shard_for_tp(cfg, gname, full, p.partition_dim, getattr(p, "partition_stride", 1), tp, tpr)
            else:
                shard = full
            assert shard.shape == p.shape, (name, shard.shape, p.shape)
            p.copy_(shard.to(p.dtype))
            local_slices[name] = (gname, p)
    if cuda:  # the oracle sees the weights as the bf16 model holds them
        W = {k: v.to(torch.bfloat16).float() for k, v in W.items()}

    # ---- data: this DP rank's samples (every model-parallel rank of a DP group builds the same micro-batches)
    dp, dpr = mpu.get_data_parallel_world_size(), mpu.get_data_parallel_rank()
    dpcp = mpu.get_data_parallel_world_size(with_context_parallel=True)  # the group gradients are reduced over
    g = torch.Generator().manual_seed(100 + dpr)
    lens = [37, 64, 19, 50, 23, 41]
    samples = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in lens]
    wts = [torch.rand(n, generator=g) for n in lens]
    mbs = [[0, 1], [2, 3], [4], [5]]
    data = {"tokens": [s.to(dev) for s in samples], "total_lengths": lens, "response_lengths": [n - 1 for n in lens]}
    it = DataIterator(data, mbs)

    def forward_step(batch, chunk, input_tensor):
        chunk.set_input_tensor(input_tensor)
        out = chunk(batch["tokens"], batch["position_ids"], packed_seq_params=batch["packed_seq_params"])
        if not chunk.post_process:
            return out, None
        from slime_b200.utils.ppo_utils import calculate_log_probs_and_entropy

        logits = out[0]
        idx = batch["_sample_ids"]
        loss, off = 0.0, 0
        cu_local = batch["packed_seq_params"].local_cu_seqlens.tolist()
        pos_all = batch["position_ids"][0].long()
        for j, i in enumerate(idx):
            n = lens[i]
            a, b = cu_local[j], cu_local[j + 1]  # this rank's rows of the sample (all of them without context parallelism)
            pos = pos_all[a:b]  # their positions in the sample (zig-zag chunks under context parallelism)
            keep = pos + 1 < n  # the last token, and context-parallel padding, predict nothing
            tgt = samples[i].to(dev)[(pos + 1).clamp_max(n - 1)]
            lp, _ = calculate_log_probs_and_entropy(logits[a:b], tgt, mpu.get_tensor_model_parallel_group(), with_entropy=False)
            loss = loss + (lp * wts[i].to(dev)[(pos + 1).clamp_max(n - 1)] * keep).sum()
        return loss, {"loss": loss.detach()}

    # the batch builder does not say which samples it packed: wrap the iterator to remember them
    orig_next = it.get_next

    def get_next(keys):
        idx = it.micro_batch_indices[it.offset]
        b = orig_next(keys)
        b["_sample_ids"] = idx
        return b

    it.get_next = get_next
    model.zero_grad_buffer()
    model.train()
    logs = pipeline.run_forward_backward(model, it, len(mbs), forward_step, args)
    model.finalize_grads()

    # ---- oracle on every DP rank's data (cheap) so that every rank can compare
    Wg = {k: v.clone().requires_grad_() for k, v in W.items()}
    ref_loss = 0.0
    for r in range(dp):
        gr = torch.Generator().manual_seed(100 + r)
        s_r = [torch.randint(0, cfg.vocab_size, (n,), generator=gr) for n in lens]
        w_r = [torch.rand(n, generator=gr) for n in lens]
        ref_loss = ref_loss + oracle_loss(cfg, Wg, s_r, w_r)
    ref_loss.backward()

    rtol, atol = (3e-2, 3e-2) if cuda else (2e-4, 2e-5)
    # loss: last pipeline stage holds it; summed over DP
    mine = torch.zeros(1, dtype=torch.float64, device=dev)
    if mpu.is_pipeline_last_stage() and logs:
        mine += sum(float(l["loss"]) for l in logs)
    dist.all_reduce(mine, group=mpu.get_data_parallel_group(with_context_parallel=True))
    if mpu.is_pipeline_last_stage():
        torch.testing.assert_close(float(mine), float(ref_loss.detach()), rtol=rtol, atol=atol * 10)

    # gradients: every local shard against the oracle's slice. A flat buffer reduced over a group of one rank holds whole
    # gradients; one reduced over several ranks (data parallel, or expert-data parallel = the tensor-parallel ranks
    # when experts are not tensor-parallel) holds the sum over those ranks in each rank's shard of the buffer only.
    def oracle_slice(gname, p):
        gfull = Wg[gname].grad
        if getattr(p, "tensor_model_parallel", False) and not getattr(p, "is_expert", False):
            if gname in ("embedding.word_embeddings.weight", "output_layer.weight"):
                return gfull.chunk(tp, 0)[tpr]
            return convert.shard_for_tp(cfg, gname, gfull, p.partition_dim, getattr(p, "partition_stride", 1), tp, tpr)
        return gfull

    worst = 0.0
    sq = torch.zeros(1, dtype=torch.float64, device=dev)
    whole = all(b.group_size == 1 for b in model.buffers)
    for b in model.buffers:
        if b.group_size == 1:
            for name, p in zip(b.names, b.params):
                gname = global_param_name(name, p)
                want, got = oracle_slice(gname, p), p.main_grad.float().cpu()
                err = float((got - want).abs().max()) / max(float(want.abs().max()), 1e-6)
                worst = max(worst, err)
                assert err < (5e-2 if cuda else 2e-3), (name, err)
                own_tp = (not getattr(p, "tensor_model_parallel", False)) and tpr != 0 and not getattr(p, "is_expert", False)
                if not own_tp:  # replicated parameters count once
                    sq += got.double().pow(2).sum().to(dev)
        else:
            s0, e0 = b.shard_range()
            flat_ref = torch.zeros(b.numel)
            for (name, p), (ps, pe) in zip(zip(b.names, b.params), b.offsets):
                flat_ref[ps:pe] = oracle_slice(global_param_name(name, p), p).reshape(-1)
            got, want = b.grad_data[s0:e0].float().cpu(), flat_ref[s0:e0]
            err = float((got - want).abs().max()) / max(float(want.abs().max()), 1e-6)
            worst = max(worst, err)
            # bf16 router logits flip near-tie top-k choices of the random MoE: expert gradients then differ visibly
            assert err < ((0.3 if moe else 5e-2) if cuda else 2e-3), ("reduced shard", b.names[0], err)
    if whole:
        dist.all_reduce(sq)  # tp / pp / ep ranks hold disjoint parameters (replicated ones were counted once)
        ref_sq = sum(float(v.grad.double().pow(2).sum()) for v in Wg.values() if v.grad is not None)
        torch.testing.assert_close(float(sq) ** 0.5, ref_sq**0.5, rtol=rtol, atol=atol)
    dist.barrier()
    if rank == 0:
        print(f"RESULT ok mode={mode} world={world} device={dev.type} worst_grad_rel_err={worst:.2e}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
