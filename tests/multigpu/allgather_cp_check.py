"""Run under torchrun with 2 gloo ranks: all-gather context parallelism of a sparse-latent-attention model.

The micro-batch's concatenated stream is cut into two contiguous pieces. Checked against the same model run on the
whole stream by one rank: (1) this rank's logits rows, (2) parameter gradients summed over the two ranks, (3) the
response log-probs after the redistribution into zig-zag pieces, (4) a top-p keep mask applied to the right rows.
"""

import os
import sys
from argparse import Namespace

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from slime_b200.backends.train import loss as L
    from slime_b200.backends.train.cp_utils import ZigZag
    from slime_b200.backends.train.data import DataIterator, get_batch
    from slime_b200.models import mixers
    from slime_b200.models.config import ModelConfig
    from slime_b200.models.gpt import GPTModel, PackedSeqParams
    from slime_b200.parallel import state as mpu

    mpu.initialize_model_parallel(1, 1, None, world, 1, 1, backend="gloo")
    kind = os.environ.get("ALLGATHER_CP_MODEL", "dsa")
    extra = dict(index_topk=5, index_n_heads=8, index_head_dim=8, index_topk_freq=2, index_skip_topk_offset=1) if kind == "dsa" else {}
    cfg = ModelConfig(num_layers=3, hidden_size=64, num_attention_heads=4, num_query_groups=4, kv_channels=16, ffn_hidden_size=128,
                      vocab_size=96, rotary_base=1e4, tie_word_embeddings=False, multi_latent_attention=True, q_lora_rank=24,
                      kv_lora_rank=16, qk_head_dim=8, qk_pos_emb_head_dim=4, v_head_dim=12, rotary_interleaved=True, **extra)  # fmt: skip
    model = GPTModel(cfg, dtype=torch.float32, device="cpu", seed=11)  # same weights on both ranks
    g = torch.Generator().manual_seed(5)
    lengths, responses = [13, 7, 22], [6, 3, 9]
    samples = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in lengths]
    data = {"tokens": samples, "total_lengths": lengths, "response_lengths": responses,
            "loss_masks": [torch.ones(r) for r in responses]}  # fmt: skip

    # ---- reference: the whole stream on one rank
    real_size = mpu.get_context_parallel_world_size
    mpu.get_context_parallel_world_size = lambda: 1
    ref_batch = get_batch(DataIterator(data, [[0, 1, 2]]), list(data), pad_multiplier=4 * world)  # the same padded stream
    ref_logits = model(ref_batch["tokens"], ref_batch["position_ids"], packed_seq_params=ref_batch["packed_seq_params"])[0]
    wts = torch.randn(ref_logits.shape, generator=g)
    model.zero_grad()
    (ref_logits * wts).sum().backward()
    ref_grads = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
    args = Namespace(rollout_temperature=1.0, allgather_cp=True, log_probs_chunk_size=-1)
    _, ref_res = L.get_log_probs_and_entropy(ref_logits.detach()[None], args=args, unconcat_tokens=samples, total_lengths=lengths,
                                             response_lengths=responses, with_entropy=True)  # fmt: skip
    mpu.get_context_parallel_world_size = real_size

    # ---- all-gather context parallelism
    mixers.set_allgather_cp(True)
    batch = get_batch(DataIterator(data, [[0, 1, 2]]), list(data), pad_multiplier=4, allgather_cp=True)
    T_local = batch["tokens"].shape[1]
    assert T_local * world == ref_batch["tokens"].shape[1] and batch["packed_seq_params"].cu_seqlens.tolist() == ref_batch["packed_seq_params"].cu_seqlens.tolist()
    piece = slice(rank * T_local, (rank + 1) * T_local)
    assert torch.equal(batch["tokens"][0], ref_batch["tokens"][0, piece]) and torch.equal(batch["full_loss_masks"][0], ref_batch["full_loss_masks"][0, piece])
    logits = model(batch["tokens"], batch["position_ids"], packed_seq_params=batch["packed_seq_params"])[0]
    err = float((logits - ref_logits[piece]).abs().max())
    assert err < 1e-5, err
    model.zero_grad()
    (logits * wts[piece]).sum().backward()
    worst = 0.0
    for n, p in model.named_parameters():
        if n not in ref_grads:
            continue
        gsum = (p.grad if p.grad is not None else torch.zeros_like(p)).clone()
        dist.all_reduce(gsum)
        worst = max(worst, float((gsum - ref_grads[n]).abs().max() / (ref_grads[n].abs().max() + 1e-6)))
    assert worst < 1e-4, worst
    _, res = L.get_log_probs_and_entropy(logits.detach()[None], args=args, unconcat_tokens=samples, total_lengths=lengths,
                                         response_lengths=responses, with_entropy=True)  # fmt: skip
    for key in ("log_probs", "entropy"):
        for got, want, tl, rl in zip(res[key], ref_res[key], lengths, responses):
            s0, s1 = ZigZag.plan(tl, rl).response_slices()
            assert torch.allclose(got, torch.cat([want[s0], want[s1]]), atol=1e-5), (key, rank)
    # a kept set that contains only the sampled token: log-prob 0 on exactly this rank's response rows
    ids = [t[-r:].tolist() for t, r in zip(samples, responses)]
    offs = [list(range(r + 1)) for r in responses]
    _, kept = L.get_log_probs_and_entropy(logits.detach()[None], args=args, unconcat_tokens=samples, total_lengths=lengths,
                                          response_lengths=responses, rollout_top_p_token_ids=ids, rollout_top_p_token_offsets=offs)  # fmt: skip
    assert all(float(x.abs().max()) < 1e-6 for x in kept["log_probs"] if x.numel())
    # values of a critic head travel the same way
    _, vals = L.get_values(logits.detach()[None, :, :1], args=args, unconcat_tokens=samples, total_lengths=lengths, response_lengths=responses)
    start = 0
    for got, tl, rl in zip(vals["values"], lengths, responses):
        want = ref_logits.detach()[start + tl - rl - 1 : start + tl - 1, 0]
        s0, s1 = ZigZag.plan(tl, rl).response_slices()
        assert torch.allclose(got, torch.cat([want[s0], want[s1]]), atol=1e-5)
        start += tl
    if rank == 0:
        print(f"RESULT ok world={world} model={kind} logits_err={err:.1e} grad_rel_err={worst:.1e}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
