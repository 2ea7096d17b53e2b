"""Per-rollout data-parallel / micro-batch scheduling (pure Python).

Pack first, distribute second (parity: slime/utils/dp_schedule.py:82-209):
rollouts are grouped into steps of ``global_batch_size`` rollouts (samples that
share a rollout id stay together), each step's samples are packed into
micro-batches (first-fit on tokens, Karmarkar-Karp on FLOPs, or fixed size),
the count is aligned to ``dp * vpp_group`` and the micro-batches are dealt to
the DP ranks.

Guarantees: identical micro-batch count on every rank per step; only a single
over-long sample may exceed the token cap; kept samples are placed exactly
once; ``micro_batch_indices[r]`` tiles ``range(len(partitions[r]))``.
"""

from __future__ import annotations

from typing import Any

from slime_b200.utils.flops_utils import calculate_fwd_flops
from slime_b200.utils.seqlen_balancing import expand_bins_by_splitting, first_fit_pack, get_seqlen_balanced_partitions


def _flops_of(lengths, args):
    return [calculate_fwd_flops([n], args) for n in lengths]


def _pack(lengths, args, cap, balance_by_flops):
    if not args.use_dynamic_batch_size:
        mbs = args.micro_batch_size
        assert mbs is not None
        return [list(range(s, min(s + mbs, len(lengths)))) for s in range(0, len(lengths), mbs)]
    assert cap is not None
    if not balance_by_flops:
        return first_fit_pack(lengths, cap)
    want = max(1, -(-sum(lengths) // cap))
    if want >= len(lengths):
        return [[i] for i in range(len(lengths))]
    # FLOPs balancing trades the hard token cap for equal work per micro-batch.
    return get_seqlen_balanced_partitions(_flops_of(lengths, args), want, equal_size=False)


def build_dp_schedule(
    args: Any,
    train_parallel_config: dict,
    total_lengths: list[int],
    *,
    global_batch_size: int,
    rollout_indices: list[int],
):
    """Return ``(partitions, micro_batch_indices, num_microbatches, global_batch_sizes)``.

    ``partitions[r]`` are global sample positions owned by DP rank ``r``;
    ``micro_batch_indices[r][k]`` are positions into ``partitions[r]``.
    """
    dp = train_parallel_config["dp_size"]
    cp = train_parallel_config["cp_size"]
    vpp = train_parallel_config["vpp_size"]
    group = train_parallel_config["microbatch_group_size_per_vp_stage"]
    cap = None
    if args.use_dynamic_batch_size:
        assert args.max_tokens_per_gpu is not None
        cap = args.max_tokens_per_gpu * cp
    align = dp * (group if vpp > 1 else 1)

    by_rollout: dict[int, list[int]] = {}
    for pos, rid in enumerate(rollout_indices):
        by_rollout.setdefault(rid, []).append(pos)
    rids = list(by_rollout)
    steps = len(rids) // global_batch_size
    assert steps >= 1, (
        f"num_rollouts ({len(rids)}) < global_batch_size ({global_batch_size}); need at least one rollout per step."
    )

    partitions = [[] for _ in range(dp)]
    mb_indices = [[] for _ in range(dp)]
    num_mb, gbs_out = [], []
    balance_by_flops = getattr(args, "balance_by_flops", False)
    for s in range(steps):
        chosen = rids[s * global_batch_size : (s + 1) * global_batch_size]
        positions = [p for rid in chosen for p in by_rollout[rid]]
        lengths = [total_lengths[p] for p in positions]
        gbs_out.append(global_batch_size)
        assert len(positions) >= dp, f"step {s}: {len(positions)} samples < dp_size {dp}"

        bins = _pack(lengths, args, cap, balance_by_flops)
        want = max(-(-len(bins) // align) * align, align)
        if want != len(bins):
            if not args.use_dynamic_batch_size:
                raise AssertionError(
                    f"static batching: {len(bins)} micro-batches is not a multiple of dp_size*vpp_group ({align}); "
                    f"step_size={len(positions)}, micro_batch_size={args.micro_batch_size}"
                )
            expand_bins_by_splitting(bins, want, lengths)
            assert len(bins) == want, (
                f"dynamic batching: only {len(bins)} micro-batches after maximal splitting, need {want} "
                f"(step {s} has {len(positions)} samples)"
            )
        K = len(bins)
        num_mb.append(K // dp)

        if getattr(args, "balance_data", False):
            w = _flops_of(lengths, args)
            deal = get_seqlen_balanced_partitions([sum(w[i] for i in b) for b in bins], dp, equal_size=True)
        else:
            deal = [list(range(r, K, dp)) for r in range(dp)]

        for r in range(dp):
            for b in deal[r]:
                base = len(partitions[r])
                partitions[r].extend(positions[i] for i in bins[b])
                mb_indices[r].append(list(range(base, base + len(bins[b]))))
    return partitions, mb_indices, num_mb, gbs_out
