"""Train/inference mismatch correction: importance weights, rejection masks and mismatch metrics.

The rollout engine and the trainer never produce bit-identical log-probs (different kernels, batch shapes, quantised
rollout weights). This module corrects the policy-gradient loss for that gap. It plugs into the loss as

    --use-tis --custom-tis-function-path slime_b200.utils.mis.compute_mis_weights_with_cp --custom-config-path mis.yaml

Configuration (fields of ``args``; the YAML supplies them):
  use_tis, tis_level (token | sequence | geometric), tis_mode (truncate | clip | mask), tis_lower_bound, tis_upper_bound
  use_rs, rs_level, rs_lower_bound, rs_upper_bound, rs_veto_threshold, tis_batch_normalize

Definitions, per sequence with loss mask m and d_t = log pi_train(t) - log pi_rollout(t):
  level token: r_t = d_t; sequence: r_t = sum_t m d; geometric: r_t = mean_t m d   (clamped to +-20 before exp)
  truncate: w = min(exp r, upper); clip: w = clamp(exp r, lower, upper); mask: w = exp r, tokens outside the
  bounds leave the loss mask. Rejection sampling removes tokens whose (rs-level) ratio leaves [rs_lower, rs_upper]
  and whole sequences that contain a token with exp(d_t) < rs_veto_threshold. Optionally all weights are divided by
  their batch mean. Weights and masks carry no gradient.

All sequences of the micro-batch are processed as ONE flat tensor with segment reductions (``index_add_`` /
``scatter_reduce_``), so the cost is a handful of kernels regardless of how many samples there are; the reference
implementation loops over samples in Python. Metrics come back token-shaped (one value per token, sequence-level
quantities repeated) because the caller reduces them with the per-sample mean.
Parity: examples/train_infer_mismatch_helper/mis.py:82-451.
"""

from __future__ import annotations

from typing import Any

import torch

SAFETY_BOUND = 20.0


class _Segments:
    """Segment reductions over a flat tensor of concatenated sequences."""

    def __init__(self, lengths: list[int], device):
        self.n = len(lengths)
        self.lengths = lengths
        self.ids = torch.repeat_interleave(torch.arange(self.n, device=device),
                                           torch.tensor(lengths, device=device, dtype=torch.long))  # fmt: skip

    def sum(self, x: torch.Tensor) -> torch.Tensor:
        return torch.zeros(self.n, dtype=x.dtype, device=x.device).index_add_(0, self.ids, x)

    def reduce(self, x: torch.Tensor, how: str, init: float) -> torch.Tensor:
        out = torch.full((self.n,), init, dtype=x.dtype, device=x.device)
        return out.scatter_reduce_(0, self.ids, x, reduce=how, include_self=True)

    def expand(self, per_seq: torch.Tensor) -> torch.Tensor:
        return per_seq[self.ids]

    def split(self, x: torch.Tensor) -> list[torch.Tensor]:
        return list(x.split(self.lengths))


def _bounds(args):
    lower = args.tis_lower_bound if getattr(args, "tis_lower_bound", None) is not None else 1.0 / args.tis_upper_bound
    rs_lo = args.rs_lower_bound if getattr(args, "rs_lower_bound", None) is not None else lower
    rs_hi = args.rs_upper_bound if getattr(args, "rs_upper_bound", None) is not None else args.tis_upper_bound
    return lower, rs_lo, rs_hi


def _level_log_ratio(d: torch.Tensor, m: torch.Tensor, seg: _Segments, level: str) -> torch.Tensor:
    if level == "token":
        return d
    total = seg.sum(d * m)
    if level == "sequence":
        return seg.expand(total)
    if level == "geometric":
        return seg.expand(total / seg.sum(m).clamp_min(1))
    raise ValueError(f"invalid level: {level}")


def mismatch_metrics(train: torch.Tensor, rollout: torch.Tensor, m: torch.Tensor, seg: _Segments) -> dict[str, torch.Tensor]:
    """Perplexities, KL estimators and chi-square divergences between the two policies (token-shaped)."""
    cnt = seg.sum(m).clamp_min(1)
    mean_train, mean_roll = seg.expand(seg.sum(train * m) / cnt), seg.expand(seg.sum(rollout * m) / cnt)
    d = train - rollout
    diff = mean_roll - mean_train
    rho = torch.exp(d.clamp(-SAFETY_BOUND, SAFETY_BOUND))
    chi2_tok = seg.expand(seg.sum(rho.square() * m) / cnt - 1.0)
    chi2_seq = torch.exp(2.0 * seg.expand(seg.sum(d * m)).clamp(-SAFETY_BOUND, SAFETY_BOUND)) - 1.0
    return {"training_log_ppl": -mean_train, "training_ppl": torch.exp(-mean_train), "rollout_log_ppl": -mean_roll,
            "rollout_ppl": torch.exp(-mean_roll), "kl": -d, "k3_kl": torch.exp(d) - d - 1, "log_ppl_diff": diff,
            "log_ppl_abs_diff": diff.abs(), "ppl_ratio": torch.exp(diff), "chi2_token": chi2_tok, "chi2_seq": chi2_seq}  # fmt: skip


def _mask_mode(w, m, lo, hi, metrics, prefix):
    inside = (w >= lo) & (w <= hi)
    cnt = m.sum().clamp_min(1)
    metrics[f"{prefix}mask_fraction_low"] = ((w < lo).float() * m).sum().div(cnt).expand_as(w)
    metrics[f"{prefix}mask_fraction_high"] = ((w > hi).float() * m).sum().div(cnt).expand_as(w)
    return m * inside.float()


def compute_mis_weights(args, *, train_log_probs: list[torch.Tensor], rollout_log_probs: list[torch.Tensor],
                        loss_masks: list[torch.Tensor]):  # fmt: skip
    """-> (weights per sequence | None, modified loss masks per sequence, metrics {name: [token-shaped per sequence]})."""
    assert len(train_log_probs) == len(rollout_log_probs) == len(loss_masks), "one entry per sequence in every list"
    for i, (a, b, c) in enumerate(zip(train_log_probs, rollout_log_probs, loss_masks)):
        assert a.shape == b.shape == c.shape, f"sequence {i}: shapes differ: {a.shape} {b.shape} {c.shape}"
    if not train_log_probs:
        return ([] if args.use_tis else None), [], {}
    seg = _Segments([t.numel() for t in train_log_probs], train_log_probs[0].device)
    train, rollout = torch.cat(train_log_probs).detach().float(), torch.cat(rollout_log_probs).detach().float()
    m = torch.cat(loss_masks).float()
    metrics = mismatch_metrics(train, rollout, m, seg)
    if not args.use_tis:
        return None, loss_masks, {k: seg.split(v) for k, v in metrics.items()}
    lower, rs_lo, rs_hi = _bounds(args)
    d = train - rollout
    new_mask = m.clone()

    r_tis = _level_log_ratio(d, m, seg, args.tis_level)
    w = torch.exp(r_tis.clamp(-SAFETY_BOUND, SAFETY_BOUND))
    metrics["tis_weight_before_bound"] = w
    cnt = m.sum().clamp_min(1)
    if args.tis_mode == "truncate":
        metrics["tis_truncate_fraction"] = ((w > args.tis_upper_bound).float() * m).sum().div(cnt).expand_as(w)
        w = w.clamp(max=args.tis_upper_bound)
    elif args.tis_mode == "clip":
        metrics["tis_clip_fraction_low"] = ((w < lower).float() * m).sum().div(cnt).expand_as(w)
        metrics["tis_clip_fraction_high"] = ((w > args.tis_upper_bound).float() * m).sum().div(cnt).expand_as(w)
        w = w.clamp(lower, args.tis_upper_bound)
    elif args.tis_mode == "mask":
        new_mask = _mask_mode(w, new_mask, lower, args.tis_upper_bound, metrics, "tis_")
    else:
        raise ValueError(f"unsupported tis_mode: {args.tis_mode}")
    metrics["tis_weight_after_bound"] = w

    if getattr(args, "use_rs", False):
        r_rs = r_tis if args.rs_level == args.tis_level else _level_log_ratio(d, m, seg, args.rs_level)
        new_mask = _mask_mode(torch.exp(r_rs.clamp(-SAFETY_BOUND, SAFETY_BOUND)), new_mask, rs_lo, rs_hi, metrics, "rs_")
        veto = getattr(args, "rs_veto_threshold", None)
        if veto is not None:
            # a sequence survives only if none of its trained tokens has a ratio below the threshold
            bad = ((d < torch.log(torch.tensor(float(veto), device=d.device))) & (m > 0)).float()
            vetoed = seg.sum(bad) > 0
            metrics["rs_veto_fraction"] = vetoed.float().mean().expand_as(w)
            new_mask = new_mask * seg.expand((~vetoed).float())
    metrics["is_ratio_mean_after_tis_rs"] = w

    if getattr(args, "tis_batch_normalize", False):
        if args.tis_level == "token":
            mean = (w * m).sum() / m.sum().clamp_min(1)
        elif args.tis_level == "sequence":
            mean = (seg.sum(w * m) / seg.sum(m).clamp_min(1)).mean()
        else:
            raise ValueError(f"batch normalisation is not defined for tis_level {args.tis_level}")
        factor = torch.where(mean > 1e-8, mean, torch.ones_like(mean))
        w = w / factor
        metrics["batch_norm_factor"] = factor.expand_as(w)

    per_cnt = seg.sum(m).clamp_min(1)
    metrics["is_ratio_mean_final"] = seg.expand(seg.sum(w * m) / per_cnt)
    metrics["is_ratio_min_final"] = seg.expand(seg.reduce(torch.where(m > 0, w, torch.full_like(w, float("inf"))), "amin", float("inf")))
    metrics["is_ratio_max_final"] = seg.expand(seg.reduce(torch.where(m > 0, w, torch.full_like(w, float("-inf"))), "amax", float("-inf")))
    return seg.split(w.detach()), seg.split(new_mask.detach()), {k: seg.split(v.detach()) for k, v in metrics.items()}


def compute_mis_weights_with_cp(args, *, pg_loss: torch.Tensor, train_log_probs: list[torch.Tensor],
                                rollout_log_probs: list[torch.Tensor], loss_masks: list[torch.Tensor],
                                total_lengths: list[int], response_lengths: list[int], **kwargs: Any):  # fmt: skip
    """The ``--custom-tis-function-path`` entry: context-parallel shards are gathered to whole responses, weighted, and
    sliced back. -> (pg_loss * weights (flat), modified masks (whole responses), metrics (flat, ``mis_`` prefix))."""
    from slime_b200.backends.train.cp_utils import all_gather_with_cp, slice_log_prob_with_cp

    full_roll = [all_gather_with_cp(x, t, r) for x, t, r in zip(rollout_log_probs, total_lengths, response_lengths)]
    full_train = [all_gather_with_cp(x, t, r) for x, t, r in zip(train_log_probs, total_lengths, response_lengths)]
    weights, masks, metrics = compute_mis_weights(args, train_log_probs=full_train, rollout_log_probs=full_roll,
                                                  loss_masks=loss_masks)  # fmt: skip

    def local(values: list[torch.Tensor]) -> torch.Tensor:
        return torch.cat([slice_log_prob_with_cp(v, t, r) for v, t, r in zip(values, total_lengths, response_lengths)], dim=0)

    if weights is not None:
        pg_loss = pg_loss * local(weights)
    return pg_loss, masks, {f"mis_{k}": local(v) for k, v in metrics.items()}
