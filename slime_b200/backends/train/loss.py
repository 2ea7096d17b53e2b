"""Loss library of the training backend.

Covers what slime/backends/megatron_utils/loss.py provides on top of Megatron:
log-prob / entropy extraction from packed logits (:513-604), values (:607-660),
advantage estimators (:704-881), TIS / icepop (:884-931), the policy loss with
GSPO / CISPO / OPSM / KL-loss / entropy bonus (:934-1173), the critic loss
(:1176-1230), SFT loss (:1233-1280) and the dispatcher (:1283-1383).

Scaling convention of this backend (the training loop sums micro-batch losses and
the DP reduction is a SUM): per-sample mode divides by the step's global batch size
(number of rollouts), per-token mode divides by the step's global token count.
"""

from __future__ import annotations

from argparse import Namespace
from collections.abc import Callable
from typing import Any

import torch
import torch.distributed as dist
import torch.nn.functional as F

from slime_b200.backends.train.cp_utils import (
    ZigZag,
    all_gather_with_cp,
    get_sum_of_sample_mean,
    local_loss_masks,
    slice_log_prob_with_cp,
)
from slime_b200.parallel import state as mpu
from slime_b200.utils.misc import load_function
from slime_b200.utils.ppo_utils import (
    calculate_log_probs_and_entropy,
    compute_approx_kl,
    compute_cispo_loss,
    compute_gspo_kl,
    compute_opsm_mask,
    compute_policy_loss,
    get_advantages_and_returns_batch,
    get_grpo_returns,
    get_reinforce_plus_plus_baseline_advantages,
    get_reinforce_plus_plus_returns,
)

RolloutBatch = dict

_CAPTURE = {"on": False, "store": {}}


def enable_log_prob_capture(flag: bool = True):
    _CAPTURE["on"] = flag
    _CAPTURE["store"] = {}


def drain_captured_log_probs() -> dict:
    out, _CAPTURE["store"] = _CAPTURE["store"], {}
    return out


def _maybe_capture_log_probs(batch, log_probs):
    if _CAPTURE["on"]:
        for idx, lp in zip(batch.get("sample_indices", range(len(log_probs))), log_probs):
            _CAPTURE["store"][int(idx)] = lp.detach().float().cpu()


# ------------------------------------------------------------ response iteration
def get_responses(logits, *, args, unconcat_tokens, total_lengths, response_lengths, max_seq_lens=None):
    """Yield ``(logits_rows, target_tokens)`` per sample for the response positions this rank holds.

    ``logits`` is ``[1, T, V/tp]`` (or ``[T, V/tp]``) over the packed micro-batch; row ``i`` of a
    sample predicts its token ``i+1``. Temperature is applied here. With zig-zag CP a sample's
    local rows are its two chunks laid out back to back in the packed stream.
    """
    logits = logits.squeeze(0) if logits.dim() == 3 else logits
    temp = getattr(args, "rollout_temperature", 1.0)
    if temp != 1.0:
        logits = logits / temp
    cp = mpu.get_context_parallel_world_size()
    if cp > 1 and getattr(args, "allgather_cp", False):
        # this rank holds one contiguous piece of the concatenated stream: a sample's local rows are one interval
        for (r0, r1, s0, s1), tokens, tl, rl in zip(allgather_cp_rows(total_lengths, response_lengths, logits.shape[0]),
                                                      unconcat_tokens, total_lengths, response_lengths):  # fmt: skip
            yield logits[r0:r1], tokens[tl - rl + s0 : tl - rl + s1]
        return
    end = 0
    for i, (tokens, tl, rl) in enumerate(zip(unconcat_tokens, total_lengths, response_lengths)):
        if cp == 1:
            end += tl
            start = end - rl
            yield logits[start - 1 : end - 1], tokens[-rl:]
        else:
            z = ZigZag.plan(tl, rl)
            base = end
            (l0a, l0b), (l1a, l1b) = z.logits
            c0 = z.chunks[0][0]
            c1 = z.chunks[1][0]
            rows0 = logits[base + (l0a - c0) : base + (l0b - c0)] if l0b > l0a else logits[0:0]
            rows1 = logits[base + z.chunk_size + (l1a - c1) : base + z.chunk_size + (l1b - c1)] if l1b > l1a else logits[0:0]
            t0 = tokens[z.tokens[0][0] : z.tokens[0][1]]
            t1 = tokens[z.tokens[1][0] : z.tokens[1][1]]
            end += 2 * z.chunk_size
            yield torch.cat([rows0, rows1], dim=0), torch.cat([t0, t1], dim=0)


def allgather_cp_rows(total_lengths, response_lengths, local_len: int):
    """Per sample ``(first local row, end local row, first response position, end response position)``: which rows of
    this rank's contiguous piece (``local_len`` rows of the concatenated stream) predict response tokens of the sample, and
    which response positions those are. Empty intervals are ``(0, 0, 0, 0)``."""
    lo = mpu.get_context_parallel_rank() * local_len
    hi = lo + local_len
    out, start = [], 0
    for tl, rl in zip(total_lengths, response_lengths):
        g0, g1 = start + tl - rl - 1, start + tl - 1  # stream rows whose next token is a response token
        s, e = max(g0, lo), min(g1, hi)
        out.append((s - lo, e - lo, s - g0, e - g0) if e > s else (0, 0, 0, 0))
        start += tl
    return out


def redistribute_allgather_cp(res: dict, total_lengths, response_lengths, local_len: int) -> None:
    """Per-sample response tensors computed on contiguous pieces -> the zig-zag pieces every reducer downstream expects:
    each rank places what it has into a zero vector of the sample's response length, one differentiable sum over the
    context-parallel group rebuilds the whole vectors, each rank then keeps its zig-zag rows. In place. (Same device as
    slime/backends/megatron_utils/loss.py:194-271 in the reference.)"""
    from slime_b200.backends.train.cp_utils import _AllReduceSum

    spans = allgather_cp_rows(total_lengths, response_lengths, local_len)
    for key, values in res.items():
        if not values or all(v is None for v in values):
            continue
        ref = next(v for v in values if v is not None)
        full = []
        for v, (_r0, _r1, s0, s1), rl in zip(values, spans, response_lengths):
            if v is None or s1 <= s0:
                full.append(ref.new_zeros(rl))
            else:
                full.append(F.pad(v, (s0, rl - s1)))
        whole = _AllReduceSum.apply(torch.cat(full), mpu.get_context_parallel_group())
        res[key] = [slice_log_prob_with_cp(x, tl, rl) for x, tl, rl in zip(whole.split(list(response_lengths)), total_lengths, response_lengths)]


def get_rollout_top_p_logprob_kwargs(args, batch) -> dict:
    """Top-p keep-mask replay is active when the rollout sampled with ``top_p != 1``."""
    if getattr(args, "rollout_top_p", 1.0) == 1.0 or not batch.get("rollout_top_p_token_ids"):
        return {}
    return {
        "rollout_top_p_token_ids": batch["rollout_top_p_token_ids"],
        "rollout_top_p_token_offsets": batch["rollout_top_p_token_offsets"],
    }


def _keep_mask_rows(ids, offsets, row_slices, vocab_lo, vocab_n, device):
    """Boolean ``[rows, V/tp]`` mask from the ragged kept-id lists for the given response rows."""
    rows = [r for sl in row_slices for r in range(sl.start, sl.stop)]
    mask = torch.zeros(len(rows), vocab_n, dtype=torch.bool, device=device)
    offs = torch.as_tensor(offsets).tolist()
    ids = torch.as_tensor(ids)
    for out_r, r in enumerate(rows):
        a, b = offs[r], offs[r + 1]
        if b == a:
            mask[out_r] = True  # empty span (tool tokens): nothing was filtered
            continue
        local = ids[a:b].long() - vocab_lo
        local = local[(local >= 0) & (local < vocab_n)]
        mask[out_r, local.to(device)] = True
    return mask


def get_log_probs_and_entropy(
    logits,
    *,
    args,
    unconcat_tokens,
    total_lengths,
    response_lengths,
    with_entropy: bool = False,
    non_loss_data: bool = True,
    max_seq_lens=None,
    rollout_top_p_token_ids=None,
    rollout_top_p_token_offsets=None,
    with_entropy_grad: bool = True,
):
    """Per-sample response log-probs (and entropies) from packed vocab-parallel logits."""
    tp_group = mpu.get_tensor_model_parallel_group()
    tp_rank = mpu.get_tensor_model_parallel_rank()
    allgather = mpu.get_context_parallel_world_size() > 1 and getattr(args, "allgather_cp", False)
    local_len = (logits.shape[1] if logits.dim() == 3 else logits.shape[0]) if allgather else 0
    spans = allgather_cp_rows(total_lengths, response_lengths, local_len) if allgather else None
    lps, ents = [], []
    for i, (rows, toks) in enumerate(
        get_responses(logits, args=args, unconcat_tokens=unconcat_tokens, total_lengths=total_lengths,
                      response_lengths=response_lengths, max_seq_lens=max_seq_lens)
    ):  # fmt: skip
        keep = None
        if rollout_top_p_token_ids is not None:
            rl, tl = response_lengths[i], total_lengths[i]
            if allgather:
                slices = (slice(spans[i][2], spans[i][3]),)
            else:
                slices = (slice(0, rl),) if mpu.get_context_parallel_world_size() == 1 else ZigZag.plan(tl, rl).response_slices()
            vp = rows.shape[-1]
            keep = _keep_mask_rows(rollout_top_p_token_ids[i], rollout_top_p_token_offsets[i], slices, tp_rank * vp, vp,
                                   rows.device)  # fmt: skip
        lp, en = calculate_log_probs_and_entropy(
            rows, toks, tp_group, with_entropy=with_entropy, chunk_size=getattr(args, "log_probs_chunk_size", -1),
            log_prob_keep_mask=keep, with_entropy_grad=with_entropy_grad,
        )  # fmt: skip
        lps.append(lp)
        if with_entropy:
            ents.append(en)
    res = {"log_probs": lps}
    if with_entropy:
        res["entropy"] = ents
    if allgather:
        redistribute_allgather_cp(res, total_lengths, response_lengths, local_len)
    return torch.empty(0, device=logits.device), res


def get_values(logits, *, args, unconcat_tokens, total_lengths, response_lengths, with_entropy=False, non_loss_data=True,
               max_seq_lens=None, **_):  # fmt: skip
    """Critic values for the response positions (value head output ``[1, T, 1]``)."""
    vals = []
    a = Namespace(**{**vars(args), "rollout_temperature": 1.0})
    for rows, _t in get_responses(logits, args=a, unconcat_tokens=unconcat_tokens, total_lengths=total_lengths,
                                  response_lengths=response_lengths, max_seq_lens=max_seq_lens):  # fmt: skip
        vals.append(rows.squeeze(-1).float())
    res = {"values": vals}
    if mpu.get_context_parallel_world_size() > 1 and getattr(args, "allgather_cp", False):
        redistribute_allgather_cp(res, total_lengths, response_lengths, logits.shape[1] if logits.dim() == 3 else logits.shape[0])
    return torch.empty(0, device=logits.device), res


# ------------------------------------------------------------------- advantages
def distributed_masked_whiten(values, mask, process_group=None, shift_mean=True, eps=1e-8):
    """Whiten with mean/variance taken over masked entries of the whole group (3-float all-reduce)."""
    stats = torch.stack([(values * mask).sum(), (values * values * mask).sum(), mask.sum().to(values.dtype)])
    if process_group is not None and dist.is_available() and dist.is_initialized() and dist.get_world_size(process_group) > 1:
        dist.all_reduce(stats, group=process_group)
    n = stats[2].clamp_min(1)
    mean = stats[0] / n
    var = (stats[1] / n - mean * mean).clamp_min(0) * n / (n - 1).clamp_min(1)
    out = (values - mean) * torch.rsqrt(var + eps)
    return out if shift_mean else out + mean


def apply_opd_kl_to_advantages(args, rollout_data, advantages, student_log_probs):
    """On-policy distillation: ``A -= opd_kl_coef * (logp_student - logp_teacher)`` per token."""
    teacher = rollout_data.get("teacher_log_probs")
    assert teacher, "OPD needs teacher_log_probs in the rollout data"
    rev = []
    for i, (adv, s, t) in enumerate(zip(advantages, student_log_probs, teacher)):
        t = torch.as_tensor(t, dtype=torch.float32, device=adv.device)
        if t.numel() < s.numel():  # a silent zero here would train without the distillation signal
            raise ValueError(f"sample {i}: teacher log-probs cover {t.numel()} tokens, the response has {s.numel()}")
        d = s.detach().float() - t[-s.numel():]
        advantages[i] = adv - args.opd_kl_coef * d
        rev.append(d)
    rollout_data["opd_reverse_kl"] = rev


def compute_advantages_and_returns(args: Namespace, rollout_data: RolloutBatch) -> None:
    """Fill ``rollout_data['advantages'|'returns'|'kl']`` according to ``args.advantage_estimator``."""
    rollout_lp = rollout_data.get("rollout_log_probs")
    log_probs = rollout_lp if args.use_rollout_logprobs else rollout_data.get("log_probs")
    ref = rollout_data.get("ref_log_probs")
    rewards = rollout_data.get("rewards")
    values = rollout_data.get("values")
    response_lengths = rollout_data.get("response_lengths")
    loss_masks = rollout_data.get("loss_masks")
    total_lengths = rollout_data.get("total_lengths")
    if not mpu.is_pipeline_last_stage():
        return

    # computed on the concatenated batch and handed out as per-sample views (a few kernels, not a few per sample)
    if args.kl_coef == 0 or not log_probs:
        xs = log_probs or rollout_lp or values
        lens = [x.numel() for x in xs]
        kl = list(torch.split(torch.zeros(sum(lens), dtype=torch.float32, device=xs[0].device), lens)) if xs else []
    else:
        lens = [x.numel() for x in log_probs]
        kl = list(torch.split(compute_approx_kl(torch.cat(log_probs), torch.cat(ref), kl_loss_type=args.kl_loss_type), lens))
    rollout_data["kl"] = kl
    dev = kl[0].device if kl else "cpu"

    est = args.advantage_estimator
    if getattr(args, "custom_advantage_function_path", None):
        load_function(args.custom_advantage_function_path)(args, rollout_data)
        advantages, returns = rollout_data["advantages"], rollout_data["returns"]
    elif est in ("grpo", "gspo", "cispo"):
        returns = get_grpo_returns(torch.tensor(rewards, dtype=torch.float32, device=dev), kl)
        advantages = list(returns)
    elif est == "ppo":
        tok_rewards = []
        for r, k in zip(rewards, kl):
            tr = -args.kl_coef * k
            if mpu.get_context_parallel_rank() == 0 and tr.numel():
                tr[-1] += r
            tok_rewards.append(tr)
        advantages, returns = get_advantages_and_returns_batch(
            total_lengths, response_lengths, values, tok_rewards, args.gamma, args.lambd
        )
    elif est == "reinforce_plus_plus":
        returns = get_reinforce_plus_plus_returns(
            rewards=torch.tensor(rewards, dtype=torch.float32, device=dev), kl=kl, loss_masks=loss_masks,
            response_lengths=response_lengths, total_lengths=total_lengths, kl_coef=args.kl_coef, gamma=args.gamma,
        )  # fmt: skip
        advantages = list(returns)
    elif est == "reinforce_plus_plus_baseline":
        advantages = get_reinforce_plus_plus_baseline_advantages(
            rewards=torch.tensor(rewards, dtype=torch.float32, device=dev), kl=kl, loss_masks=loss_masks,
            kl_coef=args.kl_coef,
        )  # fmt: skip
        returns = advantages
    else:
        raise NotImplementedError(f"advantage_estimator {est} is not supported.")

    if getattr(args, "use_opd", False):
        apply_opd_kl_to_advantages(args, rollout_data, advantages, log_probs)

    if args.normalize_advantages:
        masks, _ = local_loss_masks(total_lengths, response_lengths, loss_masks)
        flat, fmask = torch.cat(advantages), torch.cat(masks).to(torch.float32)
        assert flat.size() == fmask.size(), f"advantages {flat.size()} vs masks {fmask.size()}"
        # statistics over DP x CP: every rank (even one holding zero response tokens) must join
        white = distributed_masked_whiten(flat, fmask, mpu.get_data_parallel_group(with_context_parallel=True))
        advantages = list(torch.split(white, [a.numel() for a in advantages]))

    rollout_data["advantages"] = advantages
    rollout_data["returns"] = returns


# ---------------------------------------------------------- off-policy correction
def vanilla_tis_function(args, *, pg_loss, train_log_probs, rollout_log_probs, loss_masks, **kw):
    """Truncated importance sampling: weight = clamp(pi_train_old / pi_rollout, low, high)."""
    ro = torch.cat(rollout_log_probs, dim=0)
    old = torch.cat(train_log_probs, dim=0)
    ratio = torch.exp(old - ro)
    w = ratio.clamp(min=args.tis_clip_low, max=args.tis_clip)
    metrics = {"tis": ratio.detach().clone(), "tis_clipfrac": (w != ratio).float(), "tis_abs": (ratio - 1).abs().detach()}
    return pg_loss * w, loss_masks, metrics


def icepop_function(args, *, pg_loss, train_log_probs, rollout_log_probs, loss_masks, **kw):
    """IcePop: tokens whose ratio leaves [low, high] get weight zero instead of a clamped weight."""
    ro = torch.cat(rollout_log_probs, dim=0)
    old = torch.cat(train_log_probs, dim=0)
    ratio = torch.exp(old - ro)
    w = torch.where((ratio >= args.tis_clip_low) & (ratio <= args.tis_clip), ratio, torch.zeros_like(ratio))
    metrics = {"tis": ratio.detach().clone(), "tis_clipfrac": (w != ratio).float(), "tis_abs": (ratio - 1).abs().detach()}
    return pg_loss * w, loss_masks, metrics


# ------------------------------------------------------------------ policy loss
def policy_loss_function(args, batch, logits, sum_of_sample_mean):
    """PPO-clip / GSPO / CISPO surrogate (+ OPSM, TIS, entropy bonus, KL loss). Returns (loss, metrics)."""
    advantages = torch.cat(batch["advantages"], dim=0)
    old_lp = batch["rollout_log_probs"] if args.use_rollout_logprobs else batch.get("log_probs")
    rls, tls = batch["response_lengths"], batch["total_lengths"]

    _, res = get_log_probs_and_entropy(
        logits, args=args, unconcat_tokens=batch["unconcat_tokens"], total_lengths=tls, response_lengths=rls,
        with_entropy=True, with_entropy_grad=args.entropy_coef != 0, **get_rollout_top_p_logprob_kwargs(args, batch),
    )  # fmt: skip
    lps = res["log_probs"]
    _maybe_capture_log_probs(batch, lps)
    if not args.use_rollout_logprobs and not old_lp:
        old_lp = [x.detach() for x in lps]  # single step per rollout: ratio == 1 on the first pass
    train_lp_for_tis = batch.get("log_probs") or [x.detach() for x in lps]

    full_lp = full_old = None
    if args.use_opsm or args.advantage_estimator == "gspo":
        full_lp = [all_gather_with_cp(x, t, r) for x, t, r in zip(lps, tls, rls)]
        full_old = [all_gather_with_cp(x, t, r) for x, t, r in zip(old_lp, tls, rls)]
    if args.use_opsm:
        opsm_mask, opsm_clipfrac = compute_opsm_mask(args, full_lp, full_old, batch["advantages"], batch["loss_masks"])

    if args.advantage_estimator == "gspo":
        ppo_kl = compute_gspo_kl(full_lp, full_old, lps, batch["loss_masks"])
        old_cat, lp_cat = torch.cat(old_lp), torch.cat(lps)
    else:
        old_cat, lp_cat = torch.cat(old_lp), torch.cat(lps)
        ppo_kl = old_cat - lp_cat

    if args.advantage_estimator == "cispo":
        pg_loss, clipfrac = compute_cispo_loss(ppo_kl, lp_cat, advantages, args.eps_clip, args.eps_clip_high)
    else:
        pg_loss, clipfrac = compute_policy_loss(ppo_kl, advantages, args.eps_clip, args.eps_clip_high, args.eps_clip_c)
    if args.use_opsm:
        pg_loss = pg_loss * opsm_mask

    metric_reducer = sum_of_sample_mean
    tis_metrics, ois, masks_for_pg = {}, None, batch["loss_masks"]
    if args.get_mismatch_metrics or args.use_tis:
        assert "rollout_log_probs" in batch, "rollout_log_probs must be provided for TIS"
        ois = torch.exp(-ppo_kl)
        fn = load_function(args.custom_tis_function_path) if args.custom_tis_function_path else vanilla_tis_function
        pg_loss, masks_for_pg, tis_metrics = fn(
            args=args, pg_loss=pg_loss, train_log_probs=train_lp_for_tis, rollout_log_probs=batch["rollout_log_probs"],
            loss_masks=batch["loss_masks"], total_lengths=tls, response_lengths=rls,
        )  # fmt: skip
        # rejected tokens leave the numerator; denominators stay the pre-rejection rollout totals
        sum_of_sample_mean = get_sum_of_sample_mean(tls, rls, masks_for_pg, batch.get("rollout_mask_sums"),
                                                    args.calculate_per_token_loss)  # fmt: skip

    if getattr(args, "custom_pg_loss_reducer_function_path", None):
        reducer = load_function(args.custom_pg_loss_reducer_function_path)(tls, rls, masks_for_pg, args.calculate_per_token_loss)
    else:
        reducer = sum_of_sample_mean
    pg = reducer(pg_loss)
    clipfrac = sum_of_sample_mean(clipfrac)
    kl_metric = sum_of_sample_mean(ppo_kl)
    entropy = sum_of_sample_mean(torch.cat(res["entropy"], dim=0))
    loss = pg - args.entropy_coef * entropy

    kl_loss = None
    if args.use_kl_loss:
        ref = torch.cat(batch["ref_log_probs"], dim=0)
        ir = torch.exp(lp_cat - old_cat) if args.use_unbiased_kl else None
        kl_loss = sum_of_sample_mean(compute_approx_kl(lp_cat, ref, kl_loss_type=args.kl_loss_type, importance_ratio=ir))
        loss = loss + args.kl_loss_coef * kl_loss
    if lp_cat.numel() == 0:
        loss = loss + 0 * logits.sum()

    out = {"loss": loss.detach().clone(), "pg_loss": pg.detach().clone(), "entropy_loss": entropy.detach().clone(),
           "pg_clipfrac": clipfrac.detach().clone(), "ppo_kl": kl_metric.detach().clone()}  # fmt: skip
    if batch.get("rollout_log_probs"):
        ro = torch.cat(batch["rollout_log_probs"], dim=0)
        cmp = lp_cat if args.use_rollout_logprobs else old_cat
        out["train_rollout_logprob_abs_diff"] = sum_of_sample_mean((cmp - ro).abs()).detach().clone()
    if kl_loss is not None:
        out["kl_loss"] = kl_loss.detach().clone()
    if ois is not None:
        out["ois"] = metric_reducer(ois).detach().clone()
        for k, v in tis_metrics.items():
            out[k] = metric_reducer(v)
    if args.use_opsm:
        out["opsm_clipfrac"] = opsm_clipfrac
    if batch.get("opd_reverse_kl"):
        out["opd_reverse_kl"] = sum_of_sample_mean(torch.cat(batch["opd_reverse_kl"], dim=0)).detach().clone()
    return loss, out


def value_loss_function(args, batch, logits, sum_of_sample_mean):
    """Clipped value loss: max((v-R)^2, (clip(v, v_old +- eps) - R)^2)."""
    old_values = torch.cat(batch["values"], dim=0)
    _, res = get_values(logits, args=args, unconcat_tokens=batch["unconcat_tokens"], total_lengths=batch["total_lengths"],
                        response_lengths=batch["response_lengths"])  # fmt: skip
    values = torch.cat(res["values"], dim=0)
    returns = torch.cat(batch["returns"], dim=0)
    clipped = old_values + (values - old_values).clamp(-args.value_clip, args.value_clip)
    l1, l2 = (values - returns) ** 2, (clipped - returns) ** 2
    loss = sum_of_sample_mean(torch.maximum(l1, l2))
    clipfrac = sum_of_sample_mean((l2 > l1).float())
    if values.numel() == 0:
        loss = loss + 0 * logits.sum()
    return loss, {"value_loss": loss.detach().clone(), "value_clipfrac": clipfrac.detach().clone()}


def sft_loss_function(args, batch, logits, sum_of_sample_mean):
    """Negative log-likelihood over the masked response tokens."""
    _, res = get_log_probs_and_entropy(logits, args=args, unconcat_tokens=batch["unconcat_tokens"],
                                       total_lengths=batch["total_lengths"], response_lengths=batch["response_lengths"],
                                       with_entropy=False)  # fmt: skip
    lp = torch.cat(res["log_probs"], dim=0)
    loss = -sum_of_sample_mean(lp)
    if lp.numel() == 0:
        loss = loss + 0 * logits.sum()
    return loss, {"loss": loss.detach().clone()}


def loss_function(args, batch, num_microbatches, step_global_batch_size, logits, step_total_tokens=None):
    """Dispatch on ``args.loss_type`` and apply this backend's step normalisation.

    Returns ``(scaled_loss, normalizer, {"keys": [...], "values": tensor})`` where ``values[0]`` is the
    micro-batch token count in per-token mode (0 otherwise) followed by the metric sums.
    """
    num_tokens = sum(torch.clamp_min(m.sum(), 1) for m in batch["loss_masks"])
    reducer = get_sum_of_sample_mean(batch["total_lengths"], batch["response_lengths"], batch["loss_masks"],
                                     batch.get("rollout_mask_sums"), args.calculate_per_token_loss)  # fmt: skip
    kind = args.loss_type
    fn: Callable[..., Any]
    if kind == "policy_loss":
        fn = policy_loss_function
    elif kind == "value_loss":
        fn = value_loss_function
    elif kind == "sft_loss":
        fn = sft_loss_function
    elif kind == "custom_loss":
        fn = load_function(args.custom_loss_function_path)
    else:
        raise ValueError(f"Unknown loss type: {kind}")
    if getattr(args, "recompute_loss_function", False):
        from torch.utils.checkpoint import checkpoint

        loss, log = checkpoint(fn, args, batch, logits, reducer, use_reentrant=False)
    else:
        loss, log = fn(args, batch, logits, reducer)
    if getattr(args, "allgather_cp", False) and mpu.get_context_parallel_world_size() > 1:
        loss = loss + 0 * logits.sum()  # keep every CP rank's graph alive for the gather's backward

    if args.calculate_per_token_loss:
        denom = step_total_tokens if step_total_tokens is not None else num_tokens
        scaled = loss / denom
    else:
        scaled = loss / step_global_batch_size
    dev = logits.device
    vals = torch.stack(
        [torch.as_tensor(num_tokens if args.calculate_per_token_loss else 0, dtype=torch.float32, device=dev)]
        + [torch.as_tensor(v, dtype=torch.float32, device=dev).reshape(()) for v in log.values()]
    )
    return scaled, (num_tokens if args.calculate_per_token_loss else torch.tensor(1, device=dev)), {
        "keys": list(log.keys()), "values": vals,
    }  # fmt: skip
