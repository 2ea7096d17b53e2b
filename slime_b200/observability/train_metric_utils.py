"""Training-side metrics: per-step reduction, rollout-data statistics, perf (tok/s, TFLOPs).

Parity: slime/observability/train_metric_utils.py (reduce :18, gather :86-117,
log_rollout_data :142, log_perf_data :358-405). Metric names are kept:
``train/{loss,pg_loss,entropy_loss,pg_clipfrac,ppo_kl,grad_norm,lr-pg_0,...}``,
``rollout/{log_probs,advantages,returns,...}``, ``perf/{actor_train_time,
actor_train_tok_per_s,actor_train_tflops,log_probs_time,update_weights_time,step_time,...}``.
"""

from __future__ import annotations

import logging

import torch
import torch.distributed as dist

from slime_b200.observability import logging_utils
from slime_b200.observability.timer import Timer
from slime_b200.parallel import state as mpu
from slime_b200.utils.flops_utils import calculate_fwd_flops

logger = logging.getLogger(__name__)


def gather_and_reduce_log_dict(log_dict: dict, group=None) -> dict | None:
    """Mean of every metric over the DP ranks (object gather on the Gloo group); main rank gets the result."""
    size = mpu.get_data_parallel_world_size(with_context_parallel=True)
    if size == 1 or not (dist.is_available() and dist.is_initialized()):
        return log_dict
    gathered = [None] * size if mpu.get_data_parallel_rank(with_context_parallel=True) == 0 else None
    dist.gather_object(log_dict, gathered, dst=mpu.get_data_parallel_ranks(True)[0],
                       group=mpu.get_data_parallel_group_gloo(with_context_parallel=True))  # fmt: skip
    if gathered is None:
        return None
    keys = gathered[0].keys()
    return {k: sum(g[k] for g in gathered) / len(gathered) for k in keys}


def _masked_mean_list(vals, masks, total_lengths=None, response_lengths=None):
    from slime_b200.backends.train.cp_utils import local_loss_masks

    if total_lengths is not None and mpu.get_context_parallel_world_size() > 1:
        masks, _ = local_loss_masks(total_lengths, response_lengths, masks)
    v = torch.cat([x.reshape(-1).float() for x in vals])
    m = torch.cat([x.reshape(-1) for x in masks]).to(v.device, torch.float32)
    return (v * m).sum() / torch.clamp_min(m.sum(), 1.0)  # stays on the device: the caller reads all metrics at once


def log_rollout_data(rollout_id, args, rollout_data: dict):
    """``rollout/*`` statistics of the batch about to be trained on (last PP stage, tp rank 0)."""
    if not (mpu.get_tensor_model_parallel_rank() == 0 and mpu.is_pipeline_last_stage()):
        return
    log = {}
    masks = rollout_data.get("loss_masks")
    tl, rl = rollout_data.get("total_lengths"), rollout_data.get("response_lengths")
    for key in ("log_probs", "ref_log_probs", "rollout_log_probs", "advantages", "returns", "values", "entropy", "kl"):
        vals = rollout_data.get(key)
        if vals and torch.is_tensor(vals[0]) and masks:
            try:
                log[key] = _masked_mean_list(vals, masks, tl, rl)
            except RuntimeError:
                continue
    if log:  # one device->host read for every tensor metric
        keys = list(log)
        for k, v in zip(keys, torch.stack([log[k].reshape(()) for k in keys]).tolist()):
            log[k] = v
    for key in ("rewards", "local_raw_reward", "response_lengths", "truncated"):
        vals = rollout_data.get(key)
        if vals:
            log[key if key != "local_raw_reward" else "raw_reward"] = float(sum(map(float, vals)) / len(vals))
    if getattr(args, "ci_test", False) and "log_probs" in log:
        assert -50.0 < log["log_probs"] < 0.0, f"log_probs out of range: {log['log_probs']}"
        if rollout_id == 0 and "ref_log_probs" in log and not getattr(args, "ci_disable_kl_checker", False):
            assert abs(log["log_probs"] - log["ref_log_probs"]) < 1e-6, "ref and actor log-probs differ at rollout 0"
    reduced = gather_and_reduce_log_dict(log)
    if reduced is not None and mpu.get_data_parallel_rank(with_context_parallel=True) == 0:
        out = {f"rollout/{k}": v for k, v in reduced.items()}
        out["rollout/step"] = rollout_id
        logging_utils.log(args, out, "rollout/step")
        logger.info("rollout %s: %s", rollout_id, {k: round(v, 5) for k, v in out.items()})


def log_train_steps(rollout_id, args, history, model, prefix="train/") -> list[dict]:
    """Log every optimizer step's reduced metrics; returns them as python floats."""
    out = []
    steps_per_rollout = len(history)
    for step_id, (metrics, grad_norm) in enumerate(history):
        if not metrics and grad_norm is None:
            continue
        rec = {f"{prefix}{k}": float(v) for k, v in metrics.items()}
        if grad_norm is not None:
            rec[f"{prefix}grad_norm"] = float(grad_norm)
        if model.scheduler is not None:
            rec[f"{prefix}lr-pg_0"] = model.scheduler.get_lr()
        rec[f"{prefix}step"] = rollout_id * steps_per_rollout + step_id
        if getattr(args, "ci_test", False) and step_id == 0 and not getattr(args, "ci_disable_kl_checker", False):
            if f"{prefix}ppo_kl" in rec and not args.use_rollout_logprobs:
                assert abs(rec[f"{prefix}ppo_kl"]) < 1e-8, f"first-step ppo_kl should be 0, got {rec[f'{prefix}ppo_kl']}"
        if f"{prefix}train_rollout_logprob_abs_diff" in rec and getattr(args, "ci_test", False):
            thr = args.ci_train_rollout_logprob_abs_diff_threshold
            assert rec[f"{prefix}train_rollout_logprob_abs_diff"] <= thr, rec
        if mpu.is_main_rank():
            logging_utils.log(args, rec, f"{prefix}step")
            logger.info("step %s: %s", rec[f"{prefix}step"], {k: round(v, 6) for k, v in rec.items()})
        out.append(rec)
    return out


def log_perf_data(rollout_id, args, extra_metrics=None):
    t = Timer()
    times = t.log_dict()
    log = {f"perf/{k}_time": v for k, v in times.items()}
    seq_lens = t.seq_lens
    if seq_lens and "actor_train" in times and times["actor_train"] > 0:
        world = max(dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1, 1)
        try:
            flops = 3 * calculate_fwd_flops(seq_lens, args)
            log["perf/actor_train_tflops"] = flops / world / times["actor_train"] / 1e12
        except (AttributeError, TypeError):
            pass
        log["perf/actor_train_tok_per_s"] = sum(seq_lens) / times["actor_train"]
    if "train_wait" in times and "train" in times:
        log["perf/step_time"] = times["train_wait"] + times["train"]
        log["perf/wait_time_ratio"] = times["train_wait"] / max(log["perf/step_time"], 1e-9)
    if extra_metrics:
        log.update(extra_metrics)
    if mpu.is_main_rank():
        log["rollout/step"] = rollout_id
        logging_utils.log(args, log, "rollout/step")
    t.reset()
    return log
