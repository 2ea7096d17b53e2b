"""Debug dump of the per-rank training batch (``--save-debug-train-data``), format version 2.

``{"format_version": 2, "rollout_id", "rank", "samples": [...], "dp_shards": [...], raw_reward}``;
per-sample tensors are moved to CPU and, under context parallelism, restored to full
response length before saving. Parity: slime/observability/train_data_utils.py:38-242.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from slime_b200.parallel import state as mpu

_PER_SAMPLE = ("tokens", "loss_masks", "log_probs", "ref_log_probs", "rollout_log_probs", "advantages", "returns", "values",
               "response_lengths", "total_lengths", "rewards", "sample_indices", "rollout_ids", "teacher_log_probs")  # fmt: skip
_CP_SLICED = ("log_probs", "ref_log_probs", "advantages", "returns", "values", "rollout_log_probs", "teacher_log_probs")


def _to_cpu(v):
    return v.detach().cpu() if torch.is_tensor(v) else v


def restore_context_parallel_fields_to_cpu(rollout_data: dict) -> dict:
    """Rebuild full-length per-sample tensors from their CP-local pieces, on CPU."""
    from slime_b200.backends.train.cp_utils import all_gather_with_cp

    out = {}
    cp = mpu.get_context_parallel_world_size()
    for key in _PER_SAMPLE:
        vals = rollout_data.get(key)
        if vals is None:
            continue
        if cp > 1 and key in _CP_SLICED and vals and torch.is_tensor(vals[0]):
            vals = [all_gather_with_cp(v, tl, rl) for v, tl, rl in zip(vals, rollout_data["total_lengths"], rollout_data["response_lengths"])]
        out[key] = [_to_cpu(v) for v in vals] if isinstance(vals, list) else _to_cpu(vals)
    return out


def _build_dump_payload(rollout_id: int, rollout_data: dict) -> dict:
    fields = restore_context_parallel_fields_to_cpu(rollout_data)
    n = len(fields.get("tokens", []))
    samples = [{k: v[i] for k, v in fields.items() if isinstance(v, list) and len(v) == n} for i in range(n)]
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    return {
        "format_version": 2,
        "rollout_id": rollout_id,
        "rank": rank,
        "samples": samples,
        "dp_shards": [{"partition": rollout_data.get("partition"), "micro_batch_indices": rollout_data.get("micro_batch_indices"),
                       "num_microbatches": rollout_data.get("num_microbatches")}],
        "raw_reward": rollout_data.get("raw_reward"),
    }  # fmt: skip


def save_debug_train_data(args, *, rollout_id: int, rollout_data: dict):
    template = getattr(args, "save_debug_train_data", None)
    if template is None:
        return
    if not (mpu.get_tensor_model_parallel_rank() == 0 and mpu.is_pipeline_last_stage()):
        return
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    path = template.format(rollout_id=rollout_id, rank=rank)
    if "{rank}" not in template and rank != 0:
        root, ext = os.path.splitext(path)
        path = f"{root}_rank{rank}{ext}"
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    torch.save(_build_dump_payload(rollout_id, rollout_data), path)
