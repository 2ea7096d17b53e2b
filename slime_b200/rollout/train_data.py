"""Samples -> training payload: reward post-processing, the train-data dict and the DP split.

These are the pure-function halves of the rollout manager (parity:
slime/ray/rollout.py:608-633 reward post-processing, :635-752 train-data conversion,
:757-824 DP split; wire dtypes slime/observability/rollout_data_utils.py:12-20).
"""

from __future__ import annotations

import torch

from slime_b200.utils.data import get_source
from slime_b200.utils.dp_schedule import build_dp_schedule
from slime_b200.utils.misc import load_function
from slime_b200.utils.types import Sample

GROUP_NORM_ESTIMATORS = ("grpo", "gspo", "cispo", "reinforce_plus_plus_baseline")
STD_NORM_ESTIMATORS = ("grpo", "gspo", "cispo")

# per-sample list fields and their tensor dtype on the wire
_TENSOR_FIELDS = {
    "tokens": torch.long,
    "loss_masks": torch.int,
    "rollout_log_probs": torch.float32,
    "teacher_log_probs": torch.float32,
    "rollout_top_p_token_ids": torch.int32,
    "rollout_top_p_token_offsets": torch.int32,
    "rollout_routed_experts": torch.int32,
}

_PER_SAMPLE_KEYS = [
    "tokens", "multimodal_train_inputs", "response_lengths", "rewards", "truncated", "loss_masks", "round_number",
    "sample_indices", "rollout_ids", "rollout_mask_sums", "rollout_log_probs", "rollout_top_p_token_ids",
    "rollout_top_p_token_offsets", "rollout_routed_experts", "source_names", "prompt", "teacher_log_probs", "metadata",
]  # fmt: skip


def post_process_rewards(args, samples: list[Sample]):
    """Returns ``(raw_rewards, rewards)``. GRPO-family estimators subtract the group mean and (grpo/gspo/
    cispo) divide by the unbiased group std + 1e-6; groups are consecutive blocks of n_samples_per_prompt."""
    custom = getattr(args, "custom_reward_post_process_path", None)
    if custom:
        return load_function(custom)(args, samples)
    raw = [s.get_reward_value(args) for s in samples]
    if args.advantage_estimator in GROUP_NORM_ESTIMATORS and args.rewards_normalization:
        r = torch.tensor(raw, dtype=torch.float)
        n = args.n_samples_per_prompt
        # groups are consecutive blocks of n samples; a rank that generated only its own slice of the rollout batch
        # still has whole groups (a ragged tail, e.g. after dynamic filtering, is normalised as one group)
        r = r.reshape(-1, n) if r.numel() % n == 0 else r.view(1, -1)
        r = r - r.mean(dim=-1, keepdim=True)
        if args.advantage_estimator in STD_NORM_ESTIMATORS and args.grpo_std_normalization:
            r = r / (r.std(dim=-1, keepdim=True) + 1e-6)
        return raw, r.flatten().tolist()
    return raw, raw


def _fill_rollout_ids(samples) -> list[int]:
    ids = [s.rollout_id for s in samples]
    used = {i for i in ids if i is not None}
    nxt = 0
    for k, v in enumerate(ids):
        if v is None:
            while nxt in used:
                nxt += 1
            ids[k] = nxt
            used.add(nxt)
    return ids


def convert_samples_to_train_data(args, samples: list[Sample]) -> dict:
    custom = getattr(args, "custom_convert_samples_to_train_data_path", None)
    if custom:
        return load_function(custom)(args, samples)
    raw, rewards = post_process_rewards(args, samples)
    assert len(raw) == len(samples) == len(rewards)
    rollout_ids = _fill_rollout_ids(samples)
    data = {
        "tokens": [s.tokens for s in samples],
        "response_lengths": [s.response_length for s in samples],
        "rewards": rewards,
        "raw_reward": raw,
        "truncated": [int(s.status == Sample.Status.TRUNCATED) for s in samples],
        "sample_indices": [s.index for s in samples],
        "rollout_ids": rollout_ids,
    }
    masks = []
    for s in samples:
        if s.loss_mask is None:
            s.loss_mask = [1] * s.response_length
        assert len(s.loss_mask) == s.response_length, f"loss mask length {len(s.loss_mask)} != response length {s.response_length}"
        if s.remove_sample:
            s.loss_mask = [0] * s.response_length
        masks.append(s.loss_mask)
    data["loss_masks"] = masks
    # whole-rollout mask totals, so a rollout split over micro-batches still averages once
    per_rollout: dict[int, int] = {}
    for rid, m in zip(rollout_ids, masks):
        per_rollout[rid] = per_rollout.get(rid, 0) + sum(m)
    data["rollout_mask_sums"] = [per_rollout[rid] for rid in rollout_ids]

    if any(s.metadata and "raw_reward" in s.metadata for s in samples):
        data["raw_reward"] = [s.metadata["raw_reward"] if s.metadata and "raw_reward" in s.metadata else s.reward for s in samples]
    first = samples[0]
    if first.metadata and "round_number" in first.metadata:
        data["round_number"] = [s.metadata["round_number"] for s in samples]
    if first.rollout_log_probs is not None:
        data["rollout_log_probs"] = [s.rollout_log_probs for s in samples]
    if getattr(args, "rollout_top_p", 1.0) != 1.0:
        for s in samples:
            assert s.rollout_top_p_token_ids is not None and s.rollout_top_p_token_offsets is not None
            assert len(s.rollout_top_p_token_offsets) == s.response_length + 1
            assert int(s.rollout_top_p_token_offsets[-1]) == len(s.rollout_top_p_token_ids)
        data["rollout_top_p_token_ids"] = [s.rollout_top_p_token_ids for s in samples]
        data["rollout_top_p_token_offsets"] = [s.rollout_top_p_token_offsets for s in samples]
    if first.rollout_routed_experts is not None:
        data["rollout_routed_experts"] = [torch.as_tensor(s.rollout_routed_experts) for s in samples]
        if getattr(args, "use_rollout_routing_replay", False):
            from slime_b200.observability.rollout_data_utils import validate_rollout_routed_experts_for_replay

            validate_rollout_routed_experts_for_replay(data["rollout_routed_experts"], args)
    if first.train_metadata is not None:
        data["metadata"] = [s.train_metadata for s in samples]
    if any(s.multimodal_train_inputs is not None for s in samples):
        data["multimodal_train_inputs"] = [s.multimodal_train_inputs for s in samples]
    if first.teacher_log_probs is not None:
        data["teacher_log_probs"] = [s.teacher_log_probs for s in samples]
    if first.metadata is not None:
        data["source_names"] = [get_source(s) for s in samples]
    return data


def tensorize_rollout_data_for_training(rollout_data: dict, pin: bool = False) -> dict:
    """Lists of python numbers -> CPU tensors with the wire dtypes (pinned when they will be copied H2D)."""
    for key, dtype in _TENSOR_FIELDS.items():
        vals = rollout_data.get(key)
        if vals is None:
            continue
        out = []
        for v in vals:
            t = v.to(dtype) if torch.is_tensor(v) else torch.tensor(v, dtype=dtype)
            out.append(t.pin_memory() if pin and not t.is_pinned() and t.numel() else t)
        rollout_data[key] = out
    if rollout_data.get("multimodal_train_inputs"):  # processor outputs travel as plain CPU tensors (no autograd history)
        rollout_data["multimodal_train_inputs"] = [
            d if d is None else {k: (v.detach().cpu() if torch.is_tensor(v) else v) for k, v in d.items()}
            for d in rollout_data["multimodal_train_inputs"]]  # fmt: skip
    if "rollout_mask_sums" in rollout_data and not torch.is_tensor(rollout_data["rollout_mask_sums"]):
        rollout_data["rollout_mask_sums"] = torch.as_tensor([float(x) for x in rollout_data["rollout_mask_sums"]], dtype=torch.float32)
    return rollout_data


def split_train_data_by_dp(args, data: dict, train_parallel_config: dict, pin: bool = False) -> list[dict]:
    """Schedule micro-batches and return one payload per DP rank (see ``build_dp_schedule``)."""
    dp = train_parallel_config["dp_size"]
    total_lengths = [len(t) for t in data["tokens"]]
    data["total_lengths"] = total_lengths
    partitions, mb_indices, num_mb, gbs = build_dp_schedule(
        args, train_parallel_config, total_lengths, global_batch_size=args.global_batch_size, rollout_indices=data["rollout_ids"]
    )
    out = []
    for r in range(dp):
        part = partitions[r]
        payload = {"partition": part}
        for key in _PER_SAMPLE_KEYS:
            if key in data:
                payload[key] = [data[key][j] for j in part]
        for key in ("raw_reward", "total_lengths"):  # whole-batch fields, localised by the trainer
            if key in data:
                payload[key] = data[key]
        payload["global_batch_sizes"] = gbs
        payload["num_microbatches"] = num_mb
        payload["micro_batch_indices"] = mb_indices[r]
        out.append(tensorize_rollout_data_for_training(payload, pin=pin))
    return out
