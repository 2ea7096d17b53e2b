"""Built-in group filters (parity: slime/rollout/filter_hub/dynamic_sampling_filters.py:9,18)."""

import torch

from slime_b200.rollout.filter_hub.base_types import DynamicFilterOutput
from slime_b200.utils.types import Sample

__all__ = ["check_reward_nonzero_std", "check_reward_nonzero_std_with_fallback"]


def _std(args, samples):
    return torch.tensor([s.get_reward_value(args) for s in samples], dtype=torch.float).std()


def check_reward_nonzero_std(args, samples: list[Sample], **kwargs):
    """DAPO-style: a group whose rewards are all equal carries no GRPO signal."""
    keep = _std(args, samples) > 0.0
    rewards = [s.get_reward_value(args) for s in samples]
    return DynamicFilterOutput(keep=bool(keep), reason=None if keep else f"zero_std_{round(rewards[0], 1)}")


def check_reward_nonzero_std_with_fallback(args, samples: list[Sample], **kwargs):
    out = check_reward_nonzero_std(args, samples, **kwargs)
    out.keep_when_insufficient = True
    return out
