"""User hooks applied to every finished ``Sample`` (``--rollout-sample-hook-path``).

A hook is ``(args, sample, *, rollout_id, evaluation) -> Sample | None`` and
may be sync or async; returning a Sample replaces the input.
Parity: slime/rollout/sample_hooks.py:24-50.
"""

from __future__ import annotations

import inspect

from slime_b200.utils.misc import load_function
from slime_b200.utils.types import Sample


def load_sample_hooks(args):
    return [load_function(p) for p in (getattr(args, "rollout_sample_hook_path", None) or [])]


async def _run_hooks_on_one(args, sample: Sample, hooks, rollout_id, evaluation) -> Sample:
    for hook in hooks:
        out = hook(args, sample, rollout_id=rollout_id, evaluation=evaluation)
        if inspect.isawaitable(out):
            out = await out
        if out is not None:
            if not isinstance(out, Sample):
                raise TypeError(f"sample hook {hook} must return Sample or None, got {type(out)}")
            sample = out
    return sample


async def apply_rollout_sample_hooks(args, samples, *, rollout_id=None, evaluation=False, hooks=None):
    """Apply hooks to a Sample or to every Sample leaf of a (nested) list; structure is preserved."""
    hooks = load_sample_hooks(args) if hooks is None else hooks
    if not hooks:
        return samples
    if isinstance(samples, Sample):
        return await _run_hooks_on_one(args, samples, hooks, rollout_id, evaluation)
    return [
        await apply_rollout_sample_hooks(args, s, rollout_id=rollout_id, evaluation=evaluation, hooks=hooks)
        for s in samples
    ]
