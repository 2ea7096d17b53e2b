"""User hooks applied to every finished ``Sample`` (``--rollout-sample-hook-path``).

A hook is ``(args, sample, **context) -> Sample | None``, sync or async; returning a Sample replaces the input. The
context offers ``rollout_id`` (the rollout being produced, set by the rollout manager through ``set_current_rollout_id``),
``evaluation`` and whatever else the caller passes; a hook receives the entries its signature names (all of them if it
takes ``**kwargs``). Parity: slime/rollout/sample_hooks.py:9-50.
"""

from __future__ import annotations

import inspect

from slime_b200.utils.misc import load_function
from slime_b200.utils.types import Sample

_current_rollout_id: int | None = None


def set_current_rollout_id(rollout_id: int | None) -> None:
    global _current_rollout_id
    _current_rollout_id = rollout_id


def load_sample_hooks(args):
    return [load_function(p) for p in (getattr(args, "rollout_sample_hook_path", None) or [])]


def _accepted(hook, context: dict) -> dict:
    params = inspect.signature(hook).parameters
    if any(p.kind is inspect.Parameter.VAR_KEYWORD for p in params.values()):
        return context
    return {k: v for k, v in context.items() if k in params}


async def _run_hooks_on_one(args, sample: Sample, hooks, context: dict) -> Sample:
    for hook in hooks:
        out = hook(args, sample, **_accepted(hook, context))
        if inspect.isawaitable(out):
            out = await out
        if out is not None:
            if not isinstance(out, Sample):
                raise TypeError(f"sample hook {hook} returned {type(out).__name__}: expected Sample or None")
            sample = out
    return sample


async def apply_rollout_sample_hooks(args, samples, *, hooks=None, **context):
    """Apply hooks to a Sample or to every Sample leaf of a (nested) list; the structure is preserved (new lists)."""
    hooks = load_sample_hooks(args) if hooks is None else hooks
    if not hooks:
        return samples
    if context.get("rollout_id") is None:
        context["rollout_id"] = _current_rollout_id
    context.setdefault("evaluation", False)
    if isinstance(samples, Sample):
        return await _run_hooks_on_one(args, samples, hooks, context)
    return [await apply_rollout_sample_hooks(args, s, hooks=hooks, **context) for s in samples]
