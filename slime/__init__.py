"""Compatibility namespace: ``import slime.<module>`` resolves to the matching ``slime_b200`` module.

Configs, launch scripts and user plug-ins written for the reference name their hooks by dotted path
(``--rollout-function-path slime.rollout.sglang_rollout.generate_rollout``, ``--data-source-path
slime.rollout.data_source.RolloutDataSourceWithBuffer``, ``from slime.utils.types import Sample``). This package
keeps those paths working: a meta-path finder maps each ``slime.*`` name to its ``slime_b200`` home (same relative
name unless the table below says otherwise) and returns that very module object, so classes are identical under
both names (``slime.utils.types.Sample is slime_b200.utils.types.Sample``).
"""

from __future__ import annotations

import importlib
import importlib.abc
import importlib.machinery
import sys

# reference module (prefix) -> home in this framework; longest prefix wins
_MOVED = {
    "slime.ray.rollout": "slime_b200.runtime.rollout_manager",
    "slime.ray.actor_group": "slime_b200.runtime.train_group",
    "slime.ray.train_actor": "slime_b200.runtime.train_group",
    "slime.ray.placement_group": "slime_b200.runtime.placement",
    "slime.ray.utils": "slime_b200.runtime.actors",
    "slime.ray": "slime_b200.runtime",
    "slime.backends.megatron_utils.update_weight": "slime_b200.weight_sync",
    "slime.backends.megatron_utils.megatron_to_hf": "slime_b200.weight_sync.convert",
    "slime.backends.megatron_utils.arguments": "slime_b200.utils.arguments",
    "slime.backends.megatron_utils": "slime_b200.backends.train",
    "slime.backends.sglang_utils.sglang_engine": "slime_b200.engine.engine_actor",
    "slime.backends.sglang_utils.arguments": "slime_b200.engine.server_args",
    "slime.backends.sglang_utils": "slime_b200.engine",
    "slime.utils.tensor_backper": "slime_b200.utils.tensor_backuper",
    "slime.utils.memory_utils": "slime_b200.runtime.memory",
}


def resolve(name: str) -> str | None:
    """``slime.a.b`` -> the ``slime_b200`` module that serves it, or None for names outside the namespace."""
    if name == "slime":
        return "slime_b200"
    if not name.startswith("slime."):
        return None
    best = ""
    for prefix in _MOVED:
        if (name == prefix or name.startswith(prefix + ".")) and len(prefix) > len(best):
            best = prefix
    if best:
        return _MOVED[best] + name[len(best) :]
    return "slime_b200" + name[len("slime") :]


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        real = resolve(fullname)
        if real is None or fullname == "slime":
            return None
        try:
            found = importlib.util.find_spec(real)
        except (ImportError, ValueError):
            found = None
        if found is None:
            return None
        return importlib.machinery.ModuleSpec(fullname, self, is_package=found.submodule_search_locations is not None)

    def create_module(self, spec):
        return importlib.import_module(resolve(spec.name))  # the real module object: one class identity under both names

    def exec_module(self, module):
        return None


import importlib.util  # noqa: E402

if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())
