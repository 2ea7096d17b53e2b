"""Instruction-following (IFBench) reward. The evaluation library is loaded lazily from
``IFBENCH_PATH`` (or an importable ``instructions_registry``); the reward is the fraction of
instructions followed (strict), or 0/1 when ``metadata['all_or_nothing']``.
Parity: slime/rollout/rm_hub/ifbench.py:19-170 (which clones the library on first use; no network
here, so a missing library raises with instructions instead)."""

from __future__ import annotations

import importlib
import os
import sys

_registry = None


def _load_registry():
    global _registry
    if _registry is not None:
        return _registry
    path = os.environ.get("IFBENCH_PATH")
    if path and path not in sys.path:
        sys.path.insert(0, path)
    for mod in ("instructions_registry", "ifbench.instructions_registry", "instruction_following_eval.instructions_registry"):
        try:
            _registry = importlib.import_module(mod)
            return _registry
        except ImportError:
            continue
    raise ImportError("IFBench evaluation library not found: set IFBENCH_PATH to a checkout containing instructions_registry.py")


def _strip_cot(text: str) -> str:
    return text.split("</think>")[-1].strip() if "</think>" in text else text.strip()


def compute_ifbench_reward(response: str, label, metadata: dict | None = None) -> float:
    md = metadata or {}
    ids = md.get("instruction_id_list") or []
    kwargs_list = md.get("kwargs") or [{} for _ in ids]
    if not ids or not response or not response.strip():
        return 0.0
    reg = _load_registry()
    table = getattr(reg, "INSTRUCTION_DICT")
    text = _strip_cot(response)
    followed = []
    for iid, kw in zip(ids, kwargs_list):
        inst = table[iid](iid)
        kw = {k: v for k, v in (kw or {}).items() if v is not None}
        inst.build_description(**kw)
        args = inst.get_instruction_args() or {}
        if "prompt" in args:
            inst.build_description(prompt=md.get("prompt_text", ""))
        followed.append(bool(text.strip() and inst.check_following(text)))
    if md.get("all_or_nothing"):
        return float(all(followed))
    return sum(followed) / len(followed)
