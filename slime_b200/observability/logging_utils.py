"""Logger set-up and tracker fan-out (wandb / tensorboard / in-memory).

Parity: slime/observability/logging_utils.py:12-51. ``log(args, metrics, step_key)``
sends one metrics dict to every enabled tracker; the in-memory sink keeps the last
records so tests and the bench can read what was logged without a tracker installed.
"""

from __future__ import annotations

import logging

_CONFIGURED = False
_MEMORY_SINK: list[dict] = []


def configure_logger(prefix: str = ""):
    global _CONFIGURED
    if _CONFIGURED:
        return
    logging.basicConfig(level=logging.INFO, format=f"[%(asctime)s{prefix}] %(filename)s:%(lineno)d - %(message)s",
                        datefmt="%Y-%m-%d %H:%M:%S", force=True)  # fmt: skip
    _CONFIGURED = True


def init_tracking(args, primary: bool = True, **kwargs):
    if getattr(args, "use_wandb", False):
        from slime_b200.observability import wandb_utils

        if primary:
            wandb_utils.init_wandb_primary(args, **kwargs)
        else:
            wandb_utils.init_wandb_secondary(args, **kwargs)
    if getattr(args, "use_tensorboard", False):
        from slime_b200.observability.tensorboard_utils import _TensorboardAdapter

        _TensorboardAdapter(args)


def finish_tracking(args):
    if getattr(args, "use_wandb", False):
        try:
            import wandb

            wandb.finish()
        except ImportError:
            pass


def log(args, metrics: dict, step_key: str):
    record = {k: (float(v) if hasattr(v, "item") else v) for k, v in metrics.items()}
    _MEMORY_SINK.append(record)
    del _MEMORY_SINK[:-256]
    if getattr(args, "use_wandb", False):
        try:
            import wandb

            wandb.log(record)
        except ImportError:
            pass
    if getattr(args, "use_tensorboard", False):
        from slime_b200.observability.tensorboard_utils import _TensorboardAdapter

        step = record.get(step_key)
        _TensorboardAdapter(args).log({k: v for k, v in record.items() if k != step_key}, step)


def recent_records() -> list[dict]:
    return list(_MEMORY_SINK)
