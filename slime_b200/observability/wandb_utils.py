"""Weights & Biases glue. The driver opens the run (``init_wandb_primary``) and publishes its id on
``args.wandb_run_id``; every other process (rollout manager, trainer rank 0) attaches to that run in shared mode
(``init_wandb_secondary``), so all metrics land in one run. Offline mode (``--wandb-mode offline`` or ``WANDB_MODE``)
writes under ``--wandb-dir``. ``wandb`` is imported lazily: a missing package only matters with ``--use-wandb``.
Parity: slime/observability/wandb_utils.py:11-176.
"""

from __future__ import annotations

import logging
import os
from copy import deepcopy

logger = logging.getLogger(__name__)

_STEP_AXES = (("train/step", ("train/*",)), ("rollout/step", ("rollout/*", "multi_turn/*", "passrate/*", "perf/*")),
              ("eval/step", ("eval/*",)))  # fmt: skip


def _wandb():
    try:
        import wandb

        return wandb
    except ImportError as e:  # pragma: no cover - depends on the environment
        raise RuntimeError("--use-wandb needs the `wandb` package, which is not installed") from e


def _is_offline_mode(args) -> bool:
    return (args.wandb_mode or os.environ.get("WANDB_MODE")) == "offline"


def _apply_mode(args) -> bool:
    if args.wandb_mode:
        os.environ["WANDB_MODE"] = args.wandb_mode
        logger.info("W&B mode: %s", args.wandb_mode)
    return _is_offline_mode(args)


def _config_of(args, prefix: str | None = None) -> dict:
    cfg = deepcopy(vars(args))
    return {f"{prefix}/{k}": v for k, v in cfg.items()} if prefix else cfg


def _compute_config_for_logging(args) -> dict:
    cfg = _config_of(args)
    cfg["env_vars"] = {k: os.environ[k] for k in ("SLURM_JOB_ID",) if k in os.environ}
    if getattr(args, "use_critic", False):
        from slime_b200.utils.arguments import get_role_args

        cfg.update(_config_of(get_role_args(args, "critic"), "critic"))
    return cfg


def _define_axes(wandb) -> None:
    for step, families in _STEP_AXES:
        wandb.define_metric(step)
        for fam in families:
            wandb.define_metric(fam, step_metric=step)


def init_wandb_primary(args, **_):
    if not args.use_wandb:
        args.wandb_run_id = None
        return
    wandb = _wandb()
    offline = _apply_mode(args)
    if not offline and args.wandb_key is not None:
        wandb.login(key=args.wandb_key, host=args.wandb_host)
    group = args.wandb_group
    name = group
    if args.wandb_random_suffix:
        group = f"{group}_{wandb.util.generate_id()}"
        name = f"{group}-RANK_{getattr(args, 'rank', 0)}"
    kw = dict(entity=args.wandb_team, project=args.wandb_project, group=group, name=name,
              config=_compute_config_for_logging(args),
              settings=wandb.Settings(mode="offline") if offline else wandb.Settings(mode="shared", x_primary=True))  # fmt: skip
    if args.wandb_dir:
        os.makedirs(args.wandb_dir, exist_ok=True)
        kw["dir"] = args.wandb_dir
    wandb.init(**kw)
    _define_axes(wandb)
    args.wandb_run_id = wandb.run.id


def init_wandb_secondary(args, role: str | None = None, **_):
    run_id = getattr(args, "wandb_run_id", None)
    if run_id is None:
        return
    wandb = _wandb()
    offline = _apply_mode(args)
    if not offline and args.wandb_key is not None:
        wandb.login(key=args.wandb_key, host=args.wandb_host)
    settings = (wandb.Settings(mode="offline") if offline
                else wandb.Settings(mode="shared", x_primary=False, x_update_finish_state=False))  # fmt: skip
    kw = dict(id=run_id, entity=args.wandb_team, project=args.wandb_project, resume="allow", reinit=True,
              config=_config_of(args, "critic" if role == "critic" else None), settings=settings)  # fmt: skip
    if args.wandb_dir:
        os.makedirs(args.wandb_dir, exist_ok=True)
        kw["dir"] = args.wandb_dir
    wandb.init(**kw)
    _define_axes(wandb)
