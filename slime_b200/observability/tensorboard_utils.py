"""TensorBoard sink: one ``SummaryWriter`` per process under ``$TENSORBOARD_DIR`` or
``tensorboard_log/<tb_project_name>/<tb_experiment_name>`` (experiment defaults to a timestamp).
Parity: slime/observability/tensorboard_utils.py:17-61."""

from __future__ import annotations

import datetime
import logging
import os

from slime_b200.utils.misc import SingletonMeta

logger = logging.getLogger(__name__)
__all__ = ["_TensorboardAdapter"]


class _TensorboardAdapter(metaclass=SingletonMeta):
    def __init__(self, args):
        assert args.use_tensorboard
        project, experiment = args.tb_project_name, args.tb_experiment_name
        env_dir = os.environ.get("TENSORBOARD_DIR")
        if project is None and not env_dir:
            raise ValueError("TensorBoard needs --tb-project-name (and optionally --tb-experiment-name) or $TENSORBOARD_DIR")
        if experiment is None:
            experiment = datetime.datetime.now().strftime("%Y%m%d_%H%M%S")
        self.log_dir = env_dir or os.path.join("tensorboard_log", str(project), str(experiment))
        os.makedirs(self.log_dir, exist_ok=True)
        try:
            from torch.utils.tensorboard import SummaryWriter
        except ImportError as e:  # pragma: no cover - depends on the environment
            raise RuntimeError("--use-tensorboard needs the `tensorboard` package") from e
        self._writer = SummaryWriter(self.log_dir)
        logger.info("TensorBoard events go to %s", self.log_dir)

    def log(self, data: dict, step):
        for k, v in data.items():
            if isinstance(v, (int, float)):
                self._writer.add_scalar(k, v, step)

    def finish(self):
        self._writer.close()
