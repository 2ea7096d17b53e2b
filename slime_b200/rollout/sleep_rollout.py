"""A rollout function that never returns: keeps the engines up (serving, debugging) while the driver waits.
``--rollout-function-path slime.rollout.sleep_rollout.sleep``. Parity: slime/rollout/sleep_rollout.py:7-12."""

import logging
import time

logger = logging.getLogger(__name__)


def sleep(args, rollout_id, data_source, evaluation=False):
    hours = 0
    while True:
        time.sleep(3600)
        hours += 1
        logger.info("rollout function has been sleeping for %d h", hours)
