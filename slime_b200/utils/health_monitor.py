"""Rollout-engine failure detection.

One monitor thread per server group polls ``engine.health_generate(timeout)``; an engine that fails is
shut down, killed and its slot set to ``None`` so the next weight update restarts and fully re-syncs it.
Monitoring is paused while engines are offloaded (they cannot answer) and resumed before generation.
Parity: slime/utils/health_monitor.py:10-177; defaults interval 30 s / timeout 30 s / first wait 0 s.
All failures are observed on the host (RPC errors, HTTP timeouts); nothing is done to a GPU.
"""

from __future__ import annotations

import logging
import threading
import time

logger = logging.getLogger(__name__)


class RolloutHealthMonitor:
    def __init__(self, server_group, args, get=None, kill=None):
        from slime_b200.runtime import actors

        self.group = server_group
        self.interval = args.rollout_health_check_interval
        self.timeout = args.rollout_health_check_timeout
        self.first_wait = args.rollout_health_check_first_wait
        self._get = get or actors.get
        self._kill = kill or actors.kill
        self._stop = threading.Event()
        self._paused = threading.Event()
        self._paused.set()  # starts paused until the first resume()
        self._thread: threading.Thread | None = None
        self._need_first_wait = True
        self.failures = 0

    def start(self) -> bool:
        if not getattr(self.group, "all_engines", None):
            return False
        if self._thread is not None:
            return True
        self._thread = threading.Thread(target=self._loop, daemon=True, name="rollout-health-monitor")
        self._thread.start()
        return True

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=self.interval + self.timeout + 5)
            self._thread = None

    def pause(self):
        self._paused.set()

    def resume(self):
        self._need_first_wait = True
        self._paused.clear()

    def is_checking_enabled(self) -> bool:
        return not self._paused.is_set()

    def _sleep(self, seconds: float) -> bool:
        """Sleep in small slices; False when stopped or paused meanwhile."""
        end = time.time() + seconds
        while time.time() < end:
            if self._stop.is_set() or self._paused.is_set():
                return False
            time.sleep(min(0.05, max(end - time.time(), 0)))
        return True

    def _loop(self):
        while not self._stop.is_set():
            if self._paused.is_set():
                time.sleep(0.05)
                continue
            if self._need_first_wait:
                self._need_first_wait = False
                if self.first_wait > 0 and not self._sleep(self.first_wait):
                    continue
            self._check_all()
            self._sleep(self.interval)

    def _check_all(self):
        for i, engine in enumerate(list(self.group.all_engines)):
            if self._stop.is_set() or self._paused.is_set():
                return
            if engine is None:
                continue
            try:
                self._get(engine.health_generate.remote(timeout=self.timeout), timeout=self.timeout + 5)
            except Exception as e:  # noqa: BLE001
                logger.error("health check failed for rollout engine %d: %r", i, e)
                self._kill_engine(i)

    def _kill_engine(self, i: int):
        """Mark the whole engine (all its node slots) dead and free its process."""
        per = max(1, getattr(self.group, "nodes_per_engine", 1))
        first = (i // per) * per
        self.failures += 1
        for j in range(first, first + per):
            engine = self.group.all_engines[j]
            if engine is None:
                continue
            try:
                self._get(engine.shutdown.remote(), timeout=10)
            except Exception:  # noqa: BLE001
                pass
            try:
                self._kill(engine)
            except Exception as e:  # noqa: BLE001
                logger.warning("killing engine %d failed: %r", j, e)
            self.group.all_engines[j] = None
