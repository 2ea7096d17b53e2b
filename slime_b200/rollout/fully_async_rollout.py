"""Fully asynchronous rollout: a background worker keeps a fixed number of prompt groups in flight *across* rollout
boundaries, so a training step never waits for the slowest trajectory of "its" batch; it takes the first
``rollout_batch_size`` groups that finish.

``--rollout-function-path slime.rollout.fully_async_rollout.generate_rollout_fully_async`` (with ``train_async.py``).
Per-sample generation / reward hooks (``--custom-generate-function-path``, ``--custom-rm-path``) apply as usual
because the worker runs the stock ``generate_and_rm_group``.

Design: one thread owns an asyncio loop. A pump coroutine tops the in-flight set up to
``sglang_server_concurrency x engines`` whenever a task finishes (event-driven, no polling interval), and holds off
while ``concurrency`` finished groups are already waiting, so generation cannot run arbitrarily far ahead of training.
Groups with an ABORTED sample (weight update in progress) go back to the data buffer and are regenerated under the
new weights. Parity: slime/rollout/fully_async_rollout.py:45-274.
"""

from __future__ import annotations

import asyncio
import atexit
import logging
import queue
import threading
import time

from slime_b200.rollout.sglang_rollout import GenerateState, generate_and_rm_group, get_rollout_num_engines
from slime_b200.utils.types import Sample

__all__ = ["AsyncRolloutWorker", "generate_rollout_fully_async"]
logger = logging.getLogger(__name__)

_worker: "AsyncRolloutWorker | None" = None
_worker_guard = threading.Lock()


class AsyncRolloutWorker:
    def __init__(self, args, data_buffer, concurrency: int = 10, generate_group=generate_and_rm_group):
        self.args, self.data_buffer, self.concurrency = args, data_buffer, max(1, concurrency)
        self.output_queue: "queue.Queue[tuple[int, list[Sample]]]" = queue.Queue()
        self.running = False
        self.worker_thread: threading.Thread | None = None
        self._generate_group = generate_group
        self._loop: asyncio.AbstractEventLoop | None = None
        self._wake: asyncio.Event | None = None
        self._in_flight = 0
        self.requeued = 0
        self.state = GenerateState(args)

    # ------------------------------------------------------------------ control
    def start(self):
        if self.worker_thread is not None and self.worker_thread.is_alive():
            return
        self.running = True
        self.worker_thread = threading.Thread(target=lambda: asyncio.run(self._pump()), name="fully-async-rollout", daemon=True)
        self.worker_thread.start()

    def stop(self, timeout: float = 5.0):
        self.running = False
        self._poke()
        if self.worker_thread is not None and self.worker_thread.is_alive():
            self.worker_thread.join(timeout)

    def _poke(self):
        loop, wake = self._loop, self._wake
        if loop is not None and wake is not None and not loop.is_closed():
            loop.call_soon_threadsafe(wake.set)

    def queue_size(self) -> int:
        return self.output_queue.qsize()

    def get_completed_groups(self, limit: int | None = None, timeout: float = 0.0) -> list[tuple[int, list[Sample]]]:
        """Up to ``limit`` finished groups; waits at most ``timeout`` seconds for the first one. Never takes more than
        asked: a finished group has consumed its prompt and must not be dropped."""
        out: list[tuple[int, list[Sample]]] = []
        while limit is None or len(out) < limit:
            try:
                out.append(self.output_queue.get(timeout=timeout) if (timeout and not out) else self.output_queue.get_nowait())
            except queue.Empty:
                break
        if out:
            self._poke()  # room in the finished queue again
        return out

    # --------------------------------------------------------------------- loop
    async def _pump(self):
        self._loop, self._wake = asyncio.get_running_loop(), asyncio.Event()
        tasks: set[asyncio.Task] = set()
        next_gid = 0
        while self.running:
            while self.running and len(tasks) < self.concurrency and self.output_queue.qsize() < self.concurrency:
                try:
                    groups = self.data_buffer.get_samples(1)
                except Exception:  # noqa: BLE001
                    logger.exception("fully-async: data buffer failed")
                    groups = []
                if not groups:
                    break
                for group in groups:
                    t = asyncio.create_task(self._generate_group(self.args, group, sampling_params=dict(self.state.sampling_params),
                                                                 evaluation=False))  # fmt: skip
                    t.add_done_callback(self._on_done(next_gid, tasks))
                    tasks.add(t)
                    next_gid += 1
            self._in_flight = len(tasks)
            self._wake.clear()
            try:
                await asyncio.wait_for(self._wake.wait(), timeout=1.0)  # the timeout only covers an empty data buffer
            except asyncio.TimeoutError:
                pass
        if tasks:
            logger.info("fully-async: draining %d in-flight groups", len(tasks))
            await asyncio.wait(tasks, timeout=30)

    def _on_done(self, gid: int, tasks: set):
        def cb(task: asyncio.Task):
            tasks.discard(task)
            try:
                group = task.result()
            except asyncio.CancelledError:
                return
            except Exception:  # noqa: BLE001
                logger.exception("fully-async: generation of group %d raised", gid)
                group = None
            if isinstance(group, list):
                if any(getattr(s, "status", None) == Sample.Status.ABORTED for s in group):
                    self.requeued += 1
                    try:
                        self.data_buffer.add_samples([group])
                    except Exception:  # noqa: BLE001
                        logger.exception("fully-async: could not requeue aborted group %d", gid)
                else:
                    self.output_queue.put((gid, group))
            elif group is not None:
                logger.warning("fully-async: group function returned %s, expected a list of samples", type(group).__name__)
            self._wake.set()

        return cb


def _get_worker(args, data_buffer) -> AsyncRolloutWorker:
    global _worker
    with _worker_guard:
        if _worker is None or _worker.worker_thread is None or not _worker.worker_thread.is_alive():
            conc = args.sglang_server_concurrency * get_rollout_num_engines(args)
            logger.info("starting the fully-async rollout worker with %d groups in flight", conc)
            _worker = AsyncRolloutWorker(args, data_buffer, concurrency=conc)
            _worker.start()
        return _worker


def _stop_worker():
    global _worker
    with _worker_guard:
        if _worker is not None:
            _worker.stop()
            _worker = None


atexit.register(_stop_worker)


def collect_groups(worker: AsyncRolloutWorker, target: int, rollout_id: int = 0, log_every: float = 30.0) -> list[list[Sample]]:
    got: dict[int, list[Sample]] = {}
    t0 = last = time.time()
    while len(got) < target:
        for gid, group in worker.get_completed_groups(limit=target - len(got), timeout=0.05):
            got[gid] = group
        now = time.time()
        if now - last > log_every:
            last = now
            logger.info("fully-async rollout %d: %d/%d groups after %.0fs (queue %d)", rollout_id, len(got), target,
                        now - t0, worker.queue_size())  # fmt: skip

    def first_index(group):
        return next((int(s.index) for s in group if getattr(s, "index", None) is not None), 0)

    return sorted(got.values(), key=first_index)


def generate_rollout_fully_async(args, rollout_id, data_buffer, evaluation: bool = False):
    if evaluation:
        raise ValueError("the fully-async rollout has no evaluation mode; use the default eval function")
    assert args.rollout_global_dataset
    worker = _get_worker(args, data_buffer)
    t0 = time.time()
    out = collect_groups(worker, args.rollout_batch_size, rollout_id)
    logger.info("fully-async rollout %d: %d groups in %.1fs, %d finished groups waiting", rollout_id, len(out),
                time.time() - t0, worker.queue_size())  # fmt: skip
    return out
