"""Trainer-side profiling hooks.

``--use-pytorch-profiler --profile-target train_overall|train_actor|train_log_probs --profile-step-start S
--profile-step-end E`` wraps either the whole train loop (stepped once per rollout) or one of the micro-batch loops
in a ``torch.profiler`` schedule and writes gzip'd traces under ``--tensorboard-dir``.
``--record-memory-history --memory-recorder torch|memray`` records allocator history from start-up, dumps a snapshot
after ``--memory-snapshot-num-steps`` rollouts and, for the torch recorder, also when the allocator reports an
out-of-memory condition. Parity: slime/observability/profile_utils.py:14-179.
"""

from __future__ import annotations

import logging
import time
import traceback
from pathlib import Path

import torch

logger = logging.getLogger(__name__)


def _rank() -> int:
    return torch.distributed.get_rank() if torch.distributed.is_available() and torch.distributed.is_initialized() else 0


def _create_torch_profiler(args, name: str):
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    first, last = args.profile_step_start, args.profile_step_end
    return torch.profiler.profile(
        activities=acts,
        schedule=torch.profiler.schedule(wait=max(first - 1, 0), warmup=1 if first > 0 else 0, active=last - first, repeat=1),
        on_trace_ready=torch.profiler.tensorboard_trace_handler(args.tensorboard_dir, worker_name=f"{name}_rank_{_rank()}",
                                                                use_gzip=True),
        record_shapes=True, with_stack=True, profile_memory=True, with_flops=True,
    )  # fmt: skip


def _profile_simple_loop(iterator, args, name: str):
    if not (args.use_pytorch_profiler and name in args.profile_target):
        yield from iterator
        return
    prof = _create_torch_profiler(args, name)
    prof.start()
    try:
        for item in iterator:
            yield item
            prof.step()
    finally:
        prof.stop()


class _MemoryRecorder:
    def __init__(self, args):
        self.path = Path(args.memory_snapshot_dir) / f"memory_snapshot_time{time.time()}_rank{_rank()}_{args.memory_snapshot_path}"

    @staticmethod
    def create(args):
        return {"torch": _TorchMemoryRecorder, "memray": _MemrayRecorder}[args.memory_recorder](args)


class _TorchMemoryRecorder(_MemoryRecorder):
    recording = False

    def start(self):
        if not torch.cuda.is_available() or not hasattr(torch.cuda.memory, "_record_memory_history"):
            logger.warning("allocator history is unavailable on this build; memory recording is off")
            return
        torch.cuda.memory._record_memory_history(max_entries=1_000_000, stacks="all")
        self.recording = True
        attach = getattr(torch._C, "_cuda_attach_out_of_memory_observer", None)
        if attach is None:
            return

        def on_oom(device, alloc, device_alloc, device_free):
            logger.error("allocator ran out of memory (device=%s request=%s allocated=%s free=%s); snapshot -> %s",
                         device, alloc, device_alloc, device_free, self.path)  # fmt: skip
            traceback.print_stack()
            torch.cuda.memory._dump_snapshot(str(self.path))

        attach(on_oom)

    def stop(self):
        if not self.recording:
            return
        self.path.parent.mkdir(parents=True, exist_ok=True)
        torch.cuda.memory._dump_snapshot(str(self.path))
        torch.cuda.memory._record_memory_history(enabled=None)
        self.recording = False
        logger.info("memory snapshot written to %s", self.path)


class _MemrayRecorder(_MemoryRecorder):
    def __init__(self, args):
        super().__init__(args)
        assert args.memory_snapshot_num_steps is not None, "--memory-recorder memray needs --memory-snapshot-num-steps"
        self._tracker = None

    def start(self):
        import memray

        self.path.parent.mkdir(parents=True, exist_ok=True)
        self._tracker = memray.Tracker(file_name=self.path, native_traces=True)
        self._tracker.__enter__()

    def stop(self):
        if self._tracker is not None:
            self._tracker.__exit__(None, None, None)
            self._tracker = None
            logger.info("memray capture written to %s", self.path)


class TrainProfiler:
    def __init__(self, args):
        self.args = args
        overall = "train_overall" in (args.profile_target or [])
        self._prof = _create_torch_profiler(args, "train_overall") if args.use_pytorch_profiler and overall else None
        self._mem = None
        if args.record_memory_history and overall:
            self._mem = _MemoryRecorder.create(args)
            self._mem.start()

    def on_init_end(self):
        if self._prof is not None:
            self._prof.start()

    def step(self, rollout_id: int):
        if self._prof is not None:
            self._prof.step()
        n = self.args.memory_snapshot_num_steps
        if self._mem is not None and n is not None and rollout_id == n - 1:
            self._mem.stop()

    def iterate_train_actor(self, iterator):
        return _profile_simple_loop(iterator, self.args, "train_actor")

    def iterate_train_log_probs(self, iterator):
        return _profile_simple_loop(iterator, self.args, "train_log_probs")
