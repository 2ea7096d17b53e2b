"""Process-group helpers that go beyond the default world.

* ``init_extra_process_group``: a group whose members are not all in this process's default world: the weight-sync
  group made of one trainer rank and every rollout-engine GPU (the engines have no default group at all). It
  rendezvouses on its own TCP store and is registered under ``group_name`` so collectives accept it.
* a gloo side group for host-side object collectives next to the NCCL world.
* ``distributed_masked_whiten``: advantage whitening with statistics reduced over data-parallel ranks.

Parity: slime/utils/distributed_utils.py:20-170.
"""

from __future__ import annotations

from datetime import timedelta

import torch
import torch.distributed as dist

_GLOO_GROUP = None


def init_gloo_group():
    """A gloo group over the default world (object gathers, barriers that must not touch the GPU stream)."""
    global _GLOO_GROUP
    if _GLOO_GROUP is None:
        if dist.get_backend() == "gloo":
            _GLOO_GROUP = dist.group.WORLD
        else:
            _GLOO_GROUP = dist.new_group(backend="gloo")
    return _GLOO_GROUP


def get_gloo_group():
    if _GLOO_GROUP is None:
        raise RuntimeError("gloo group not initialised; call init_gloo_group() after init_process_group()")
    return _GLOO_GROUP


def set_gloo_group(group) -> None:
    global _GLOO_GROUP
    _GLOO_GROUP = group


def init_extra_process_group(backend: str = "nccl", init_method: str | None = None, world_size: int = -1, rank: int = -1,
                             group_name: str = "extra", timeout: timedelta | None = None, device_id=None):  # fmt: skip
    """Join (or create, as rank 0) the process group ``group_name`` that lives on its own rendezvous.

    Every member calls this with the same ``init_method`` (``tcp://host:port``), ``world_size`` and ``group_name``
    and a distinct ``rank``. The returned group works with ``dist.broadcast(..., group=pg)`` etc.; it does not need,
    and does not touch, the default process group. NCCL is replaced by gloo on hosts without CUDA so the same
    control flow runs on CPU.
    """
    from torch.distributed.distributed_c10d import (Backend, PrefixStore, _new_process_group_helper, _world,
                                                    default_pg_timeout, rendezvous)  # fmt: skip

    if backend == "nccl" and not torch.cuda.is_available():
        backend = "gloo"
    assert init_method is not None and world_size > 0 and 0 <= rank < world_size
    timeout = timeout or default_pg_timeout
    store, rank, world_size = next(iter(rendezvous(init_method, rank, world_size, timeout=timeout)))
    store.set_timeout(timeout)
    kwargs = {}
    if device_id is not None:
        kwargs["device_id"] = device_id
    pg, _ = _new_process_group_helper(world_size, rank, [], Backend(backend), PrefixStore(f"{group_name}/", store),
                                      group_name=group_name, timeout=timeout, **kwargs)  # fmt: skip
    _world.pg_group_ranks[pg] = {i: i for i in range(world_size)}  # global rank == group rank inside this island
    return pg


def distributed_masked_whiten(values: torch.Tensor, mask: torch.Tensor, process_group=None, shift_mean: bool = True,
                              epsilon: float = 1e-8) -> torch.Tensor:  # fmt: skip
    """(values - mean) / sqrt(var + eps) with mean / variance of the masked elements over all ranks of the group."""
    v = values.float()
    m = mask.to(v.dtype)
    stats = torch.stack([(v * m).sum(), (v * v * m).sum(), m.sum()])
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(stats, group=process_group)
    total, total_sq, count = stats.tolist()
    if count == 0:
        raise ValueError("distributed_masked_whiten: the mask selects no element on any rank")
    mean = total / count
    var = max(total_sq / count - mean * mean, 0.0)
    if count > 1:
        var *= count / (count - 1)  # unbiased, like torch.var
    out = (v - mean) * (var + epsilon) ** -0.5
    return out if shift_mean else out + mean


def shutdown_distributed(engines=()) -> None:
    """Orderly end of a distributed process: engines drop their CUDA graphs (see ``Engine.shutdown``), every rank
    arrives, then the process groups are destroyed."""
    import torch
    import torch.distributed as dist

    for e in engines:
        if e is not None and hasattr(e, "shutdown"):
            e.shutdown()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def set_numa_affinity(local_rank: int) -> list[int] | None:
    """Pin this process to the CPUs NVML reports as closest to GPU ``local_rank`` (its NUMA node). Returns the CPU list,
    or None when NVML, the GPU or an allowed CPU among them is not available (nothing is changed then). Same role as
    the affinity step of slime/ray/train_actor.py:47-94 in the reference; here it is opt-in
    (``SLIME_B200_NUMA_AFFINITY=1`` or ``--numa-affinity``), since containers often expose a CPU set of their own."""
    import os

    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        words = -(-os.cpu_count() // 64)
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = [64 * w + b for w, m in enumerate(mask) for b in range(64) if (int(m) >> b) & 1]
        allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return allowed
    except Exception:  # noqa: BLE001 - no NVML, no such GPU, no permission: affinity is an optimisation only
        return None
