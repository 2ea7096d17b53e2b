"""Data-parallel reduce-scatter + Adam + all-gather over NVLink peer memory (``csrc/dp_fused.cu``).

A ``FlatBuffer`` whose parameter and gradient storage were allocated from symmetric memory can be reached from every
rank of its data-parallel group: ``SymmetricStorage`` holds the peers' device pointers (and the NVSwitch multicast
address when the fabric supports it). ``FusedDataParallel`` then replaces

    NCCL reduce-scatter(grads) -> squared norm -> Adam on the shard -> NCCL all-gather(params)

by two kernels that read / write the peers' buffers themselves, bracketed by a bounded signal-pad barrier. The squared
norm still crosses ranks as one scalar through the regular process group.

Used when: CUDA, group size in 2..8, every rank on one NVLink domain, the trainer does not release its buffers between
phases. Anything else keeps the NCCL path in ``FlatBuffer`` (also the path every CPU test runs).
"""

from __future__ import annotations

import ctypes
import logging
import os

import torch
import torch.distributed as dist

logger = logging.getLogger(__name__)


def symmetric_memory_usable(group_size: int, device) -> bool:
    if os.environ.get("SLIME_B200_DISABLE_FUSED_DP") == "1" or os.environ.get("SLIME_B200_LIBRARY_OPS") == "1":
        return False
    if group_size < 2 or group_size > 8 or torch.device(device).type != "cuda":
        return False
    try:
        import torch.distributed._symmetric_memory as symm_mem  # noqa: F401
    except ImportError:
        return False
    return True


class SymmetricStorage:
    """One symmetric allocation plus what is needed to address it from kernels."""

    def __init__(self, numel: int, dtype, device, group):
        import torch.distributed._symmetric_memory as symm_mem

        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, group)
        self.world, self.rank = self.handle.world_size, self.handle.rank
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.mc_ptr = int(self.handle.multicast_ptr or 0)
        self.pad_ptrs = [int(p) for p in self.handle.signal_pad_ptrs]
        self.pad_words = int(symm_mem.get_signal_pad_size()) // 4

    def c_ptrs(self, use_multicast: bool):
        src = [self.mc_ptr] if use_multicast else self.ptrs
        return (ctypes.c_void_p * len(src))(*src)


class FusedDataParallel:
    """Fused collectives for one ``FlatBuffer`` (its ``param_store`` / ``grad_store`` are ``SymmetricStorage``)."""

    def __init__(self, buffer):
        from slime_b200.ops import _lib

        self.b = buffer
        self.g, self.p = buffer.grad_store, buffer.param_store
        self.world, self.rank = self.g.world, self.g.rank
        self.use_mc = bool(self.g.mc_ptr and self.p.mc_ptr) and os.environ.get("SLIME_B200_DISABLE_MULTIMEM") != "1"
        self.partials = torch.zeros(148 * 8, dtype=torch.float32, device=buffer.grad_data.device)
        self.epoch = 0
        self._lib = _lib
        # barrier words sit at the top of the signal pad, away from the slots torch's own primitives use
        self.base_word = self.g.pad_words - 16
        self._pads = (ctypes.c_void_p * self.world)(*self.g.pad_ptrs)
        self._align = torch.zeros(1, dtype=torch.float32, device=buffer.grad_data.device)
        logger.info("fused data-parallel step: %d ranks, %s", self.world, "NVSwitch multimem" if self.use_mc else "P2P loads/stores")

    def barrier(self):
        lib, P = self._lib.lib(), self._lib.ptr
        self.epoch += 1
        rc = lib.sb_symm_barrier(self._pads, self.rank, self.world, self.epoch, self.base_word,
                                 P(self._lib.status_word(self.b.grad_data.device)), self._lib.stream())  # fmt: skip
        self._lib.check(rc, "sb_symm_barrier")

    def reduce_shard(self, ctl: torch.Tensor):
        """grad shard <- sum over ranks (in place in this rank's buffer); ctl[0] += squared norm of the shard."""
        lib, P = self._lib.lib(), self._lib.ptr
        s, e = self.b.shard_range()
        # Ranks reach the optimizer step with whatever skew their rollouts and micro-batch counts left (seconds, with
        # long-tail generations). A one-element NCCL all-reduce absorbs that skew on the device with NCCL's own,
        # unbounded-by-us wait, so the bounded barrier below only ever waits for launch jitter and its limit stays a
        # fault detector instead of a limit on skew.
        dist.all_reduce(self._align, group=self.b.group)
        self.barrier()  # every rank's backward has finished writing its gradient buffer
        rc = lib.sb_dp_reduce_shard(self.g.c_ptrs(self.use_mc), self.world, self.rank, int(self.use_mc), s, e - s,
                                    P(self.b.grad_shard()), P(self.partials), P(ctl),
                                    P(self._lib.status_word(self.b.grad_data.device)), self._lib.stream())  # fmt: skip
        self._lib.check(rc, "sb_dp_reduce_shard")

    def adam_bcast(self, st: dict, *, lr, b1, b2, eps, wd, bc1, bc2, grad_scale, clip, ctl, stateless):
        lib, P = self._lib.lib(), self._lib.ptr
        s, e = self.b.shard_range()
        rc = lib.sb_dp_adam_bcast(P(st["master"]), P(st.get("exp_avg")), P(st.get("exp_avg_sq")), P(self.b.grad_shard()),
                                  self.p.c_ptrs(self.use_mc), self.world, self.rank, int(self.use_mc), s, e - s, lr, b1, b2,
                                  eps, wd, bc1, bc2, grad_scale, float(clip or 0.0), P(ctl), int(stateless),
                                  self._lib.stream())  # fmt: skip
        self._lib.check(rc, "sb_dp_adam_bcast")
        self.barrier()  # every rank's parameters are complete before anyone runs the next forward
