"""Tensor / sequence-parallel communication primitives with autograd.

Baseline transport is NCCL via ``torch.distributed``; the fused sm_100a paths
(all-gather->GEMM, GEMM->reduce-scatter over NVLink peer memory) replace the
pair (collective, GEMM) inside the linear layers when symmetric memory is up.
Sequence parallel shards the token dimension of the residual stream across TP.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from slime_b200.parallel import state as mpu


def _tp():
    return mpu.get_tensor_model_parallel_group(), mpu.get_tensor_model_parallel_world_size()


class _CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel linear)."""

    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, g):
        group, n = _tp()
        if n > 1:
            g = g.contiguous()
            dist.all_reduce(g, group=group)
        return g


class _ReduceFromTP(torch.autograd.Function):
    """All-reduce forward, identity backward (output of a row-parallel linear)."""

    @staticmethod
    def forward(ctx, x):
        group, n = _tp()
        if n > 1:
            x = x.contiguous()
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g


def _all_gather_dim0(x, group, n):
    out = torch.empty((x.shape[0] * n, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def _reduce_scatter_dim0(x, group, n):
    out = torch.empty((x.shape[0] // n, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
    return out


class _GatherFromSP(torch.autograd.Function):
    """All-gather tokens forward, reduce-scatter backward (entering a column-parallel linear under SP)."""

    @staticmethod
    def forward(ctx, x):
        group, n = _tp()
        return _all_gather_dim0(x, group, n) if n > 1 else x

    @staticmethod
    def backward(ctx, g):
        group, n = _tp()
        return _reduce_scatter_dim0(g, group, n) if n > 1 else g


class _ReduceScatterToSP(torch.autograd.Function):
    """Reduce-scatter tokens forward, all-gather backward (leaving a row-parallel linear under SP)."""

    @staticmethod
    def forward(ctx, x):
        group, n = _tp()
        return _reduce_scatter_dim0(x, group, n) if n > 1 else x

    @staticmethod
    def backward(ctx, g):
        group, n = _tp()
        return _all_gather_dim0(g, group, n) if n > 1 else g


class _ScatterToSP(torch.autograd.Function):
    """Keep this rank's token slice forward, all-gather backward (after the embedding)."""

    @staticmethod
    def forward(ctx, x):
        group, n = _tp()
        if n == 1:
            return x
        r = mpu.get_tensor_model_parallel_rank()
        per = x.shape[0] // n
        return x[r * per : (r + 1) * per].contiguous()

    @staticmethod
    def backward(ctx, g):
        group, n = _tp()
        return _all_gather_dim0(g, group, n) if n > 1 else g


class _GatherFromSPNoReduce(torch.autograd.Function):
    """All-gather forward, slice backward (before the LM head: gradients are per-token, not partial sums)."""

    @staticmethod
    def forward(ctx, x):
        group, n = _tp()
        return _all_gather_dim0(x, group, n) if n > 1 else x

    @staticmethod
    def backward(ctx, g):
        group, n = _tp()
        if n == 1:
            return g
        r = mpu.get_tensor_model_parallel_rank()
        per = g.shape[0] // n
        return g[r * per : (r + 1) * per].contiguous()


copy_to_tensor_model_parallel_region = _CopyToTP.apply
reduce_from_tensor_model_parallel_region = _ReduceFromTP.apply
gather_from_sequence_parallel_region = _GatherFromSP.apply
reduce_scatter_to_sequence_parallel_region = _ReduceScatterToSP.apply
scatter_to_sequence_parallel_region = _ScatterToSP.apply
gather_from_sequence_parallel_region_no_reduce = _GatherFromSPNoReduce.apply


def set_tp_attrs(param, is_parallel: bool, dim: int = -1, stride: int = 1, mode: str | None = None):
    """Attributes read by weight sync and checkpointing (same names as Megatron-core)."""
    param.tensor_model_parallel = is_parallel
    param.partition_dim = dim
    param.partition_stride = stride
    param.parallel_mode = mode
    return param


# CUDA RNG tracker equivalent: one generator per (tp-rank-dependent | tp-invariant) domain.
class RngTracker:
    def __init__(self):
        self.states = {}

    def add(self, name: str, seed: int, device=None):
        g = torch.Generator(device=device or ("cuda" if torch.cuda.is_available() else "cpu"))
        g.manual_seed(seed)
        self.states[name] = g

    def get(self, name: str) -> torch.Generator:
        return self.states[name]


_RNG = RngTracker()


def get_rng_tracker() -> RngTracker:
    return _RNG


def model_parallel_seed(seed: int, device=None):
    """`default`: same across TP (replicated params); `tp`: differs per TP rank (sharded params)."""
    _RNG.add("default", seed, device)
    _RNG.add("tp", seed + 2718 + mpu.get_tensor_model_parallel_rank(), device)
    _RNG.add("ep", seed + 1024 + 100 * mpu.get_expert_model_parallel_rank() + mpu.get_expert_tensor_parallel_rank(), device)
