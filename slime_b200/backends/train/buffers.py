"""Contiguous parameter / gradient buffers for data-parallel training.

All bf16 parameters of a model chunk are views into one flat buffer and every
parameter gets an fp32 ``main_grad`` view into a second flat buffer (gradients are
accumulated there directly by the wgrad GEMMs). The flat length is padded so it
splits evenly across the data-parallel group; rank ``r`` owns slice ``r`` for the
sharded optimizer (ZeRO-1), which is what Megatron's DDP + DistributedOptimizer
provide to the reference (slime/backends/megatron_utils/model.py:269-344).

Dense and expert parameters use separate buffers because they are reduced over
different groups (DP x CP vs. expert-DP).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

ALIGN = 128  # elements; keeps every shard boundary 256-byte aligned for bf16


class FlatBuffer:
    def __init__(self, params: list[torch.nn.Parameter], names: list[str], group, group_size: int, group_rank: int,
                 device, grad_dtype=torch.float32, allocator=None, symmetric=False):  # fmt: skip
        self.params, self.names = params, names
        # `group` may be a getter: communicators can be released and rebuilt between phases (parallel/state.py), so the
        # handle is looked up at every use instead of being cached
        self._group = group
        self.group_size, self.group_rank = group_size, group_rank
        self.offsets: list[tuple[int, int]] = []
        off = 0
        for p in params:
            n = p.numel()
            self.offsets.append((off, off + n))
            off += -(-n // ALIGN) * ALIGN
        chunk = ALIGN * group_size
        self.numel = max(-(-off // chunk) * chunk, chunk)
        self.shard_size = self.numel // group_size
        dtype = params[0].dtype if params else torch.bfloat16
        alloc = allocator or (lambda n, dt: torch.zeros(n, dtype=dt, device=device))
        self.fused = None  # FusedDataParallel when both buffers live in symmetric memory
        self.param_store = self.grad_store = None
        if symmetric and grad_dtype == torch.float32:
            from slime_b200.parallel.fused_dp import FusedDataParallel, SymmetricStorage

            self.param_store = SymmetricStorage(self.numel, dtype, device, self.group)
            self.grad_store = SymmetricStorage(self.numel, grad_dtype, device, self.group)
            self.param_data, self.grad_data = self.param_store.tensor, self.grad_store.tensor
            self.fused = FusedDataParallel.__new__(FusedDataParallel)  # finished below, once the views exist
        else:
            self.param_data = alloc(self.numel, dtype)
            self.grad_data = alloc(self.numel, grad_dtype)
        for p, (s, e) in zip(params, self.offsets):
            view = self.param_data[s:e].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.main_grad = self.grad_data[s:e].view(p.shape)
            p.grad_added_to_main_grad = False
        if self.fused is not None:
            self.fused.__init__(self)

    @property
    def group(self):
        g = self._group
        return g() if callable(g) else g

    # ---- shard views ----------------------------------------------------------------
    def shard_range(self, rank: int | None = None) -> tuple[int, int]:
        r = self.group_rank if rank is None else rank
        return r * self.shard_size, (r + 1) * self.shard_size

    def param_shard(self):
        s, e = self.shard_range()
        return self.param_data[s:e]

    def grad_shard(self):
        s, e = self.shard_range()
        return self.grad_data[s:e]

    def zero_grad(self):
        self.grad_data.zero_()
        for p in self.params:
            p.grad = None
            p.grad_added_to_main_grad = False

    def fold_autograd_grads(self):
        """Parameters whose backward returned a ``.grad`` (ops that do not write main_grad directly)."""
        for p in self.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None

    # ---- collectives (NCCL baseline; the fused path lives in parallel/fused_dp.py) ------------
    def reduce_scatter_grads(self, average: bool = False, async_op: bool = False):
        if self.group_size == 1 or self.fused is not None:  # fused: the optimizer step reduces over peer memory itself
            return None
        op = dist.ReduceOp.AVG if average else dist.ReduceOp.SUM
        return dist.reduce_scatter_tensor(self.grad_shard(), self.grad_data, op=op, group=self.group, async_op=async_op)

    def all_reduce_grads(self, average: bool = False):
        if self.group_size > 1:
            dist.all_reduce(self.grad_data, op=dist.ReduceOp.AVG if average else dist.ReduceOp.SUM, group=self.group)

    def all_gather_params(self, async_op: bool = False):
        if self.group_size == 1 or self.fused is not None:  # fused: the Adam kernel stored into every rank's buffer
            return None
        return dist.all_gather_into_tensor(self.param_data, self.param_shard().clone(), group=self.group, async_op=async_op)

    def params_in_range(self, s: int, e: int):
        """(name, param, param-local slice, shard-local slice) for params overlapping flat range [s, e)."""
        for name, p, (ps, pe) in zip(self.names, self.params, self.offsets):
            lo, hi = max(s, ps), min(e, pe)
            if lo < hi:
                yield name, p, (lo - ps, hi - ps), (lo - s, hi - s)
