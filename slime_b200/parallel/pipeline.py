"""Pipeline-parallel schedules (forward-only and 1F1B) over NCCL point-to-point.

Activations travel as one ``[2, T, H]`` tensor (branch output + residual stream). Every stage
builds the micro-batch locally from the same rollout payload, so tensor shapes are known
without a shape exchange even though sequence lengths vary per micro-batch. Send/recv pairs
are issued with ``batch_isend_irecv`` on the pipeline group; interleaved (virtual) stages run
their chunks back to back on the same rank.
Replaces Megatron's ``get_forward_backward_func`` (slime/backends/megatron_utils/model.py:460,647).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from slime_b200.parallel import state as mpu


def _shape_for(batch, model, args):
    T = batch["tokens"].shape[1]
    if model.chunks[0].sequence_parallel:
        T //= mpu.get_tensor_model_parallel_world_size()
    return (2, T, model.cfg.hidden_size)


def _p2p(send_prev=None, recv_prev_shape=None, send_next=None, recv_next_shape=None, dtype=torch.bfloat16, device=None):
    ops, recv_prev, recv_next = [], None, None
    prev_r, next_r = mpu.get_pipeline_model_parallel_prev_rank(), mpu.get_pipeline_model_parallel_next_rank()
    group = mpu.get_pipeline_model_parallel_group()
    if send_prev is not None:
        ops.append(dist.P2POp(dist.isend, send_prev.contiguous(), prev_r, group))
    if recv_prev_shape is not None:
        recv_prev = torch.empty(recv_prev_shape, dtype=dtype, device=device)
        ops.append(dist.P2POp(dist.irecv, recv_prev, prev_r, group))
    if send_next is not None:
        ops.append(dist.P2POp(dist.isend, send_next.contiguous(), next_r, group))
    if recv_next_shape is not None:
        recv_next = torch.empty(recv_next_shape, dtype=dtype, device=device)
        ops.append(dist.P2POp(dist.irecv, recv_next, next_r, group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return recv_prev, recv_next


def _get_batch(model, data_iterator, args):
    from slime_b200.backends.train.data import get_batch
    from slime_b200.backends.train.model import BATCH_KEYS

    keys = [k for k in BATCH_KEYS if k in data_iterator.rollout_data]
    return get_batch(data_iterator, keys, getattr(args, "data_pad_size_multiplier", 128), device=model.device)


def run_forward_only(model, data_iterator, num_microbatches: int, forward_step, args) -> list[dict]:
    pp = mpu.get_pipeline_model_parallel_world_size()
    first, last = mpu.is_pipeline_first_stage(), mpu.is_pipeline_last_stage()
    results = []
    dtype = model.chunks[0].dtype
    for _ in range(num_microbatches):
        batch = _get_batch(model, data_iterator, args)
        x = None
        if pp > 1 and not first:
            x, _ = _p2p(recv_prev_shape=_shape_for(batch, model, args), dtype=dtype, device=model.device)
        for chunk in model.chunks:  # virtual chunks hosted on this rank run back to back
            x, res = forward_step(batch, chunk, x)
        if pp > 1 and not last:
            _p2p(send_next=x)
        if last:
            results.append(res)
    return results


def run_forward_backward(model, data_iterator, num_microbatches: int, forward_step, args) -> list[dict]:
    """Non-interleaved 1F1B: warm-up forwards, steady 1F1B pairs, cool-down backwards."""
    pp, rank = mpu.get_pipeline_model_parallel_world_size(), mpu.get_pipeline_model_parallel_rank()
    first, last = mpu.is_pipeline_first_stage(), mpu.is_pipeline_last_stage()
    dtype = model.chunks[0].dtype
    logs: list[dict] = []

    def fwd(batch, inp):
        if inp is not None:
            inp.requires_grad_(True)
        x = inp
        for chunk in model.chunks:
            x, log = forward_step(batch, chunk, x)
        if last:
            logs.append(log)
        return x

    def bwd(out, inp, grad_out):
        if last:
            out.backward()
        else:
            torch.autograd.backward(out, grad_tensors=grad_out)
        return None if inp is None else inp.grad

    if pp == 1:
        for _ in range(num_microbatches):
            batch = _get_batch(model, data_iterator, args)
            bwd(fwd(batch, None), None, None)
        return logs

    warmup = min(pp - rank - 1, num_microbatches)
    steady = num_microbatches - warmup
    pending: list[tuple] = []  # (input, output, shape)
    inp = None
    for _ in range(warmup):
        batch = _get_batch(model, data_iterator, args)
        shape = _shape_for(batch, model, args)
        if not first:
            inp, _ = _p2p(recv_prev_shape=shape, dtype=dtype, device=model.device)
        out = fwd(batch, inp)
        _p2p(send_next=out.detach())
        pending.append((inp, out, shape))
    for i in range(steady):
        batch = _get_batch(model, data_iterator, args)
        shape = _shape_for(batch, model, args)
        if not first:
            inp, _ = _p2p(recv_prev_shape=shape, dtype=dtype, device=model.device)
        out = fwd(batch, inp)
        grad_out = None
        if not last:
            _, grad_out = _p2p(send_next=out.detach(), recv_next_shape=shape, dtype=dtype, device=model.device)
        pending.append((inp, out, shape))
        b_inp, b_out, _ = pending.pop(0)
        g = bwd(b_out, b_inp, grad_out)
        if not first:
            _p2p(send_prev=g)
    while pending:
        b_inp, b_out, shape = pending.pop(0)
        grad_out = None
        if not last:
            _, grad_out = _p2p(recv_next_shape=shape, dtype=dtype, device=model.device)
        g = bwd(b_out, b_inp, grad_out)
        if not first:
            _p2p(send_prev=g)
    return logs
