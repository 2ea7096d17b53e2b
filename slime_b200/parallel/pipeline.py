"""Pipeline-parallel schedules (forward-only and 1F1B) over NCCL point-to-point.

Activations travel as one ``[2, T, H]`` tensor (branch output + residual stream). Every stage
builds the micro-batch locally from the same rollout payload, so tensor shapes are known
without a shape exchange even though sequence lengths vary per micro-batch. Send/recv pairs
are issued with ``batch_isend_irecv`` on the pipeline group.

Two schedules:
  * one chunk per rank: non-interleaved 1F1B (warm-up forwards, steady 1F1B pairs, cool-down backwards);
  * ``vpp`` chunks per rank (virtual pipeline): chunk ``v`` of rank ``r`` is virtual stage ``v * pp + r``, so an
    activation visits every rank once per chunk and wraps from the last rank back to the first. Micro-batches are
    processed in groups of ``pp``: all forwards of a group in (chunk, micro-batch) order, then all backwards with the
    chunks reversed. Every rank walks the same order, sends never block and receives are posted in the order the
    peer sends, so the dependencies form a DAG ordered by (chunk, micro-batch, rank).
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
    return get_batch(data_iterator, keys, getattr(args, "data_pad_size_multiplier", 128), device=model.device,
                     allgather_cp=getattr(args, "allgather_cp", False))


def _run_interleaved(model, data_iterator, num_microbatches: int, forward_step, args, forward_only: bool) -> list[dict]:
    """Virtual-pipeline schedule (see the module docstring). Returns the last virtual stage's per-micro-batch results."""
    pp, rank = mpu.get_pipeline_model_parallel_world_size(), mpu.get_pipeline_model_parallel_rank()
    vpp = len(model.chunks)
    group = mpu.get_pipeline_model_parallel_group()
    prev_r, next_r = mpu.get_pipeline_model_parallel_prev_rank(), mpu.get_pipeline_model_parallel_next_rank()
    dtype = model.chunks[0].dtype
    results: list[dict] = []
    sends = []
    for g0 in range(0, num_microbatches, pp):
        ms = list(range(g0, min(g0 + pp, num_microbatches)))
        batches = {m: _get_batch(model, data_iterator, args) for m in ms}
        saved = {}
        for v in range(vpp):
            for m in ms:
                first_v, last_v = rank == 0 and v == 0, rank == pp - 1 and v == vpp - 1
                inp = None
                if not first_v:
                    inp = torch.empty(_shape_for(batches[m], model, args), dtype=dtype, device=model.device)
                    dist.recv(inp, src=prev_r, group=group)
                    inp.requires_grad_(not forward_only)
                out, res = forward_step(batches[m], model.chunks[v], inp)
                if last_v:
                    results.append(res)
                else:
                    sends.append(dist.isend(out.detach().contiguous(), next_r, group=group))
                if not forward_only:
                    saved[(m, v)] = (inp, out)
        if not forward_only:
            for v in reversed(range(vpp)):
                for m in ms:
                    first_v, last_v = rank == 0 and v == 0, rank == pp - 1 and v == vpp - 1
                    inp, out = saved.pop((m, v))
                    if last_v:
                        out.backward()
                    else:
                        g = torch.empty_like(out)
                        dist.recv(g, src=next_r, group=group)
                        torch.autograd.backward(out, grad_tensors=g)
                    if not first_v:
                        sends.append(dist.isend(inp.grad.contiguous(), prev_r, group=group))
        for w in sends:
            w.wait()
        sends = []
    return results


def run_forward_only(model, data_iterator, num_microbatches: int, forward_step, args) -> list[dict]:
    pp = mpu.get_pipeline_model_parallel_world_size()
    if pp > 1 and len(model.chunks) > 1:
        return _run_interleaved(model, data_iterator, num_microbatches, forward_step, args, forward_only=True)
    first, last = mpu.is_pipeline_first_stage(), mpu.is_pipeline_last_stage()
    results = []
    dtype = model.chunks[0].dtype
    for _ in range(num_microbatches):
        batch = _get_batch(model, data_iterator, args)
        x = None
        if pp > 1 and not first:
            x, _ = _p2p(recv_prev_shape=_shape_for(batch, model, args), dtype=dtype, device=model.device)
        for chunk in model.chunks:  # pp == 1: the chunks of the one rank are consecutive layers
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
    if len(model.chunks) > 1:
        return _run_interleaved(model, data_iterator, num_microbatches, forward_step, args, forward_only=False)

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
        pending.append((inp, out, shape))
        grad_out = None
        if not last:
            # the gradient that comes back now is that of the oldest forward still pending, whose token count (dynamic
            # batching) generally differs from the micro-batch just sent
            _, grad_out = _p2p(send_next=out.detach(), recv_next_shape=pending[0][2], dtype=dtype, device=model.device)
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
