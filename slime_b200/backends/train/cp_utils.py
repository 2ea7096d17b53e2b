"""Context-parallel (zig-zag ring) bookkeeping for losses and metrics.

A sample of ``total_length`` tokens is cut into ``2*cp`` equal chunks; CP rank
``r`` holds chunks ``r`` and ``2cp-1-r`` so causal-attention work is balanced.
``ZigZag`` describes, for one sample and this rank, which logits rows / tokens /
response positions are local. Every reducer then works on local pieces with
*global* per-sample denominators, and whole-sequence quantities are rebuilt with a
differentiable all-reduce of response-length vectors only.
Parity: slime/backends/megatron_utils/cp_utils.py:9-236.
"""

from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from slime_b200.parallel import state as mpu


@dataclass
class ZigZag:
    chunk_size: int
    chunks: tuple[tuple[int, int], tuple[int, int]]  # token ranges of the two local chunks (global positions)
    logits: tuple[tuple[int, int], tuple[int, int]]  # positions whose *next-token* logits are local and in the response
    tokens: tuple[tuple[int, int], tuple[int, int]]  # the predicted tokens = logits + 1
    prompt_length: int
    total_length: int

    @staticmethod
    def plan(total_length: int, response_length: int, cp_rank: int | None = None, cp_size: int | None = None) -> "ZigZag":
        r = mpu.get_context_parallel_rank() if cp_rank is None else cp_rank
        n = mpu.get_context_parallel_world_size() if cp_size is None else cp_size
        prompt = total_length - response_length
        cs = -(-total_length // (2 * n))
        c0 = (r * cs, (r + 1) * cs)
        c1 = ((2 * n - r - 1) * cs, (2 * n - r) * cs)

        def clip(c):
            lo, hi = max(c[0], prompt - 1), min(c[1], total_length - 1)
            return ((lo, hi), (lo + 1, hi + 1)) if lo < hi else ((0, 0), (0, 0))

        (l0, t0), (l1, t1) = clip(c0), clip(c1)
        return ZigZag(cs, (c0, c1), (l0, l1), (t0, t1), prompt, total_length)

    # response-relative slices (index 0 = first response token's logprob)
    def response_slices(self):
        base = self.prompt_length - 1
        return tuple(slice(a - base, b - base) for a, b in self.logits)

    def local_response_len(self) -> int:
        return sum(b - a for a, b in self.logits)


def get_logits_and_tokens_offset_with_cp(total_length: int, response_length: int):
    """Tuple form ``(chunk_size, chunks, logits_offsets, token_offsets)``; all offsets from the prompt start."""
    assert mpu.get_context_parallel_world_size() > 1
    z = ZigZag.plan(total_length, response_length)
    return z.chunk_size, z.chunks, z.logits, z.tokens


def local_loss_masks(total_lengths, response_lengths, loss_masks):
    """Per-sample loss masks restricted to the response positions this CP rank holds."""
    if mpu.get_context_parallel_world_size() == 1:
        return list(loss_masks), list(response_lengths)
    out, lens = [], []
    for tl, rl, m in zip(total_lengths, response_lengths, loss_masks):
        s0, s1 = ZigZag.plan(tl, rl).response_slices()
        piece = torch.cat([m[s0], m[s1]], dim=0)
        out.append(piece)
        lens.append(piece.numel())
    return out, lens


def get_sum_of_sample_mean(
    total_lengths: list[int],
    response_lengths: list[int],
    loss_masks: list[torch.Tensor],
    sample_denoms: list[torch.Tensor] | torch.Tensor | None = None,
    calculate_per_token_loss: bool = False,
) -> Callable[[torch.Tensor], torch.Tensor]:
    """Reducer over a concatenated per-token tensor.

    Default: sum over samples of (masked sum / that sample's *global* mask total). With
    ``sample_denoms`` every sample of a rollout carries the rollout's total mask count
    (per-rollout token-weighted mean). ``calculate_per_token_loss``: plain masked sum.
    CP-safe: numerators are local, denominators global.
    """
    masks, lens = local_loss_masks(total_lengths, response_lengths, loss_masks)
    n = len(lens)
    if n == 0:
        return lambda x: x.new_zeros(())
    # One concatenated mask and one segment-id vector for the whole micro-batch: the reduction is a masked
    # multiply, one index_add over samples and one divide, instead of a few kernels per sample.
    dev = masks[0].device
    mask_cat = torch.cat([m.reshape(-1) for m in masks]).to(torch.float32)
    seg = torch.repeat_interleave(torch.arange(n, device=dev), torch.as_tensor(lens, device=dev), output_size=sum(lens))
    if calculate_per_token_loss:
        denoms = None
    elif sample_denoms is None:
        if mpu.get_context_parallel_world_size() == 1:
            denoms = torch.zeros(n, dtype=torch.float32, device=dev).index_add_(0, seg, mask_cat)
        else:  # denominators are global (whole-sample) mask totals, numerators local to this CP rank
            denoms = torch.stack([m.sum() for m in loss_masks]).to(torch.float32)
    elif torch.is_tensor(sample_denoms):
        denoms = sample_denoms.to(torch.float32).reshape(-1)
    else:
        denoms = torch.stack([torch.as_tensor(d, dtype=torch.float32, device=dev).reshape(()) for d in sample_denoms])
    if denoms is not None:
        denoms = torch.clamp_min(denoms, 1)

    def per_sample(x: torch.Tensor) -> torch.Tensor:
        sums = torch.zeros(n, dtype=x.dtype, device=x.device).index_add(0, seg, x * mask_cat.to(x.dtype))
        return (sums / denoms.to(x.dtype)).sum()

    def per_token(x: torch.Tensor) -> torch.Tensor:
        return (x * mask_cat.to(x.dtype)).sum()

    return per_token if calculate_per_token_loss else per_sample


class _AllReduceSum(torch.autograd.Function):
    """Sum over the group forward; gradient passes through unchanged to every rank's contribution
    (each rank contributed a disjoint slice, the rest of its vector was zeros)."""

    @staticmethod
    def forward(ctx, x, group):
        out = x.clone()
        dist.all_reduce(out, group=group)
        ctx.group = group
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def all_gather_with_cp(tensor: torch.Tensor, total_length: int, response_length: int) -> torch.Tensor:
    """Rebuild a full ``[response_length, ...]`` tensor from CP-local pieces (differentiable)."""
    n = mpu.get_context_parallel_world_size()
    if n == 1:
        return tensor
    z = ZigZag.plan(total_length, response_length)
    s0, s1 = z.response_slices()
    n0 = s0.stop - s0.start
    full = tensor.new_zeros((response_length, *tensor.shape[1:]))
    pieces = []
    cursor = 0
    # assemble with cat so autograd tracks the local pieces
    for sl, piece in ((s0, tensor[:n0]), (s1, tensor[n0:])):
        if sl.stop - sl.start == 0:
            continue
        pieces.append(full[cursor : sl.start])
        pieces.append(piece)
        cursor = sl.stop
    pieces.append(full[cursor:])
    assembled = torch.cat(pieces, dim=0)
    assert assembled.shape[0] == response_length, f"Expected {response_length}, got {assembled.shape}"
    return _AllReduceSum.apply(assembled, mpu.get_context_parallel_group())


def slice_with_cp(tokens: torch.Tensor, pad_value) -> torch.Tensor:
    """This rank's two zig-zag chunks of a per-token tensor (padded to ``2*cp*chunk``)."""
    n, r = mpu.get_context_parallel_world_size(), mpu.get_context_parallel_rank()
    if n == 1:
        return tokens
    L = len(tokens)
    cs = -(-L // (2 * n))
    pad = 2 * n * cs - L
    if callable(pad_value):
        tokens = pad_value(tokens, pad)
    else:
        tokens = F.pad(tokens, (0, 0) * (tokens.dim() - 1) + (0, pad), value=pad_value)
    return torch.cat([tokens[r * cs : (r + 1) * cs], tokens[(2 * n - r - 1) * cs : (2 * n - r) * cs]])


def slice_log_prob_with_cp(log_prob, total_length: int, response_length: int):
    """Keep the response positions this CP rank holds (inverse of :func:`all_gather_with_cp`)."""
    assert len(log_prob) == response_length, (
        f"log_prob length mismatch: len(log_prob)={len(log_prob)}, response_length={response_length}, "
        f"total_length={total_length}"
    )
    if mpu.get_context_parallel_world_size() == 1:
        return log_prob
    s0, s1 = ZigZag.plan(total_length, response_length).response_slices()
    a, b = log_prob[s0], log_prob[s1]
    return a + b if isinstance(log_prob, list) else torch.cat([a, b], dim=0)


def prepare_routed_experts_for_routing_replay(routed: torch.Tensor, total_length: int, pad_to: int | None = None):
    """Align rollout-recorded experts ``[tokens-1, layers, k]`` with this rank's token rows
    (the last token has no routing: repeat the final row), then CP-slice like the tokens."""
    if routed.shape[0] == total_length - 1:
        routed = torch.cat([routed, routed[-1:]], dim=0)
    routed = slice_with_cp(routed, 0)
    if pad_to is not None and routed.shape[0] < pad_to:
        routed = F.pad(routed, (0, 0, 0, 0, 0, pad_to - routed.shape[0]))
    return routed
