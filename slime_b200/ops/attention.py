"""Packed (varlen) causal attention for training and prefill.

CUDA path: the sm_100a flash-attention kernels of this package when built
(``sb_flash_fwd`` / ``sb_flash_bwd``), else the flash-attn library kernels (a
plain library call, reported as such by the bench). CPU path: per-sequence fp32
reference.
"""

from __future__ import annotations

import math

import torch

from slime_b200.ops import reference


def _library_varlen(q, k, v, cu_seqlens, max_seqlen, scale, causal):
    from flash_attn import flash_attn_varlen_func

    cu = cu_seqlens.to(torch.int32)
    return flash_attn_varlen_func(q, k, v, cu, cu, max_seqlen, max_seqlen, softmax_scale=scale, causal=causal)


class _RefAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, scale, causal):
        ctx.save_for_backward(q, k, v, cu_seqlens)
        ctx.scale, ctx.causal = scale, causal
        return reference.varlen_attention(q, k, v, cu_seqlens, scale, causal)

    @staticmethod
    def backward(ctx, do):
        q, k, v, cu = ctx.saved_tensors
        with torch.enable_grad():
            qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
            out = reference.varlen_attention(qf, kf, vf, cu, ctx.scale, ctx.causal)
            gq, gk, gv = torch.autograd.grad(out, (qf, kf, vf), do.float())
        return gq.to(q.dtype), gk.to(k.dtype), gv.to(v.dtype), None, None, None


def varlen_attention(q, k, v, cu_seqlens, max_seqlen, scale=None, causal=True):
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if not q.is_cuda:
        return _RefAttention.apply(q, k, v, cu_seqlens, scale, causal)
    return _library_varlen(q, k, v, cu_seqlens, max_seqlen, scale, causal)
