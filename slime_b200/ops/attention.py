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


class _RopeAttentionCUDA(torch.autograd.Function):
    """(per-head RMSNorm +) RoPE + packed causal attention on a ``[T, (Hq + 2 Hkv) * D]`` qkv row, as one autograd
    node. What this buys over separate nodes is memory traffic, not math: q/k/v stay views of one buffer in both
    directions, so there is no slice-backward zero-fill and no concatenation of dq | dk | dv; the backward kernels
    write straight into one packed ``dqkv`` and the inverse rotation runs on it in place. Without qk-norm the forward
    rotation is in place on the projection output as well (nothing upstream needs the unrotated values)."""

    @staticmethod
    def forward(ctx, qkv, positions, cos_sin, q_norm_w, k_norm_w, cu_seqlens, max_seqlen, Hq, Hkv, D, eps, scale):
        from flash_attn.flash_attn_interface import _flash_attn_varlen_forward

        from slime_b200.ops import _rope_launch

        T = qkv.shape[0]
        qkv = qkv.contiguous()
        has_norm = q_norm_w is not None
        rot = torch.empty_like(qkv) if has_norm else qkv
        _rope_launch(qkv, rot, positions, cos_sin, q_norm_w, None, Hq, 0, D, eps, 1.0)
        _rope_launch(qkv, rot, positions, cos_sin, k_norm_w, None, Hkv, Hq, D, eps, 1.0)
        r3, x3 = rot.view(T, Hq + 2 * Hkv, D), qkv.view(T, Hq + 2 * Hkv, D)
        q, k, v = r3[:, :Hq], r3[:, Hq : Hq + Hkv], x3[:, Hq + Hkv :]  # v is never rotated: read it where it is
        cu = cu_seqlens.to(torch.int32)
        out, lse, _, rng = _flash_attn_varlen_forward(q, k, v, cu, cu, max_seqlen, max_seqlen, 0.0, scale, causal=True)
        ctx.save_for_backward(qkv, rot if has_norm else None, out, lse, cu, positions, cos_sin, q_norm_w, k_norm_w, rng)
        ctx.dims = (Hq, Hkv, D, eps, scale, max_seqlen)
        return out.view(T, Hq * D)

    @staticmethod
    def backward(ctx, dout):
        from flash_attn.flash_attn_interface import _flash_attn_varlen_backward

        from slime_b200.ops import _head_norm_bwd, _rope_launch

        qkv, rot, out, lse, cu, positions, cos_sin, q_norm_w, k_norm_w, rng = ctx.saved_tensors
        Hq, Hkv, D, eps, scale, max_seqlen = ctx.dims
        T = qkv.shape[0]
        has_norm = rot is not None
        r3 = (rot if has_norm else qkv).view(T, Hq + 2 * Hkv, D)
        x3 = qkv.view(T, Hq + 2 * Hkv, D)
        dqkv = torch.empty_like(qkv)
        d3 = dqkv.view(T, Hq + 2 * Hkv, D)
        _flash_attn_varlen_backward(dout.reshape(T, Hq, D), r3[:, :Hq], r3[:, Hq : Hq + Hkv], x3[:, Hq + Hkv :], out, lse,
                                    d3[:, :Hq], d3[:, Hq : Hq + Hkv], d3[:, Hq + Hkv :], cu, cu, max_seqlen, max_seqlen, 0.0,
                                    scale, True, -1, -1, 0.0, None, False, rng)  # fmt: skip
        _rope_launch(dqkv, dqkv, positions, cos_sin, None, None, Hq + Hkv, 0, D, eps, -1.0)  # inverse rotation, in place
        dqw = dkw = None
        if has_norm:
            dq, dqw = _head_norm_bwd(x3[:, :Hq], d3[:, :Hq], q_norm_w, eps)
            dk, dkw = _head_norm_bwd(x3[:, Hq : Hq + Hkv], d3[:, Hq : Hq + Hkv], k_norm_w, eps)
            d3[:, :Hq].copy_(dq)
            d3[:, Hq : Hq + Hkv].copy_(dk)
        return dqkv, None, None, dqw, dkw, None, None, None, None, None, None, None


def rope_attention(qkv, positions, cos_sin, cu_seqlens, max_seqlen, Hq, Hkv, D, q_norm_w=None, k_norm_w=None, eps=1e-6,
                   scale=None):
    """Rotary embedding (with optional per-head q/k RMSNorm) followed by packed causal GQA attention.
    ``qkv``: [T, (Hq + 2 Hkv) * D] as produced by the fused qkv projection; returns [T, Hq * D]."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if qkv.is_cuda:
        return _RopeAttentionCUDA.apply(qkv, positions, cos_sin, q_norm_w, k_norm_w, cu_seqlens, max_seqlen, Hq, Hkv, D, eps,
                                        scale)
    from slime_b200.ops import rope_qk

    T = qkv.shape[0]
    q3 = rope_qk(qkv, positions, cos_sin, Hq, Hkv, D, q_norm_w, k_norm_w, eps).view(T, Hq + 2 * Hkv, D)
    ctx = varlen_attention(q3[:, :Hq], q3[:, Hq : Hq + Hkv], q3[:, Hq + Hkv :], cu_seqlens, max_seqlen, scale)
    return ctx.reshape(T, Hq * D)
