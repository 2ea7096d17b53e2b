"""Packed (varlen) causal attention for training, prefill and context parallelism.

CUDA path: the sm_100a flash-attention kernels of this package (``csrc/flash_fwd_sm100.cu``,
``csrc/flash_bwd_sm100.cu``: tcgen05 + TMEM + TMA, head dims 64 and 128). CPU path: per-segment fp32 reference.
No library attention is called.

Work is described by SEGMENTS ``[nseg, 4] = (q_off, q_len, k_off, k_len)``: rows ``[q_off, q_off + q_len)`` of Q
attend rows ``[k_off, k_off + k_len)`` of K / V, causally aligned at the end (query ``i`` sees keys
``j <= (k_len - q_len) + i``). A packed training batch is one segment per sequence with ``q_off == k_off``; a prefill
over a cached prefix has ``k_len > q_len``; a context-parallel rank passes each local query chunk against a prefix of
the gathered keys. In the backward every key tile of a segment has one owner, so the key ranges of the segments of
one call must not overlap (query ranges never do). Replaces the flash-attn / TE attention calls of the reference
(slime_plugins/models/flash_dot_product_attention.py:25-80).
"""

from __future__ import annotations

import math

import torch

from slime_b200.ops import reference


def segments_from_cu_seqlens(cu_seqlens: torch.Tensor) -> torch.Tensor:
    """One self-attention segment per packed sequence (device op, no host sync)."""
    cu = cu_seqlens.to(torch.int32)
    off, ln = cu[:-1], cu[1:] - cu[:-1]
    return torch.stack([off, ln, off, ln], dim=1).contiguous()


def segments_extend(cu_q: torch.Tensor, cu_k: torch.Tensor) -> torch.Tensor:
    """New tokens (``cu_q``) attending cached + new context (``cu_k``), per request."""
    cq, ck = cu_q.to(torch.int32), cu_k.to(torch.int32)
    return torch.stack([cq[:-1], cq[1:] - cq[:-1], ck[:-1], ck[1:] - ck[:-1]], dim=1).contiguous()


def _reference_segments(q, k, v, seg, scale, sinks=None):
    """fp32 oracle / CPU path: q [Tq, Hq, D], k / v [Tk, Hkv, D]; rows outside every segment come out as zeros.
    ``sinks`` [Hq]: one extra logit per head that takes part in the softmax and contributes no value."""
    Hq, Hkv = q.shape[1], k.shape[1]
    out = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    pieces = []
    for q_off, q_len, k_off, k_len in seg.tolist():
        if q_len <= 0:
            continue
        qs = q[q_off : q_off + q_len].float().transpose(0, 1)
        ks = k[k_off : k_off + k_len].float().transpose(0, 1).repeat_interleave(Hq // Hkv, 0)
        vs = v[k_off : k_off + k_len].float().transpose(0, 1).repeat_interleave(Hq // Hkv, 0)
        att = (qs @ ks.transpose(-1, -2)) * scale
        mask = torch.ones(q_len, k_len, dtype=torch.bool, device=q.device).tril(diagonal=k_len - q_len)
        att = att.masked_fill(~mask, float("-inf"))
        if sinks is not None:
            col = sinks.float().view(Hq, 1, 1).expand(Hq, q_len, 1)
            o = torch.cat([att, col], -1).softmax(-1)[..., :-1] @ vs
        else:
            o = att.softmax(-1) @ vs
        pieces.append((q_off, q_len, o.transpose(0, 1)))
    for q_off, q_len, o in pieces:  # out-of-place assembly keeps autograd happy
        pad = torch.zeros_like(out)
        pad[q_off : q_off + q_len] = o
        out = out + pad
    return out.to(q.dtype)


def _strides_ok(t: torch.Tensor) -> bool:
    return t.stride(-1) == 1 and t.stride(1) == t.shape[-1] and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


def flash_fwd(q, k, v, seg, scale, max_q_len_hint: int | None = None, out=None, zero_uncovered: bool = False):
    """Forward kernel launch. q [Tq, Hq, D] (heads contiguous inside a token row, any 16-byte-multiple row pitch),
    k / v [Tk, Hkv, D]. Returns ``(out [Tq, Hq, D], lse [Hq, Tq] fp32)``. The kernel writes the rows of ``out`` that
    lie inside a segment and no others; ``zero_uncovered`` starts from zeros for callers whose segments do not cover
    every row."""
    from slime_b200.ops import _lib

    Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[0], k.shape[1]
    assert D in (64, 128), f"flash attention kernels cover head dims 64 and 128, not {D}"
    q, k, v = (t if _strides_ok(t) else t.contiguous() for t in (q, k, v))
    if out is None:
        out = (torch.zeros if zero_uncovered else torch.empty)(Tq, Hq, D, dtype=q.dtype, device=q.device)
    lse = (torch.zeros if zero_uncovered else torch.empty)(Hq, Tq, dtype=torch.float32, device=q.device)
    nseg = seg.shape[0]
    max_q_tiles = -(-Tq // 128) + nseg
    fn = _lib.bind("sb_flash_fwd", [_lib.P] * 6 + [_lib.I] * 12 + [_lib.F, _lib.P, _lib.P])
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), seg.data_ptr(), nseg, max_q_tiles, Tq, Tk,
            Hq, Hkv, D, q.stride(0), k.stride(0), v.stride(0), out.stride(0), Tq, float(scale),
            _lib.ptr(_lib.status_word(q.device)), _lib.stream())  # fmt: skip
    _lib.check(rc, "sb_flash_fwd")
    return out, lse


def flash_bwd(q, k, v, o, d_o, lse, seg, scale, dq=None, dk=None, dv=None):
    """Backward kernel launches (delta, dK/dV pass, dQ pass). Gradient tensors may be views into one packed buffer.
    Rows outside every segment are zeroed here when the outputs are allocated here, else left to the caller."""
    from slime_b200.ops import _lib

    Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[0], k.shape[1]
    q, k, v, o, d_o = (t if _strides_ok(t) else t.contiguous() for t in (q, k, v, o, d_o))
    dq = torch.zeros_like(q) if dq is None else dq
    dk = torch.zeros(Tk, Hkv, D, dtype=k.dtype, device=k.device) if dk is None else dk
    dv = torch.zeros(Tk, Hkv, D, dtype=v.dtype, device=v.device) if dv is None else dv
    delta = torch.empty_like(lse)
    nseg = seg.shape[0]
    fn = _lib.bind("sb_flash_bwd", [_lib.P] * 11 + [_lib.I] * 17 + [_lib.F, _lib.P, _lib.P])
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr(), delta.data_ptr(),
            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), seg.data_ptr(), nseg, -(-Tq // 128) + nseg, -(-Tk // 128) + nseg, Tq, Tk,
            Hq, Hkv, D, q.stride(0), k.stride(0), v.stride(0), o.stride(0), d_o.stride(0), dq.stride(0), dk.stride(0),
            dv.stride(0), lse.stride(0), float(scale), _lib.ptr(_lib.status_word(q.device)), _lib.stream())  # fmt: skip
    _lib.check(rc, "sb_flash_bwd")
    return dq, dk, dv


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, seg, scale):
        out, lse = flash_fwd(q, k, v, seg, scale, zero_uncovered=True)
        ctx.save_for_backward(q, k, v, out, lse, seg)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, out, lse, seg = ctx.saved_tensors
        dq, dk, dv = flash_bwd(q, k, v, out, d_o, lse, seg, ctx.scale)
        return dq, dk, dv, None, None


class _SinkFlashAttention(torch.autograd.Function):
    """Attention with a learnable per-head sink logit ``b_h`` in the softmax denominator, on the plain flash kernels.

    With ``lse`` the log-sum-exp of the real scores, the sink turns the probabilities into ``sigmoid(lse - b) * P``,
    so the output is the plain output times ``g = sigmoid(lse - b)`` per (head, row). Backward: the score gradient
    is ``g P (dP - g (dO . O))``, which is what the plain backward computes when it is handed ``g dO`` for ``dO`` and
    ``g O`` for ``O`` (its row term is the dot product of the two); ``d b_h = -sum_rows (1 - g) (dO . g O)``.
    Same role as slime_plugins/models/learnable_softmax_attention.py:23 in the reference.
    """

    @staticmethod
    def forward(ctx, q, k, v, seg, scale, sinks):
        out, lse = flash_fwd(q, k, v, seg, scale, zero_uncovered=True)
        gate = torch.sigmoid(lse - sinks.float()[:, None])  # [Hq, Tq]
        out = (out.float() * gate.t()[:, :, None]).to(q.dtype)
        ctx.save_for_backward(q, k, v, out, lse, seg, gate)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, out, lse, seg, gate = ctx.saved_tensors
        gt = gate.t()[:, :, None]
        d_scaled = (d_o.float() * gt).to(d_o.dtype)
        dq, dk, dv = flash_bwd(q, k, v, out, d_scaled, lse, seg, ctx.scale)
        row = (d_o.float() * out.float()).sum(-1)  # [Tq, Hq] = dO . (g O)
        d_sinks = -((1.0 - gate.t()) * row).sum(0)
        return dq, dk, dv, None, None, d_sinks


def _library_segments(q, k, v, seg, scale):
    """Comparison arm only (``ops.library_mode()``): the flash-attn library on the same segments."""
    from flash_attn import flash_attn_varlen_func

    s = seg.to(torch.int32)
    zero = torch.zeros(1, dtype=torch.int32, device=seg.device)
    # the library wants cumulative offsets: segments are laid out back to back on both sides in every caller
    cu_q = torch.cat([s[:1, 0], s[:, 0] + s[:, 1]]).contiguous()
    cu_k = torch.cat([s[:1, 2], s[:, 2] + s[:, 3]]).contiguous()
    mq, mk = int(s[:, 1].max()), int(s[:, 3].max())
    return flash_attn_varlen_func(q, k, v, cu_q, cu_k, mq, mk, softmax_scale=scale, causal=True)


def segment_attention(q, k, v, seg, scale=None, sinks=None):
    """Causal GQA attention over a segment table. q: [Tq, Hq, D], k / v: [Tk, Hkv, D] -> [Tq, Hq, D]. ``sinks`` [Hq]
    (optional, learnable): a per-head logit added to every row's softmax denominator."""
    from slime_b200 import ops

    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    from slime_b200.ops import _checks

    _checks.segments("segment_attention", seg, q.shape[0], k.shape[0])
    if not q.is_cuda or q.shape[-1] not in (64, 128):
        # the flash kernels cover head dims 64 and 128; other widths (256 in Qwen3-Next / Qwen3.5) take the explicit form
        return _reference_segments(q, k, v, seg, scale, sinks)
    if sinks is not None:
        return _SinkFlashAttention.apply(q, k, v, seg, scale, sinks)
    if ops.library_mode():
        return _library_segments(q, k, v, seg, scale)
    return _FlashAttention.apply(q, k, v, seg, scale)


def varlen_attention(q, k, v, cu_seqlens, max_seqlen=None, scale=None, causal=True, sinks=None):
    """Packed causal self-attention (one segment per sequence)."""
    assert causal, "the attention kernels are causal"
    return segment_attention(q, k, v, segments_from_cu_seqlens(cu_seqlens), scale, sinks)


def extend_attention(q, k_all, v_all, cu_q, cu_k, scale=None):
    """New tokens over (cached prefix + new) keys, per request; ``k_all`` / ``v_all`` hold each request's full context
    contiguously (``cu_k``)."""
    return segment_attention(q, k_all, v_all, segments_extend(cu_q, cu_k), scale)


class _RopeAttentionCUDA(torch.autograd.Function):
    """(per-head RMSNorm +) RoPE + packed causal attention on a ``[T, (Hq + 2 Hkv) * D]`` qkv row, as one autograd
    node. q / k / v stay views of one buffer in both directions: there is no slice-backward zero-fill and no
    concatenation of dq | dk | dv; the backward kernels write straight into one packed ``dqkv`` and the inverse rotation
    runs on it in place. Without qk-norm the forward rotation is in place on the projection output as well."""

    @staticmethod
    def forward(ctx, qkv, positions, cos_sin, q_norm_w, k_norm_w, seg, Hq, Hkv, D, eps, scale):
        from slime_b200.ops import _rope_launch

        T = qkv.shape[0]
        qkv = qkv.contiguous()
        has_norm = q_norm_w is not None
        rot = torch.empty_like(qkv) if has_norm else qkv
        _rope_launch(qkv, rot, positions, cos_sin, q_norm_w, None, Hq, 0, D, eps, 1.0)
        _rope_launch(qkv, rot, positions, cos_sin, k_norm_w, None, Hkv, Hq, D, eps, 1.0)
        r3, x3 = rot.view(T, Hq + 2 * Hkv, D), qkv.view(T, Hq + 2 * Hkv, D)
        q, k, v = r3[:, :Hq], r3[:, Hq : Hq + Hkv], x3[:, Hq + Hkv :]  # v is never rotated: read it where it is
        out, lse = flash_fwd(q, k, v, seg, scale)
        ctx.save_for_backward(qkv, rot if has_norm else None, out, lse, seg, positions, cos_sin, q_norm_w, k_norm_w)
        ctx.dims = (Hq, Hkv, D, eps, scale)
        return out.view(T, Hq * D)

    @staticmethod
    def backward(ctx, dout):
        from slime_b200.ops import _head_norm_bwd, _rope_launch

        qkv, rot, out, lse, seg, positions, cos_sin, q_norm_w, k_norm_w = ctx.saved_tensors
        Hq, Hkv, D, eps, scale = ctx.dims
        T = qkv.shape[0]
        has_norm = rot is not None
        r3 = (rot if has_norm else qkv).view(T, Hq + 2 * Hkv, D)
        x3 = qkv.view(T, Hq + 2 * Hkv, D)
        dqkv = torch.zeros_like(qkv)  # rows outside every segment (padding) carry no gradient
        d3 = dqkv.view(T, Hq + 2 * Hkv, D)
        flash_bwd(r3[:, :Hq], r3[:, Hq : Hq + Hkv], x3[:, Hq + Hkv :], out, dout.reshape(T, Hq, D), lse, seg, scale,
                  dq=d3[:, :Hq], dk=d3[:, Hq : Hq + Hkv], dv=d3[:, Hq + Hkv :])  # fmt: skip
        _rope_launch(dqkv, dqkv, positions, cos_sin, None, None, Hq + Hkv, 0, D, eps, -1.0)  # inverse rotation, in place
        dqw = dkw = None
        if has_norm:
            dq, dqw = _head_norm_bwd(x3[:, :Hq], d3[:, :Hq], q_norm_w, eps)
            dk, dkw = _head_norm_bwd(x3[:, Hq : Hq + Hkv], d3[:, Hq : Hq + Hkv], k_norm_w, eps)
            d3[:, :Hq].copy_(dq)
            d3[:, Hq : Hq + Hkv].copy_(dk)
        return dqkv, None, None, dqw, dkw, None, None, None, None, None, None


class _AllGatherRows(torch.autograd.Function):
    """[T, ...] on every rank -> [n * T, ...] (rank-major). Backward: reduce-scatter of the gradient (sum)."""

    @staticmethod
    def forward(ctx, x, group):
        import torch.distributed as dist

        ctx.group, ctx.n = group, dist.get_world_size(group)
        out = torch.empty((ctx.n * x.shape[0], *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist

        out = torch.empty((g.shape[0] // ctx.n, *g.shape[1:]), dtype=g.dtype, device=g.device)
        dist.reduce_scatter_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


def context_parallel_plan(local_cu_seqlens: torch.Tensor, cp: int, rank: int, num_local_tokens: int):
    """Index plan of zig-zag context parallelism for one packed micro-batch (device ops only).

    Every sequence is cut into ``2 * cp`` chunks of ``cs`` tokens; rank ``r`` holds chunks ``r`` and ``2cp-1-r``
    back to back, so its local piece of a sequence has ``2 * cs`` tokens (``local_cu_seqlens``). Returns
    ``(perm, seg)``: ``perm`` reorders the rank-major all-gather of the local K / V rows into global token order per
    sequence (sequence ``i`` then occupies rows ``[cp * o_i, cp * (o_i + 2 cs_i))``), and ``seg`` holds two segments per
    sequence: the local chunk ``r`` against global chunks ``0..r`` and the local chunk ``2cp-1-r`` against ``0..2cp-1-r``.
    """
    cu = local_cu_seqlens.to(torch.int64)
    dev = cu.device
    o, ln = cu[:-1], cu[1:] - cu[:-1]
    cs = ln // 2  # every local piece (the padding tail included) has an even number of tokens
    # destination row (global order) of gathered row (r', t)
    t = torch.arange(num_local_tokens, device=dev)
    i = torch.searchsorted(cu, t, right=True) - 1
    u = t - o[i]
    second = u >= cs[i]
    inner = torch.where(second, u - cs[i], u)
    dst_rows = []
    for r2 in range(cp):
        g = torch.where(second, torch.full_like(u, 2 * cp - 1 - r2), torch.full_like(u, r2))
        dst_rows.append(cp * o[i] + g * cs[i] + inner)
    dst = torch.cat(dst_rows)  # gathered row -> global row
    perm = torch.empty_like(dst)
    perm[dst] = torch.arange(dst.numel(), device=dev)  # global row -> gathered row
    a = torch.stack([o, cs, cp * o, (rank + 1) * cs], dim=1)
    b = torch.stack([o + cs, cs, cp * o, (2 * cp - rank) * cs], dim=1)
    seg = torch.cat([a, b], dim=0).to(torch.int32).contiguous()
    return perm, seg


def context_parallel_attention(q, k, v, local_cu_seqlens, cp_group, scale=None):
    """Zig-zag context-parallel causal attention: K / V are all-gathered over the context-parallel group (their
    gradients reduce-scattered back), put in global order, and every local query chunk attends its causal prefix through
    the segment kernels. Numerically the same attention as ring exchange (cp_comm_type "p2p" in the reference,
    slime_plugins/models/flash_dot_product_attention.py:42; zig-zag layout slime/backends/megatron_utils/cp_utils.py:179-209).
    """
    import torch.distributed as dist

    cp, rank = dist.get_world_size(cp_group), dist.get_rank(cp_group)
    perm, seg = context_parallel_plan(local_cu_seqlens, cp, rank, k.shape[0])
    kg = _AllGatherRows.apply(k, cp_group).index_select(0, perm)
    vg = _AllGatherRows.apply(v, cp_group).index_select(0, perm)
    # The two chunks of a sequence read overlapping key ranges, and the backward kernels give every key tile of a
    # segment one owner: segments of one call must not share keys. One call per chunk; autograd adds the two dK / dV.
    n = seg.shape[0] // 2
    return segment_attention(q, kg, vg, seg[:n].contiguous(), scale) + segment_attention(q, kg, vg, seg[n:].contiguous(), scale)


def rope_attention(qkv, positions, cos_sin, cu_seqlens, max_seqlen, Hq, Hkv, D, q_norm_w=None, k_norm_w=None, eps=1e-6,
                   scale=None, cp_local_cu_seqlens=None, cp_group=None):
    """Rotary embedding (with optional per-head q/k RMSNorm) followed by packed causal GQA attention.
    ``qkv``: [T, (Hq + 2 Hkv) * D] as produced by the fused qkv projection; returns [T, Hq * D]. With a
    context-parallel group, ``qkv`` holds this rank's zig-zag chunks (``cp_local_cu_seqlens``) and ``positions`` their
    global positions."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if cp_group is not None:
        from slime_b200.ops import rope_qk

        T = qkv.shape[0]
        q3 = rope_qk(qkv, positions, cos_sin, Hq, Hkv, D, q_norm_w, k_norm_w, eps).view(T, Hq + 2 * Hkv, D)
        ctx = context_parallel_attention(q3[:, :Hq], q3[:, Hq : Hq + Hkv], q3[:, Hq + Hkv :], cp_local_cu_seqlens, cp_group, scale)
        return ctx.reshape(T, Hq * D)
    seg = segments_from_cu_seqlens(cu_seqlens)
    from slime_b200 import ops as _ops

    if qkv.is_cuda and not _ops.library_mode():
        return _RopeAttentionCUDA.apply(qkv, positions, cos_sin, q_norm_w, k_norm_w, seg, Hq, Hkv, D, eps, scale)
    from slime_b200.ops import rope_qk

    T = qkv.shape[0]
    q3 = rope_qk(qkv, positions, cos_sin, Hq, Hkv, D, q_norm_w, k_norm_w, eps).view(T, Hq + 2 * Hkv, D)
    ctx = segment_attention(q3[:, :Hq], q3[:, Hq : Hq + Hkv], q3[:, Hq + Hkv :], seg, scale)
    return ctx.reshape(T, Hq * D)
