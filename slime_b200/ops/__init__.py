"""Fused ops of the training backend and rollout engine.

CUDA tensors run the hand-written sm_100a kernels (``csrc/*.cu`` through
``_lib``); CPU tensors run the PyTorch definitions in ``reference``. There is no
silent GPU fallback: a CUDA tensor without the built library raises.
"""

from __future__ import annotations

import math
import os

import torch

from slime_b200.ops import _checks, _lib, reference

P = _lib.ptr

# Comparison arm (``bench.py --impl library``): GEMMs go to cuBLAS through torch.matmul, training / prefill attention to
# the flash-attn library, RMSNorm / RoPE / SwiGLU / embedding to eager PyTorch, the fused loss and the peer-memory
# collectives are switched off by their own modules (NCCL runs instead). Explanatory only: it shows what the kernels of
# this package buy on the same box; it is not the reference framework.
LIBRARY_MODE = os.environ.get("SLIME_B200_LIBRARY_OPS") == "1"


def _is_cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


def library_mode() -> bool:
    return LIBRARY_MODE


def _cuda(t: torch.Tensor) -> bool:
    return t.is_cuda and not LIBRARY_MODE


def _library_gemm(a, b, a_mn, b_mn, bias, out, out_dtype, accumulate):
    A = a.t() if a_mn else a
    B = b if b_mn else b.t()
    if A.dtype != B.dtype:
        A = A.to(B.dtype)
    if out_dtype == torch.float32:
        try:
            res = torch.mm(A, B, out_dtype=torch.float32)
        except TypeError:
            res = torch.mm(A, B).float()
    else:
        res = torch.mm(A, B)
    if bias is not None:
        res = res + bias.to(res.dtype)
    if out is None:
        return res
    if accumulate:
        out.add_(res)
    else:
        out.copy_(res)
    return out


# ------------------------------------------------------------------------ GEMM
def _pick_bn(M: int, N: int, sms: int = 148) -> int:
    """Tile width by a wave model: time ~ waves x tile width / MMA efficiency (a 128-wide tile runs the tensor
    pipe at ~0.7 of a 256-wide one), waves = ceil(tiles / SMs)."""
    tiles_m = -(-M // 128)
    cost128 = -(-(tiles_m * -(-N // 128)) // sms) * 128 / 0.7
    cost256 = -(-(tiles_m * -(-N // 256)) // sms) * 256
    return 256 if cost256 <= cost128 else 128


BATCH_INVARIANT = False


def set_batch_invariant(on: bool = True):
    """A row's result must not depend on what else is in the batch (``--sglang-enable-deterministic-inference``): no
    split-K (its slices are summed by reduce-adds in arrival order, and the slice count follows the row count) and a
    decode-attention split count that follows the cache geometry only. Tile widths still follow the shape: every output
    element accumulates its K blocks in the same order whatever the tile. Same purpose as the batch-invariant operators
    of docker/patch/latest/sglang-deterministic.patch:276-375 in the reference."""
    global BATCH_INVARIANT
    BATCH_INVARIANT = bool(on)


def _pick_splitk(M: int, N: int, K: int, bn: int, sms: int = 148) -> int:
    """K slices for a GEMM whose output tiles cannot fill the machine (small weight gradients over many tokens,
    skinny decode projections with a long K): enough slices to occupy the SMs, at least 8 k-blocks of 64 each."""
    if BATCH_INVARIANT:
        return 1
    tiles = -(-M // 128) * -(-N // bn)
    kb = -(-K // 64)
    if tiles * 2 > sms or kb < 16:
        return 1
    return max(1, min(kb // 8, sms // tiles))


def gemm(a, b, *, a_mn=False, b_mn=False, bias=None, out=None, out_dtype=None, accumulate=False, bn=None, splitk=None):
    """``out (+)= op(A) @ op(B)^T (+ bias)`` with fp32 accumulation on the tcgen05 tensor cores.

    ``a``: [M, K] row-major, or [K, M] when ``a_mn``; ``b``: [N, K] row-major, or [K, N]
    when ``b_mn``. bf16 inputs; ``out`` bf16 or fp32 ([M, N], may be a strided row view).
    ``splitk``: K slices summed by TMA reduce-add into an fp32 ``out`` (None = choose; used only when the output
    is fp32 and either accumulated into or allocated here, where zero-filling it is free to arrange).
    """
    M, K = (a.shape[1], a.shape[0]) if a_mn else a.shape
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else b.shape
    assert K == Kb, f"inner dims differ: {K} vs {Kb}"
    out_dtype = out.dtype if out is not None else (out_dtype or a.dtype)
    if LIBRARY_MODE and a.is_cuda:
        return _library_gemm(a, b, a_mn, b_mn, bias, out, out_dtype, accumulate)
    if not _cuda(a):
        res = reference.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, out_dtype=torch.float32)
        if out is None:
            return res.to(out_dtype)
        if accumulate:
            out.add_(res.to(out.dtype))
        else:
            out.copy_(res.to(out.dtype))
        return out
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "sm_100a GEMM takes bf16 operands"
    assert out_dtype in (torch.bfloat16, torch.float32)
    if a.stride(-1) != 1:
        a = a.contiguous()
    if b.stride(-1) != 1:
        b = b.contiguous()
    bn = bn or _pick_bn(M, N)
    can_split = out_dtype == torch.float32 and (accumulate or out is None)
    if splitk is None:
        splitk = _pick_splitk(M, N, K, bn, _lib.sm_count(a.device)) if can_split else 1
    if out is None:
        assert not accumulate
        out = (torch.zeros if splitk > 1 else torch.empty)(M, N, dtype=out_dtype, device=a.device)
    assert out.stride(-1) == 1 and out.shape == (M, N)
    assert not (accumulate and out.dtype != torch.float32), "accumulate needs an fp32 output"
    assert splitk == 1 or out.dtype == torch.float32, "split-K sums fp32 partial products: the output must be fp32"
    lda, ldb, ldc = a.stride(0), b.stride(0), out.stride(0)
    assert lda % 8 == 0 and ldb % 8 == 0, "TMA needs 16-byte row pitches (multiples of 8 bf16)"
    if splitk > 1 and (out.data_ptr() % 16 or (ldc * 4) % 16):
        if not accumulate:
            raise ValueError("split-K needs a 16-byte aligned fp32 output")
        splitk = 1
    rc = _lib.lib().sb_gemm_bf16_splitk(
        P(a), P(b), P(out), P(bias), M, N, K, lda, ldb, ldc, int(a_mn), int(b_mn), int(out.dtype == torch.float32),
        int(accumulate), bn, int(splitk), P(_lib.status_word(a.device)), _lib.sm_count(a.device), _lib.stream(),
    )  # fmt: skip
    _lib.check(rc, "sb_gemm_bf16")
    return out


class _Linear(torch.autograd.Function):
    """y = x W^T (+ b). Backward: dx = dy W (B operand MN-major), dW = dy^T x (both MN-major),
    accumulated straight into ``weight.main_grad`` (fp32) when the parameter has one."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm(x2, weight, bias=bias)
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(-1) != 1 or (dy2.is_cuda and dy2.stride(0) % 8 != 0):
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True).view_as(x)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(weight, "main_grad", None)
            if main_grad is not None:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=main_grad, accumulate=True)
                dw = None
                weight.grad_added_to_main_grad = True
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def linear(x, weight, bias=None):
    return _Linear.apply(x, weight, bias)


# --------------------------------------------------------------------- RMSNorm
def _norm_ctas(device) -> int:
    return 2 * _lib.sm_count(device)


class _RMSNorm(torch.autograd.Function):
    """(y, h) = (rmsnorm(x + residual) * w, x + residual). The norm is computed from the
    un-rounded fp32 sum, matching the rollout engine's fused add+norm."""

    @staticmethod
    def forward(ctx, x, weight, residual, eps):
        shape = x.shape
        H = shape[-1]
        x2 = x.reshape(-1, H)
        T = x2.shape[0]
        if not _cuda(x):
            y, h, rstd = reference.rmsnorm(x2, weight, eps, None if residual is None else residual.reshape(-1, H))
            h = x2 if h is None else h
        else:
            x2 = x2.contiguous()
            r2 = None if residual is None else residual.reshape(-1, H).contiguous()
            f32x = x2.dtype == torch.float32  # the fp32 sum a split-K projection leaves behind (inference path)
            y = torch.empty(T, H, dtype=weight.dtype, device=x.device)
            h = torch.empty_like(y) if (r2 is not None or f32x) else x2
            rstd = torch.empty(T, dtype=torch.float32, device=x.device)
            fn = _lib.lib().sb_rmsnorm_fwd_f32x if f32x else _lib.lib().sb_rmsnorm_fwd
            rc = fn(P(x2), P(r2), P(weight), P(y), P(h) if h is not x2 else None, P(rstd), T, H, float(eps), _lib.stream())
            _lib.check(rc, "sb_rmsnorm_fwd")
        ctx.save_for_backward(h, weight, rstd)
        ctx.has_res = residual is not None
        ctx.shape = shape
        return y.view(shape), h.view(shape)

    @staticmethod
    def backward(ctx, dy, dh_in):
        h, weight, rstd = ctx.saved_tensors
        H = h.shape[-1]
        T = h.shape[0]
        dy2 = dy.reshape(-1, H)
        dres = None if dh_in is None else dh_in.reshape(-1, H)
        if not _cuda(dy):
            hf, dyf, wf = h.float(), dy2.float(), weight.float()
            xhat = hf * rstd[:, None]
            dyw = dyf * wf
            dot = (dyw * xhat).mean(-1, keepdim=True)
            dh = rstd[:, None] * (dyw - xhat * dot)
            if dres is not None:
                dh = dh + dres.float()
            dw = (dyf * xhat).sum(0)
            dh = dh.to(dy.dtype)
        else:
            dy2 = dy2.contiguous()
            dres = None if dres is None else dres.contiguous()
            dh = torch.empty_like(h)
            n = min(_norm_ctas(dy.device), max(T, 1))
            part = torch.empty(n, H, dtype=torch.float32, device=dy.device)
            dw = torch.empty(H, dtype=torch.float32, device=dy.device)
            rc = _lib.lib().sb_rmsnorm_bwd(P(dy2), P(h), P(weight), P(rstd), P(dres), P(dh), P(part), P(dw), T, H, n, 0,
                                           _lib.stream())
            _lib.check(rc, "sb_rmsnorm_bwd")
        main_grad = getattr(weight, "main_grad", None)
        if main_grad is not None:
            main_grad.add_(dw)
            weight.grad_added_to_main_grad = True
            dw_out = None
        else:
            dw_out = dw.to(weight.dtype)
        dh = dh.view(ctx.shape)
        return dh, dw_out, (dh if ctx.has_res else None), None


def rmsnorm(x, weight, eps=1e-6, residual=None):
    """Returns ``(normed, summed)`` where ``summed = x + residual`` (or ``x`` itself)."""
    return _RMSNorm.apply(x, weight, residual, eps)


# ------------------------------------------------------------------------ RoPE
def rope_cos_sin(max_pos, dim, base, device=None, scaling_factor=1.0):
    return reference.rope_cos_sin(max_pos, dim, base, device=device, scaling_factor=scaling_factor)


def rope_table(cfg, max_pos: int, dim: int, device=None):
    """``[max_pos, dim]`` = ``[cos | sin]`` for a model's ordinary (not latent-attention) rotary layers, with the
    frequency scaling its config names: none / linear (positions divided by the factor), ``llama3`` or ``yarn``."""
    kind = cfg.rotary_scaling_type if cfg.rotary_scaling_factor and cfg.rotary_scaling_factor != 1.0 else None
    if kind == "llama3":
        return reference.rope_cos_sin_llama3(max_pos, dim, cfg.rotary_base, cfg.rotary_scaling_factor, cfg.rotary_original_max_position,
                                             cfg.rope_low_freq_factor, cfg.rope_high_freq_factor, device=device)  # fmt: skip
    if kind == "yarn":
        return reference.rope_cos_sin_yarn(max_pos, dim, cfg.rotary_base, cfg.rotary_scaling_factor, cfg.rotary_original_max_position,
                                           cfg.yarn_beta_fast, cfg.yarn_beta_slow, cfg.mscale, cfg.mscale_all_dim, device=device)  # fmt: skip
    return reference.rope_cos_sin(max_pos, dim, cfg.rotary_base, device=device, scaling_factor=cfg.rotary_scaling_factor or 1.0)


def _rope_launch(x, out, positions, cos_sin, nw, rstd, nheads, head0, D, eps, sign):
    T = x.shape[0]
    rc = _lib.lib().sb_rope(P(x), P(out), P(positions), P(cos_sin), P(nw), P(rstd), T, nheads, head0, x.stride(0),
                            out.stride(0), D, float(eps), float(sign), _lib.stream())
    _lib.check(rc, "sb_rope")


class _RopeQK(torch.autograd.Function):
    """In a packed ``[T, (Hq + 2 Hkv) * D]`` qkv row: (per-head RMSNorm +) RoPE on the q and k heads,
    v copied through. Output is a new tensor of the same layout."""

    @staticmethod
    def forward(ctx, qkv, positions, cos_sin, q_norm_w, k_norm_w, Hq, Hkv, D, eps):
        T = qkv.shape[0]
        has_norm = q_norm_w is not None
        if not _cuda(qkv):
            x = qkv.view(T, Hq + 2 * Hkv, D)
            q = reference.rope(x[:, :Hq], positions, cos_sin, q_norm_w, eps)
            k = reference.rope(x[:, Hq : Hq + Hkv], positions, cos_sin, k_norm_w, eps)
            out = torch.cat([q, k, x[:, Hq + Hkv :]], dim=1).reshape(T, -1)
        else:
            qkv = qkv.contiguous()
            out = torch.empty_like(qkv)
            _rope_launch(qkv, out, positions, cos_sin, q_norm_w, None, Hq, 0, D, eps, 1.0)
            _rope_launch(qkv, out, positions, cos_sin, k_norm_w, None, Hkv, Hq, D, eps, 1.0)
            out.view(T, Hq + 2 * Hkv, D)[:, Hq + Hkv :].copy_(qkv.view(T, Hq + 2 * Hkv, D)[:, Hq + Hkv :])
        ctx.save_for_backward(qkv if has_norm else None, positions, cos_sin, q_norm_w, k_norm_w)
        ctx.dims = (Hq, Hkv, D, eps)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, positions, cos_sin, q_norm_w, k_norm_w = ctx.saved_tensors
        Hq, Hkv, D, eps = ctx.dims
        T = dout.shape[0]
        dout = dout.contiguous()
        d3 = dout.view(T, Hq + 2 * Hkv, D)
        # inverse rotation of the incoming gradient
        if not _cuda(dout):
            dq = reference.rope(d3[:, :Hq], positions, cos_sin, None, eps, sign=-1.0)
            dk = reference.rope(d3[:, Hq : Hq + Hkv], positions, cos_sin, None, eps, sign=-1.0)
        else:
            tmp = torch.empty_like(dout)
            _rope_launch(dout, tmp, positions, cos_sin, None, None, Hq + Hkv, 0, D, eps, -1.0)
            t3 = tmp.view(T, Hq + 2 * Hkv, D)
            dq, dk = t3[:, :Hq], t3[:, Hq : Hq + Hkv]
        dqw = dkw = None
        if q_norm_w is not None:
            x3 = qkv.view(T, Hq + 2 * Hkv, D)
            dq, dqw = _head_norm_bwd(x3[:, :Hq], dq, q_norm_w, eps)
            dk, dkw = _head_norm_bwd(x3[:, Hq : Hq + Hkv], dk, k_norm_w, eps)
        dqkv = torch.cat([dq.to(dout.dtype), dk.to(dout.dtype), d3[:, Hq + Hkv :]], dim=1).reshape(T, -1)
        return dqkv, None, None, dqw, dkw, None, None, None, None


def _head_norm_bwd(x, dy, w, eps):
    """Backward of per-head RMSNorm over the last dim (x: [T, H, D]); fp32 math."""
    D = x.shape[-1]
    if x.is_cuda:
        x2 = x.reshape(-1, D).contiguous()
        dy2 = dy.reshape(-1, D).contiguous()
        rows = x2.shape[0]
        rstd = torch.rsqrt(x2.float().pow(2).mean(-1) + eps)
        dh = torch.empty_like(x2)
        n = min(_norm_ctas(x.device), max(rows, 1))
        part = torch.empty(n, D, dtype=torch.float32, device=x.device)
        dw = torch.empty(D, dtype=torch.float32, device=x.device)
        rc = _lib.lib().sb_rmsnorm_bwd(P(dy2), P(x2), P(w), P(rstd), None, P(dh), P(part), P(dw), rows, D, n, 0,
                                       _lib.stream())
        _lib.check(rc, "sb_rmsnorm_bwd(head)")
        dx = dh.view(x.shape)
    else:
        xf, dyf = x.float(), dy.float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        xhat = xf * rstd
        dyw = dyf * w.float()
        dx = rstd * (dyw - xhat * (dyw * xhat).mean(-1, keepdim=True))
        dw = (dyf * xhat).sum((0, 1))
    main_grad = getattr(w, "main_grad", None)
    if main_grad is not None:
        main_grad.add_(dw)
        w.grad_added_to_main_grad = True
        return dx, None
    return dx, dw.to(w.dtype)


def rope_qk(qkv, positions, cos_sin, Hq, Hkv, D, q_norm_w=None, k_norm_w=None, eps=1e-6):
    return _RopeQK.apply(qkv, positions, cos_sin, q_norm_w, k_norm_w, Hq, Hkv, D, eps)


def rope_kv_write(qkv, positions, cos_sin, slots, k_cache, v_cache, Hq, Hkv, D, q_norm_w=None, k_norm_w=None, eps=1e-6):
    """Inference path: (per-head RMSNorm +) RoPE on the q and k heads of a packed qkv row IN PLACE, and the new k / v
    rows scattered into cache slot ``slots[t]`` (negative: skipped), as one launch. Returns ``qkv``."""
    T = qkv.shape[0]
    if _checks.enabled():
        _checks.index_range("rope_kv_write", "slots", slots, upper=k_cache.shape[0], lower=-(1 << 31))
        _checks.index_range("rope_kv_write", "positions", positions, upper=cos_sin.shape[0])
    if not _is_cuda(qkv):
        x = qkv.view(T, Hq + 2 * Hkv, D)
        x[:, :Hq] = reference.rope(x[:, :Hq], positions, cos_sin, q_norm_w, eps)
        x[:, Hq : Hq + Hkv] = reference.rope(x[:, Hq : Hq + Hkv], positions, cos_sin, k_norm_w, eps)
        kv_write(x[:, Hq : Hq + Hkv].reshape(T, -1), x[:, Hq + Hkv :].reshape(T, -1), slots, k_cache, v_cache)
        return qkv
    assert qkv.stride(1) == 1 and k_cache.is_contiguous() and v_cache.is_contiguous()
    rc = _lib.lib().sb_rope_kv_write(P(qkv), P(positions), P(cos_sin), P(q_norm_w), P(k_norm_w), P(slots), P(k_cache),
                                     P(v_cache), T, Hq, Hkv, D, qkv.stride(0), float(eps), _lib.stream())
    _lib.check(rc, "sb_rope_kv_write")
    return qkv


# ---------------------------------------------------------------------- SwiGLU
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        if not _is_cuda(gu):
            return reference.swiglu(gu)
        shape = gu.shape
        F_ = shape[-1] // 2
        g2 = gu.reshape(-1, 2 * F_).contiguous()
        act = torch.empty(g2.shape[0], F_, dtype=gu.dtype, device=gu.device)
        _lib.check(_lib.lib().sb_swiglu_fwd(P(g2), P(act), g2.shape[0], F_, _lib.stream()), "sb_swiglu_fwd")
        return act.view(*shape[:-1], F_)

    @staticmethod
    def backward(ctx, dact):
        (gu,) = ctx.saved_tensors
        F_ = gu.shape[-1] // 2
        if not _is_cuda(gu):
            g, u, d = gu[..., :F_].float(), gu[..., F_:].float(), dact.float()
            sg = torch.sigmoid(g)
            silu = g * sg
            return torch.cat([d * u * (sg + silu * (1 - sg)), d * silu], dim=-1).to(gu.dtype)
        g2 = gu.reshape(-1, 2 * F_).contiguous()
        d2 = dact.reshape(-1, F_).contiguous()
        dgu = torch.empty_like(g2)
        _lib.check(_lib.lib().sb_swiglu_bwd(P(g2), P(d2), P(dgu), g2.shape[0], F_, _lib.stream()), "sb_swiglu_bwd")
        return dgu.view_as(gu)


def swiglu(gu):
    return _SwiGLU.apply(gu)


# ------------------------------------------------------------------- embedding
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, vocab_lo):
        ctx.save_for_backward(ids)
        ctx.table = table
        ctx.vocab_lo = vocab_lo
        V, H = table.shape
        if not _cuda(table):
            local = ids.long() - vocab_lo
            ok = (local >= 0) & (local < V)
            out = table[local.clamp(0, V - 1)]
            return torch.where(ok[:, None], out, torch.zeros_like(out))
        ids32 = ids.to(torch.int32).contiguous()
        out = torch.empty(ids32.numel(), H, dtype=table.dtype, device=table.device)
        rc = _lib.lib().sb_embedding_fwd(P(ids32), P(table), P(out), ids32.numel(), H, vocab_lo, vocab_lo + V, _lib.stream())
        _lib.check(rc, "sb_embedding_fwd")
        return out

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        table = ctx.table
        V, H = table.shape
        main_grad = getattr(table, "main_grad", None)
        target = main_grad if main_grad is not None else torch.zeros(V, H, dtype=torch.float32, device=table.device)
        if not _cuda(table):
            local = ids.long() - ctx.vocab_lo
            ok = (local >= 0) & (local < V)
            target.index_add_(0, local[ok], dout.float()[ok])
        else:
            ids32 = ids.to(torch.int32).contiguous()
            rc = _lib.lib().sb_embedding_bwd(P(ids32), P(dout.contiguous()), P(target), ids32.numel(), H, ctx.vocab_lo,
                                             ctx.vocab_lo + V, _lib.stream())
            _lib.check(rc, "sb_embedding_bwd")
        if main_grad is not None:
            table.grad_added_to_main_grad = True
            return None, None, None
        return None, target.to(table.dtype), None


def embedding(ids, table, vocab_lo: int = 0):
    if _checks.enabled():  # ids of other vocabulary shards are legal (their rows come out as zeros); negatives are not
        _checks.index_range("embedding", "ids", ids, upper=1 << 31, lower=0)
    return _Embedding.apply(ids.reshape(-1), table, vocab_lo)


# ------------------------------------------------------------------- attention
def rope_attention(qkv, positions, cos_sin, cu_seqlens, max_seqlen, Hq, Hkv, D, q_norm_w=None, k_norm_w=None, eps=1e-6,
                   scale=None, cp_local_cu_seqlens=None, cp_group=None):
    """RoPE (+ per-head q/k RMSNorm) and packed causal attention on a fused qkv row, as one autograd node."""
    from slime_b200.ops import attention

    return attention.rope_attention(qkv, positions, cos_sin, cu_seqlens, max_seqlen, Hq, Hkv, D, q_norm_w, k_norm_w, eps, scale,
                                    cp_local_cu_seqlens, cp_group)


def varlen_attention(q, k, v, cu_seqlens, max_seqlen, scale=None, causal=True, sinks=None):
    """Packed causal GQA attention. q: [T, Hq, D], k/v: [T, Hkv, D]; ``sinks`` [Hq]: learnable per-head sink logits."""
    from slime_b200.ops import attention

    return attention.varlen_attention(q, k, v, cu_seqlens, max_seqlen, scale, causal, sinks)


def paged_decode_attention(q, k_cache, v_cache, block_table, seq_lens, page_size, scale=None, out=None, splits=None,
                           workspace=None, use_tensor_cores=True, sinks=None):
    """One query token per request over a paged KV cache. q: [B, Hq, D]; caches [slots, Hkv, D]."""
    B, Hq, D = q.shape
    Hkv = k_cache.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if _checks.enabled():
        _checks.paged("paged_decode_attention", block_table, seq_lens, page_size, k_cache.shape[0])
    if not _is_cuda(q) or D not in (64, 128) or sinks is not None:
        # the decode kernels cover head dims 64 and 128 without sinks; other widths (256: Qwen3-Next / Qwen3.5) and
        # softmax sinks take the plain form
        return reference.paged_decode_attention(q, k_cache, v_cache, block_table, seq_lens, page_size, scale, sinks)
    caller_splits = splits
    if splits is None and BATCH_INVARIANT:
        # the partial results of the splits are merged in split order: fix their number by the table width alone
        tiles = -(-block_table.shape[1] * page_size // 128)
        caller_splits = splits = max(1, min(16, -(-tiles // 16)))
    if splits is None:
        ctas = B * Hkv
        splits = 1 if ctas >= _lib.sm_count(q.device) else min(16, max(1, (2 * _lib.sm_count(q.device)) // max(ctas, 1)))
        tiles = -(-block_table.shape[1] * page_size // 128)  # 128-token tiles of the longest context the table can hold
        # Long contexts: one CTA per (request, kv head) would walk up to `tiles` tiles in sequence, and once most requests
        # of a batch have finished the few long ones left keep only a few SMs busy. At most ~16 tiles per CTA.
        splits = max(splits, min(16, -(-tiles // 16)))
        splits = max(1, min(splits, tiles))  # never more splits than tiles
    if out is None:
        out = torch.empty_like(q)
    same_layout = k_cache.stride() == v_cache.stride() and k_cache.stride(2) == 1
    # Head dim 64: the persistent warp-specialised kernel (four softmax groups per SM, one work item each). Measured
    # against the two-chain kernel below: 28.7 / 36.1 us at 256 requests x 2 kv heads and context 768, 50.4 / 74.0 us at
    # 512 requests, 21.6 / 33.6 us at 192, 16.0 / 17.0 us at 96, 112.7 / 158.1 us at context 4096, 13.3 / 12.9 us at 64
    # requests; below half an item per SM the two-chain kernel stays. SLIME_B200_DECODE_ATTN_WS=1 / 0 forces it on / off.
    ws_env = os.environ.get("SLIME_B200_DECODE_ATTN_WS", "")
    ws_ok = use_tensor_cores and D == 64 and Hq % Hkv == 0 and Hq // Hkv <= 8 and same_layout and ws_env != "0"
    if ws_ok and (ws_env == "1" or (not BATCH_INVARIANT and 2 * B * Hkv >= _lib.sm_count(q.device))):  # one kernel for every batch size
        ns = splits
        if caller_splits is None:
            # its own split rule: enough items for the 4 x SMs groups, at least 8 tiles of 128 tokens per split
            tiles = -(-block_table.shape[1] * page_size // 128)
            ns = max(1, min(16, (4 * _lib.sm_count(q.device)) // max(B * Hkv, 1), tiles // 8))
        if workspace is not None and workspace.numel() >= B * Hq * ns * (D + 2):
            ws_buf = workspace
        else:
            ws_buf = torch.empty(B * Hq * ns * (D + 2) if ns > 1 else 2, dtype=torch.float32, device=q.device)
        rc = _lib.lib().sb_paged_decode_ws(P(q), P(k_cache), P(v_cache), P(block_table), P(seq_lens), P(out),
                                           P(ws_buf[: B * Hq * ns * D]), P(ws_buf[B * Hq * ns * D : B * Hq * ns * (D + 2)]),
                                           B, Hq, Hkv, D, page_size, block_table.shape[1], k_cache.shape[0], q.stride(0),
                                           out.stride(0), ns, float(scale), P(_lib.status_word(q.device)),
                                           _lib.sm_count(q.device), k_cache.stride(0), k_cache.stride(1), _lib.stream())  # fmt: skip
        if rc != -1:
            _lib.check(rc, "sb_paged_decode_ws")
            return out
    assert k_cache.is_contiguous() and v_cache.is_contiguous(), "only the warp-specialised kernel takes a strided KV cache"
    if workspace is None and splits > 1:
        workspace = torch.empty(B * Hq * splits * (D + 2), dtype=torch.float32, device=q.device)
    part_o = workspace[: B * Hq * splits * D] if splits > 1 else None
    part_ml = workspace[B * Hq * splits * D : B * Hq * splits * (D + 2)] if splits > 1 else None
    if use_tensor_cores:
        # tcgen05 + TMA kernel; -1 = shape outside its coverage (odd head dim / group size / page size / alignment)
        rc = _lib.lib().sb_paged_decode_tc(P(q), P(k_cache), P(v_cache), P(block_table), P(seq_lens), P(out), P(part_o), P(part_ml),
                                           B, Hq, Hkv, D, page_size, block_table.shape[1], k_cache.shape[0], q.stride(0),
                                           out.stride(0), splits, float(scale), P(_lib.status_word(q.device)), _lib.stream())
        if rc != -1:
            _lib.check(rc, "sb_paged_decode_tc")
            return out
    if splits == 1:
        workspace = torch.empty(B * Hq * (D + 2), dtype=torch.float32, device=q.device)
        part_o, part_ml = workspace[: B * Hq * D], workspace[B * Hq * D :]
    rc = _lib.lib().sb_paged_decode(P(q), P(k_cache), P(v_cache), P(block_table), P(seq_lens), P(out), P(part_o), P(part_ml),
                                    B, Hq, Hkv, D, page_size, block_table.shape[1], q.stride(0), out.stride(0), splits,
                                    float(scale), _lib.stream())
    _lib.check(rc, "sb_paged_decode")
    return out


def kv_write(k, v, slots, k_cache, v_cache):
    """Scatter rows ``k[t], v[t]`` ([T, Hkv*D] views, possibly strided) into cache slot ``slots[t]``."""
    if _checks.enabled():
        _checks.index_range("kv_write", "slots", slots, upper=k_cache.shape[0], lower=-(1 << 31))
    row = k_cache.shape[1] * k_cache.shape[2]
    if not _is_cuda(k):
        ok = slots >= 0
        k_cache.view(-1, row)[slots[ok].long()] = k[ok].reshape(-1, row)
        v_cache.view(-1, row)[slots[ok].long()] = v[ok].reshape(-1, row)
        return
    rc = _lib.lib().sb_kv_write(P(k), P(v), P(slots), P(k_cache), P(v_cache), k.shape[0], row, k.stride(0), v.stride(0),
                                _lib.stream())
    _lib.check(rc, "sb_kv_write")


# -------------------------------------------------------------------- sampling
def sample(logits, temperature, top_k=None, top_p=None, min_p=None, seeds=None, positions=None, kept_cap=0):
    """Draw one token per row. Returns ``(token int32 [B], logprob fp32 [B], kept_ids, kept_count)``.

    ``logprob`` is the log-probability of the drawn token under the temperature-scaled
    distribution, renormalised over the kept set when top-k/top-p/min-p are active.
    """
    B, V = logits.shape
    dev = logits.device
    token = torch.empty(B, dtype=torch.int32, device=dev)
    logprob = torch.empty(B, dtype=torch.float32, device=dev)
    kept_ids = torch.empty(B, kept_cap, dtype=torch.int32, device=dev) if kept_cap > 0 else None
    kept_count = torch.zeros(B, dtype=torch.int32, device=dev) if kept_cap > 0 else None
    if not _is_cuda(logits):
        from slime_b200.ops.sampling_ref import sample_reference

        return sample_reference(logits, temperature, top_k, top_p, min_p, seeds, positions, kept_cap)
    assert logits.stride(-1) == 1
    rc = _lib.lib().sb_sample(P(logits), int(logits.dtype == torch.bfloat16), logits.stride(0), B, V, P(temperature),
                              P(top_k), P(top_p), P(min_p), P(seeds), P(positions), P(token), P(logprob), P(kept_ids),
                              P(kept_count), kept_cap, _lib.stream())
    _lib.check(rc, "sb_sample")
    return token, logprob, kept_ids, kept_count


# ----------------------------------------------------------------- quantisers
def block_fp8_quant(x, block=(128, 128), pow2_scale=False, out=None):
    """Block-scaled e4m3 of ``x`` [M, N]: ``(q, scale_inv [ceil(M/bm), ceil(N/bn)])``. ``out=(q, scale_inv)`` writes into
    existing contiguous tensors (the engine's resident fp8 buffers during a weight sync) instead of allocating."""
    if not _cuda(x):
        q, s = reference.block_fp8_quant(x, block, pow2_scale)
        if out is not None:
            out[0].copy_(q)
            out[1].copy_(s)
            return out
        return q, s
    x = x.contiguous()
    M, N = x.shape
    if out is not None:
        q, s = out
        assert q.is_contiguous() and s.is_contiguous() and q.shape == x.shape and s.dtype == torch.float32
        assert tuple(s.shape) == (-(-M // block[0]), -(-N // block[1]))
    else:
        q = torch.empty(M, N, dtype=torch.float8_e4m3fn, device=x.device)
        s = torch.empty(-(-M // block[0]), -(-N // block[1]), dtype=torch.float32, device=x.device)
    rc = _lib.lib().sb_block_fp8_quant(P(x), P(q), P(s), M, N, x.stride(0), q.stride(0), block[0], block[1],
                                       int(pow2_scale), _lib.stream())
    _lib.check(rc, "sb_block_fp8_quant")
    return q, s


def fp8_act_quant(x, pow2_scale=False):
    """1 x 128 activation quantisation to e4m3 -> (q [M, K], scale [M, K/128], scale_t [K/128, M]); ``scale_t`` is the
    K-block-major copy the fp8 GEMM reads (pass it as ``a_scale_t`` to skip a transpose)."""
    M, K = x.shape
    assert K % 128 == 0
    if not _cuda(x):
        q, s = reference.block_fp8_quant(x, (1, 128), pow2_scale)
        return q, s, s.t().contiguous()
    x = x.contiguous()
    q = torch.empty(M, K, dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty(M, K // 128, dtype=torch.float32, device=x.device)
    st = torch.empty(K // 128, M, dtype=torch.float32, device=x.device)
    rc = _lib.lib().sb_group_fp8_quant_1x128(P(x), P(q), P(s), P(st), M, K, x.stride(0), q.stride(0), int(pow2_scale), _lib.stream())
    _lib.check(rc, "sb_group_fp8_quant_1x128")
    return q, s, st


def fp8_block_gemm(a_q, a_scale, b_q, b_scale, out_dtype=torch.bfloat16, a_scale_t=None):
    """``(a_q * a_scale) @ (b_q * b_scale)^T`` for block-quantised e4m3 operands (W8A8 as block-fp8 checkpoints use it).

    ``a_q`` [M, K] e4m3 with ``a_scale`` [M, K/128] (one scale per row and 128-wide K group: ``block_fp8_quant(x, (1, 128))``);
    ``b_q`` [N, K] e4m3 with ``b_scale`` [ceil(N/128), K/128] (128 x 128 blocks). On CUDA the product runs on the tcgen05
    fp8 tensor cores with per-K-block promotion to fp32; on CPU it is the dequantised fp32 product.
    """
    M, K = a_q.shape
    N = b_q.shape[0]
    assert b_q.shape[1] == K and K % 128 == 0, "K must be a multiple of the 128-wide scale block"
    assert a_scale.shape == (M, K // 128) and b_scale.shape == (-(-N // 128), K // 128)
    if not _cuda(a_q):
        a = a_q.float() * a_scale.float().repeat_interleave(128, dim=1)
        b = b_q.float() * b_scale.float().repeat_interleave(128, dim=0)[:N].repeat_interleave(128, dim=1)
        return (a @ b.t()).to(out_dtype)
    a_q, b_q = a_q.contiguous(), b_q.contiguous()
    # [K/128, M]: the kernel reads one K block's row scales coalesced
    sa_t = a_scale_t if a_scale_t is not None else a_scale.float().t().contiguous()
    out = torch.empty(M, N, dtype=out_dtype, device=a_q.device)
    rc = _lib.lib().sb_gemm_fp8_block(P(a_q), P(b_q), P(sa_t), P(b_scale.float().contiguous()), P(out), M, N, K, a_q.stride(0),
                                      b_q.stride(0), out.stride(0), int(out_dtype == torch.float32),
                                      P(_lib.status_word(a_q.device)), _lib.sm_count(a_q.device), _lib.stream())  # fmt: skip
    _lib.check(rc, "sb_gemm_fp8_block")
    return out


def block_fp8_dequant(q, scale_inv, block=(128, 128), dtype=torch.bfloat16):
    if not _cuda(q):
        return reference.block_fp8_dequant(q, scale_inv, block, dtype)
    M, N = q.shape
    out = torch.empty(M, N, dtype=torch.bfloat16, device=q.device)
    rc = _lib.lib().sb_block_fp8_dequant(P(q.contiguous()), P(scale_inv.contiguous()), P(out), M, N, block[0], block[1],
                                         _lib.stream())
    _lib.check(rc, "sb_block_fp8_dequant")
    return out.to(dtype)


def fake_int4_quant(x, group=(1, 32), symmetric=True):
    """Quant-dequant to INT4 code values; returns (y, scales, zeros)."""
    if not _cuda(x):
        return reference.fake_int4(x, group, symmetric)
    x = x.contiguous()
    M, N = x.shape
    gm, gn = group
    y = torch.empty_like(x)
    s = torch.empty(-(-M // gm), -(-N // gn), dtype=torch.float32, device=x.device)
    z = torch.empty_like(s)
    rc = _lib.lib().sb_fake_int4(P(x), P(y), P(s), P(z), M, N, gm, gn, int(symmetric), _lib.stream())
    _lib.check(rc, "sb_fake_int4")
    return y, s, z


class FakeInt4STE(torch.autograd.Function):
    """Fake INT4 in forward, identity in backward (QAT on expert weights)."""

    @staticmethod
    def forward(ctx, w, group_size):
        return fake_int4_quant(w.reshape(-1, w.shape[-1]), (1, group_size), True)[0].view_as(w)

    @staticmethod
    def backward(ctx, g):
        return g, None


def router_gemm(x, w):
    """fp32 router logits ``x @ w^T`` with a batch-invariant reduction order (tokens in chunks of 16)."""
    if not _cuda(x):
        return x.float() @ w.float().t()
    x = x.contiguous()
    T, K = x.shape
    E = w.shape[0]
    out = torch.empty(T, E, dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().sb_router_gemm(P(x), P(w), P(out), T, K, E, _lib.stream()), "sb_router_gemm")
    return out
