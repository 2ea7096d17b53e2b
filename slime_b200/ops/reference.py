"""Plain PyTorch (fp32 math) definitions of every fused op.

They are the CPU execution path and the numerical oracle the GPU tests compare
the sm_100a kernels against.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def gemm(a, b, *, a_mn=False, b_mn=False, bias=None, out_dtype=None):
    """op(A)[M,K] @ op(B)[N,K]^T. ``a_mn``: A is stored [K,M]; ``b_mn``: B is stored [K,N]."""
    A = a.float().t() if a_mn else a.float()
    Bm = b.float() if b_mn else b.float().t()
    out = A @ Bm
    if bias is not None:
        out = out + bias.float()
    return out.to(out_dtype or a.dtype)


def rmsnorm(x, w, eps, residual=None):
    h = x.float() if residual is None else x.float() + residual.float()
    rstd = torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    y = (h * rstd * w.float()).to(x.dtype)
    return y, (h.to(x.dtype) if residual is not None else None), rstd.squeeze(-1)


def rope_cos_sin(max_pos: int, dim: int, base: float, device=None, scaling_factor: float = 1.0) -> torch.Tensor:
    """Table ``[max_pos, dim]`` fp32 = ``[cos(dim/2) | sin(dim/2)]`` per position."""
    inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float64, device=device) / dim))
    pos = torch.arange(max_pos, dtype=torch.float64, device=device) / scaling_factor
    ang = pos[:, None] * inv_freq[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=-1).float()


def rope_cos_sin_llama3(max_pos: int, dim: int, base: float, factor: float, original_max_position: int, low_freq_factor: float = 1.0,
                        high_freq_factor: float = 4.0, device=None) -> torch.Tensor:
    """Table with Llama-3.1 style frequencies: bands whose wavelength exceeds ``original / low_freq_factor`` are slowed
    by ``factor``, bands shorter than ``original / high_freq_factor`` are kept, the ones in between blend linearly in
    ``original / wavelength`` (what ``--use-rope-scaling --rope-scaling-factor`` selects in the reference's trainer)."""
    import math

    inv = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
    wavelen = 2 * math.pi / inv
    smooth = ((original_max_position / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)).clamp(0, 1)
    inv = (1 - smooth) * inv / factor + smooth * inv  # smooth = 0 for long waves, 1 for short ones
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    out = torch.cat([ang.cos(), ang.sin()], dim=-1).float()
    return out.to(device) if device is not None else out


def yarn_inv_freq(dim: int, base: float, factor: float, original_max_position: int, beta_fast: float = 32.0,
                  beta_slow: float = 1.0) -> torch.Tensor:
    """YaRN frequencies: dimensions that turn more than ``beta_fast`` times over the original context keep their
    frequency, those that turn less than ``beta_slow`` times are slowed by ``factor`` (position interpolation), the
    ones in between blend linearly."""
    import math

    idx = torch.arange(0, dim, 2, dtype=torch.float64)
    extra = 1.0 / (base ** (idx / dim))
    inter = extra / factor

    def correction_dim(rotations: float) -> float:
        return dim * math.log(original_max_position / (rotations * 2 * math.pi)) / (2 * math.log(base))

    low = max(math.floor(correction_dim(beta_fast)), 0)
    high = min(math.ceil(correction_dim(beta_slow)), dim - 1)
    ramp = ((torch.arange(dim // 2, dtype=torch.float64) - low) / max(high - low, 1e-3)).clamp(0, 1)
    keep = 1.0 - ramp
    return inter * (1 - keep) + extra * keep


def yarn_mscale(factor: float, mscale: float = 1.0) -> float:
    import math

    return 1.0 if factor <= 1 else 0.1 * mscale * math.log(factor) + 1.0


def rope_cos_sin_yarn(max_pos: int, dim: int, base: float, factor: float, original_max_position: int, beta_fast: float = 32.0,
                      beta_slow: float = 1.0, mscale: float = 1.0, mscale_all_dim: float = 0.0, device=None) -> torch.Tensor:
    """Table ``[max_pos, dim]`` = ``[cos | sin]`` with YaRN frequencies; the table carries the magnitude correction
    ``yarn_mscale(factor, mscale) / yarn_mscale(factor, mscale_all_dim)`` (1 when both are equal)."""
    inv = yarn_inv_freq(dim, base, factor, original_max_position, beta_fast, beta_slow)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    m = yarn_mscale(factor, mscale) / yarn_mscale(factor, mscale_all_dim)
    return (torch.cat([ang.cos(), ang.sin()], dim=-1) * m).float().to(device) if device is not None else (
        torch.cat([ang.cos(), ang.sin()], dim=-1) * m).float()


def rope(x, positions, cos_sin, norm_weight=None, eps=1e-6, sign=1.0):
    """x: [T, H, D]; rotate-half RoPE, optionally preceded by per-head RMSNorm over D."""
    T, H, D = x.shape
    a = x.float()
    if norm_weight is not None:
        a = a * torch.rsqrt(a.pow(2).mean(-1, keepdim=True) + eps) * norm_weight.float()
    cs = cos_sin[positions.long()]
    c, s = cs[:, None, : D // 2], cs[:, None, D // 2 :] * sign
    lo, hi = a[..., : D // 2], a[..., D // 2 :]
    return torch.cat([lo * c - hi * s, hi * c + lo * s], dim=-1).to(x.dtype)


def swiglu(gu):
    F_ = gu.shape[-1] // 2
    g, u = gu[..., :F_].float(), gu[..., F_:].float()
    return (F.silu(g) * u).to(gu.dtype)


def varlen_attention(q, k, v, cu_seqlens, scale=None, causal=True):
    """q: [T, Hq, D], k/v: [T, Hkv, D] packed; per-sequence causal attention with GQA."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty_like(q)
    cu = cu_seqlens.tolist()
    for s, e in zip(cu[:-1], cu[1:]):
        if e == s:
            continue
        qs = q[s:e].float().transpose(0, 1)  # [Hq, L, D]
        ks = k[s:e].float().transpose(0, 1).repeat_interleave(Hq // Hkv, dim=0)
        vs = v[s:e].float().transpose(0, 1).repeat_interleave(Hq // Hkv, dim=0)
        att = (qs @ ks.transpose(-1, -2)) * scale
        if causal:
            L = e - s
            mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
            att = att.masked_fill(~mask, float("-inf"))
        out[s:e] = (att.softmax(-1) @ vs).transpose(0, 1).to(q.dtype)
    return out


def paged_decode_attention(q, k_cache, v_cache, block_table, seq_lens, page_size, scale=None, sinks=None):
    """q: [B, Hq, D]; caches [slots, Hkv, D]; attends over the first seq_lens[b] cached tokens. ``sinks`` [Hq]: one extra
    logit per head in the softmax denominator (it carries no value)."""
    B, Hq, D = q.shape
    Hkv = k_cache.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty_like(q)
    for b in range(B):
        n = int(seq_lens[b])
        pos = torch.arange(n, device=q.device)
        slots = block_table[b, pos // page_size].long() * page_size + pos % page_size
        ks = k_cache[slots].float().repeat_interleave(Hq // Hkv, dim=1)  # [n, Hq, D]
        vs = v_cache[slots].float().repeat_interleave(Hq // Hkv, dim=1)
        logits = torch.einsum("hd,nhd->hn", q[b].float() * scale, ks)
        if sinks is not None:
            att = torch.cat([logits, sinks.float()[:, None]], dim=-1).softmax(-1)[:, :-1]
        else:
            att = logits.softmax(-1)
        out[b] = torch.einsum("hn,nhd->hd", att, vs).to(q.dtype)
    return out


def logprob_entropy(logits, targets, inv_temperature=1.0):
    z = logits.float() * inv_temperature
    lse = torch.logsumexp(z, -1)
    lp = z.gather(-1, targets.long()[:, None]).squeeze(-1) - lse
    p = torch.softmax(z, -1)
    ent = lse - (p * z).sum(-1)
    return lp, ent, lse


def pg_loss(logp, old_logp, adv, w, eps_lo, eps_hi, eps_c=None, mode=0, tis=None):
    """Weighted clipped surrogate; returns (sum w*L, sum w*clipfrac, sum w*kl, sum w, dL/dlogp)."""
    logp = logp.detach().clone().requires_grad_(True)
    kl = old_logp - logp
    ratio = torch.exp(-kl)
    rc = ratio.clamp(1 - eps_lo, 1 + eps_hi)
    if mode == 1:
        L = -rc.detach() * adv * logp
        clip = (rc != ratio).float()
    else:
        l1, l2 = -ratio * adv, -rc * adv
        L = torch.maximum(l1, l2)
        clip = (l2 > l1).float()
        if eps_c is not None and eps_c > 1:
            L = torch.where(adv < 0, torch.minimum(-eps_c * adv, L), L)
    wt = w if tis is None else w * tis
    total = (L * wt).sum()
    (g,) = torch.autograd.grad(total, logp)
    return total.detach(), (clip * w).sum(), (kl.detach() * w).sum(), w.sum(), g


def adam_step(p, m, v, g, lr, beta1, beta2, eps, wd, step, grad_scale=1.0, clip_coef=1.0):
    g = g.float() * grad_scale * clip_coef
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1, bc2 = 1 - beta1**step, 1 - beta2**step
    p.mul_(1 - lr * wd)
    p.addcdiv_(m / bc1, (v / bc2).sqrt() + eps, value=-lr)
    return p


def block_fp8_quant(x, block=(128, 128), pow2_scale=False):
    """128x128 block-scaled e4m3: returns (q fp8, scale_inv fp32 [ceil(M/bm), ceil(N/bn)])."""
    M, N = x.shape
    bm, bn = block
    pm, pn = -(-M // bm) * bm, -(-N // bn) * bn
    xp = torch.zeros(pm, pn, dtype=torch.float32, device=x.device)
    xp[:M, :N] = x.float()
    blocks = xp.view(pm // bm, bm, pn // bn, bn)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-10)
    scale = amax / 448.0
    if pow2_scale:
        scale = torch.exp2(torch.ceil(torch.log2(scale)))
    q = (blocks / scale[:, None, :, None]).clamp(-448, 448).view(pm, pn)[:M, :N].to(torch.float8_e4m3fn)
    return q, scale


def block_fp8_dequant(q, scale_inv, block=(128, 128), dtype=torch.bfloat16):
    M, N = q.shape
    bm, bn = block
    s = scale_inv.repeat_interleave(bm, 0)[:M].repeat_interleave(bn, 1)[:, :N]
    return (q.float() * s).to(dtype)


def fake_int4(x, group=(1, 32), symmetric=True):
    M, N = x.shape
    gm, gn = group
    xf = x.float().view(M // gm, gm, N // gn, gn)
    if symmetric:
        s = xf.abs().amax(dim=(1, 3), keepdim=True).clamp_min(1e-8) / 7.0
        y = torch.round(xf / s).clamp(-8, 7) * s
        z = torch.zeros_like(s)
    else:
        mx, mn = xf.amax(dim=(1, 3), keepdim=True), xf.amin(dim=(1, 3), keepdim=True)
        s = (mx - mn).clamp_min(1e-8) / 15.0
        z = torch.round(-mn / s).clamp(0, 15)
        y = ((torch.round(xf / s) + z).clamp(0, 15) - z) * s
    return y.view(M, N).to(x.dtype), s.view(M // gm, N // gn), z.view(M // gm, N // gn)


def topp_topk_keep_mask(probs, top_k, top_p, min_p=0.0):
    """Keep token i iff (#tokens with larger p) < top_k and (mass of larger p) <= top_p and p >= p_max*min_p."""
    sp, idx = probs.sort(-1, descending=True)
    mass_above = sp.cumsum(-1) - sp
    rank = torch.arange(probs.shape[-1], device=probs.device).expand_as(sp)
    keep_sorted = mass_above <= top_p
    if top_k is not None and top_k > 0:
        keep_sorted &= rank < top_k
    if min_p > 0:
        keep_sorted &= sp >= sp[..., :1] * min_p
    keep = torch.zeros_like(keep_sorted)
    keep.scatter_(-1, idx, keep_sorted)
    return keep
