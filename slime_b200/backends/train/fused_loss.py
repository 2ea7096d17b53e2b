"""Fused LM-head + log-prob/entropy + clipped policy loss (forward and backward in one sweep).

The ``[T, V]`` logits are never kept: response rows are processed in chunks; for each chunk
the LM-head GEMM writes fp32 logits into a reusable workspace, one kernel reduces every row to
(max, sum-exp, target logit, sum p*z), a [rows]-sized kernel evaluates the PPO-clip / CISPO
surrogate and its derivative, a second row kernel turns the workspace into bf16 dlogits and
two more tcgen05 GEMMs produce dH and accumulate dW into the fp32 main-grad buffer.
Because every per-token loss weight is known before the forward (mask / denominators / global
batch), the backward of this op is a multiplication by the upstream scalar.

This is the fast path for the standard GRPO / GSPO-free objective; every other option takes the
general path in ``loss.py`` (which is also this path's numerical oracle).
Replaces the logits materialisation + ``_VocabParallelLogProbEntropy`` + ``compute_policy_loss``
sequence of the reference (slime/utils/ppo_utils.py:187-336, 124-171).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from slime_b200 import ops
from slime_b200.ops import _lib, reference
from slime_b200.parallel import state as mpu

P = _lib.ptr


def _reduce_stats_tp(stats: torch.Tensor, group):
    """stats[:, 0]=max, 1=sumexp (rel. max), 2=target logit, 3=sum e*z (rel. max); combine over TP."""
    if group is None or dist.get_world_size(group) == 1:
        return stats
    gmax = stats[:, 0].clone()
    dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
    scale = torch.exp(stats[:, 0] - gmax)
    packed = torch.stack([stats[:, 1] * scale, stats[:, 2], stats[:, 3] * scale], dim=1)
    dist.all_reduce(packed, group=group)
    return torch.stack([gmax, packed[:, 0], packed[:, 1], packed[:, 2]], dim=1).contiguous()


def logprob_entropy_rows(h_rows, weight, targets, *, inv_temperature=1.0, vocab_lo=0, tp_group=None, chunk=4096,
                         with_entropy=True, workspace=None):
    """No-grad log-prob / entropy of ``targets`` for hidden rows ``[R, H]`` (chunked, fused kernels)."""
    R = h_rows.shape[0]
    Vp = weight.shape[0]
    dev = h_rows.device
    logp = torch.empty(R, dtype=torch.float32, device=dev)
    ent = torch.empty(R, dtype=torch.float32, device=dev) if with_entropy else None
    if R == 0:
        return logp, ent
    if not h_rows.is_cuda:
        z = reference.gemm(h_rows, weight, out_dtype=torch.float32)
        assert tp_group is None or dist.get_world_size(tp_group) == 1
        lp, en, _ = reference.logprob_entropy(z, targets - vocab_lo, inv_temperature)
        return lp, (en if with_entropy else None)
    chunk = min(chunk, R)
    ws = workspace if workspace is not None else torch.empty(chunk, Vp, dtype=torch.float32, device=dev)
    stats = torch.empty(chunk, 4, dtype=torch.float32, device=dev)
    lse = torch.empty(chunk, dtype=torch.float32, device=dev)
    lib = _lib.lib()
    tg = targets.to(torch.int32).contiguous()
    for s in range(0, R, chunk):
        n = min(chunk, R - s)
        ops.gemm(h_rows[s : s + n], weight, out=ws[:n])
        _lib.check(lib.sb_softmax_stats(P(ws), P(tg[s:]), P(stats), n, Vp, ws.stride(0), vocab_lo, float(inv_temperature),
                                        _lib.stream()), "sb_softmax_stats")  # fmt: skip
        st = _reduce_stats_tp(stats[:n], tp_group)
        _lib.check(lib.sb_finalize_logprob(P(st), P(logp[s:]), P(ent[s:]) if with_entropy else None, P(lse), n,
                                           _lib.stream()), "sb_finalize_logprob")  # fmt: skip
    return logp, ent


class _FusedPolicyLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h_rows, weight, targets, old_logp, adv, w, tis, cfg):
        (eps_lo, eps_hi, eps_c, mode, entropy_coef, inv_t, vocab_lo, tp_group, chunk) = cfg
        R, H = h_rows.shape
        Vp = weight.shape[0]
        dev = h_rows.device
        lib = _lib.lib()
        chunk = max(1, min(chunk, R))
        ws = torch.empty(chunk, Vp, dtype=torch.float32, device=dev)
        dl = torch.empty(chunk, Vp, dtype=torch.bfloat16, device=dev)
        stats = torch.empty(chunk, 4, dtype=torch.float32, device=dev)
        logp = torch.empty(R, dtype=torch.float32, device=dev)
        ent = torch.empty(R, dtype=torch.float32, device=dev)
        lse = torch.empty(R, dtype=torch.float32, device=dev)
        g_lp = torch.empty(R, dtype=torch.float32, device=dev)
        acc = torch.zeros(4, dtype=torch.float32, device=dev)
        dh = torch.empty(R, H, dtype=h_rows.dtype, device=dev)
        tg = targets.to(torch.int32).contiguous()
        main_grad = getattr(weight, "main_grad", None)
        dw = main_grad if main_grad is not None else torch.zeros(Vp, H, dtype=torch.float32, device=dev)
        g_ent = (-entropy_coef * w).contiguous() if entropy_coef != 0 else None
        for s in range(0, R, chunk):
            n = min(chunk, R - s)
            ops.gemm(h_rows[s : s + n], weight, out=ws[:n])
            _lib.check(lib.sb_softmax_stats(P(ws), P(tg[s:]), P(stats), n, Vp, ws.stride(0), vocab_lo, float(inv_t),
                                            _lib.stream()), "sb_softmax_stats")  # fmt: skip
            st = _reduce_stats_tp(stats[:n], tp_group)
            _lib.check(lib.sb_finalize_logprob(P(st), P(logp[s:]), P(ent[s:]), P(lse[s:]), n, _lib.stream()),
                       "sb_finalize_logprob")  # fmt: skip
            old = old_logp[s:] if old_logp is not None else logp[s:]  # no stored old policy: ratio == 1
            _lib.check(lib.sb_pg_loss(P(logp[s:]), P(old), P(adv[s:]), P(w[s:]), P(tis[s:]) if tis is not None else None,
                                      P(g_lp[s:]), None, P(acc), n, eps_lo, eps_hi, eps_c, mode, _lib.stream()),
                       "sb_pg_loss")  # fmt: skip
            _lib.check(lib.sb_dlogits(P(ws), P(tg[s:]), P(lse[s:]), P(ent[s:]), P(g_lp[s:]),
                                      P(g_ent[s:]) if g_ent is not None else None, P(dl), n, Vp, ws.stride(0),
                                      dl.stride(0), vocab_lo, float(inv_t), _lib.stream()), "sb_dlogits")  # fmt: skip
            ops.gemm(dl[:n], weight, b_mn=True, out=dh[s : s + n])
            ops.gemm(dl[:n], h_rows[s : s + n], a_mn=True, b_mn=True, out=dw, accumulate=True)
        ent_sum = (ent * w).sum()
        loss = acc[0] - entropy_coef * ent_sum
        if tp_group is not None and dist.get_world_size(tp_group) > 1:
            dist.all_reduce(dh, group=tp_group)
        ctx.save_for_backward(dh)
        ctx.weight = weight
        ctx.dw = None if main_grad is not None else dw
        ctx.mark_non_differentiable(logp, ent)
        metrics = torch.stack([acc[0], acc[1], acc[2], ent_sum, acc[3]])
        ctx.mark_non_differentiable(metrics)
        return loss, logp, ent, metrics

    @staticmethod
    def backward(ctx, g_loss, *_):
        (dh,) = ctx.saved_tensors
        w = ctx.weight
        if ctx.dw is None:
            # dW already sits in main_grad with unit upstream scale; the training loop calls backward
            # with the scalar 1 (loss scaling is folded into the per-token weights)
            w.grad_added_to_main_grad = True
            dw = None
        else:
            dw = (ctx.dw * g_loss).to(w.dtype)
        return dh * g_loss.to(dh.dtype), dw, None, None, None, None, None, None


def fused_policy_loss(h_rows, weight, targets, old_logp, adv, w, *, eps_clip, eps_clip_high, eps_clip_c=None,
                      cispo=False, entropy_coef=0.0, temperature=1.0, tis=None, chunk=4096):
    """Returns ``(loss, logp, entropy, metrics)`` with ``metrics = [sum w*L, sum w*clipfrac, sum w*(old-new),
    sum w*entropy, sum w]``. ``w`` carries mask / denominator / global-batch normalisation per token."""
    tp_group = mpu.get_tensor_model_parallel_group()
    vocab_lo = mpu.get_tensor_model_parallel_rank() * weight.shape[0]
    if not h_rows.is_cuda:
        return _reference_policy_loss(h_rows, weight, targets, old_logp, adv, w, eps_clip, eps_clip_high, eps_clip_c,
                                      cispo, entropy_coef, temperature, tis, vocab_lo)  # fmt: skip
    cfg = (float(eps_clip), float(eps_clip_high), float(eps_clip_c or 0.0), int(cispo), float(entropy_coef),
           1.0 / float(temperature), int(vocab_lo), tp_group, int(chunk))  # fmt: skip
    return _FusedPolicyLoss.apply(h_rows, weight, targets, old_logp, adv.contiguous(), w.contiguous(), tis, cfg)


def _reference_policy_loss(h_rows, weight, targets, old_logp, adv, w, eps_lo, eps_hi, eps_c, cispo, entropy_coef,
                           temperature, tis, vocab_lo):
    """CPU / oracle path: same contract through autograd."""
    from slime_b200.utils.ppo_utils import compute_cispo_loss, compute_policy_loss

    z = (h_rows.float() @ weight.float().t()) / temperature
    lse = torch.logsumexp(z, -1)
    logp = z.gather(-1, (targets.long() - vocab_lo)[:, None]).squeeze(-1) - lse
    p = torch.softmax(z, -1)
    ent = lse - (p * z).sum(-1)
    old = logp.detach() if old_logp is None else old_logp
    kl = old - logp
    if cispo:
        L, clip = compute_cispo_loss(kl, logp, adv, eps_lo, eps_hi)
    else:
        L, clip = compute_policy_loss(kl, adv, eps_lo, eps_hi, eps_c)
    wt = w if tis is None else w * tis
    ent_sum = (ent * w).sum()
    loss = (L * wt).sum() - entropy_coef * ent_sum
    metrics = torch.stack([(L * wt).sum(), (clip * w).sum(), (kl * w).sum(), ent_sum, w.sum()]).detach()
    return loss, logp.detach(), ent.detach(), metrics
