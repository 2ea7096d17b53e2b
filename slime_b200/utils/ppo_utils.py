"""Policy-gradient math: KL estimators, clipped surrogates, returns/GAE and
vocab-parallel log-prob/entropy.

Parity with slime/utils/ppo_utils.py: compute_approx_kl :11-51,
compute_opsm_mask :54-92, compute_gspo_kl :95-121, compute_policy_loss
:124-148, compute_cispo_loss :151-171, vocab-parallel logprob/entropy
:187-336, returns/GAE :361-715, calculate_log_probs_and_entropy :718-769.

Everything here is plain fp32 PyTorch and runs on CPU; on a GPU the fused
sm_100a kernels in ``slime_b200.ops`` (LM-head GEMM + online softmax + target
gather + clipped loss) are used by the training backend instead of the
[T, V] logits path, and these functions are their numerical oracle.
"""

from __future__ import annotations

from argparse import Namespace

import torch
import torch.distributed as dist

from slime_b200.parallel import state as mpu


# --------------------------------------------------------------------------- KL
def compute_approx_kl(
    log_probs: torch.Tensor,
    log_probs_base: torch.Tensor,
    kl_loss_type: str,
    importance_ratio: torch.Tensor | None = None,
) -> torch.Tensor:
    """Per-token KL(new || base) estimators k1 / k2 / k3 / low_var_kl.

    ``importance_ratio`` (pi_theta / pi_old) makes the estimate unbiased under
    off-policy sampling. ``low_var_kl`` is k3 clamped to [-10, 10].
    """
    d = log_probs.float() - log_probs_base.float()
    if kl_loss_type == "k1":
        kl = d
    elif kl_loss_type == "k2":
        kl = 0.5 * d * d
    elif kl_loss_type in ("k3", "low_var_kl"):
        nd = -d
        kl = torch.expm1(nd) - nd
    else:
        raise ValueError(f"Unknown kl_loss_type: {kl_loss_type}")
    if importance_ratio is not None:
        kl = importance_ratio * kl
    if kl_loss_type == "low_var_kl":
        kl = kl.clamp(-10.0, 10.0)
    return kl


def _seq_mean_kl(old_lp, new_lp, mask):
    return ((old_lp - new_lp) * mask).sum() / mask.sum().clamp_min(1)


def compute_opsm_mask(
    args: Namespace,
    full_log_probs: list[torch.Tensor],
    full_old_log_probs: list[torch.Tensor],
    advantages: list[torch.Tensor],
    loss_masks: list[torch.Tensor],
) -> tuple[torch.Tensor, torch.Tensor]:
    """Off-policy sequence masking: drop tokens with A<0 in sequences whose mean
    ``old - new`` log-ratio exceeds ``args.opsm_delta``. Returns the concatenated
    keep-mask and the per-sequence-normalised count of dropped tokens."""
    keep, frac = [], torch.zeros((), device=advantages[0].device)
    for lp, old, adv, m in zip(full_log_probs, full_old_log_probs, advantages, loss_masks):
        kl = _seq_mean_kl(old, lp, m)
        drop = ((adv < 0) & (kl > args.opsm_delta)).float()
        frac = frac + drop.sum() / m.sum().clamp_min(1)
        keep.append(1.0 - drop)
    return torch.cat(keep, dim=0), frac


def compute_gspo_kl(
    full_log_probs: list[torch.Tensor],
    full_old_log_probs: list[torch.Tensor],
    local_log_probs: list[torch.Tensor],
    loss_masks: list[torch.Tensor],
) -> torch.Tensor:
    """GSPO: one sequence-level KL per sample, broadcast over its (CP-local) tokens."""
    pieces = []
    for lp, old, local, m in zip(full_log_probs, full_old_log_probs, local_log_probs, loss_masks):
        pieces.append(_seq_mean_kl(old, lp, m).expand_as(local))
    return torch.cat(pieces, dim=0)


# ----------------------------------------------------------------- surrogates
def compute_policy_loss(
    ppo_kl: torch.Tensor,
    advantages: torch.Tensor,
    eps_clip: float,
    eps_clip_high: float,
    eps_clip_c: float | None = None,
):
    """PPO clipped surrogate with asymmetric clip range and optional dual clip.

    ``ppo_kl = old_logp - new_logp`` so ``ratio = exp(-ppo_kl)``. Returns the
    per-token loss and the 0/1 indicator that the clipped branch was active.
    """
    ratio = torch.exp(-ppo_kl)
    unclipped = -ratio * advantages
    clipped = -ratio.clamp(1.0 - eps_clip, 1.0 + eps_clip_high) * advantages
    loss = torch.maximum(unclipped, clipped)
    clipfrac = (clipped > unclipped).float()
    if eps_clip_c is not None:
        assert eps_clip_c > 1.0, f"dual-clip bound eps_clip_c must be > 1.0, got {eps_clip_c}"
        dual = torch.minimum(-eps_clip_c * advantages, loss)
        loss = torch.where(advantages < 0, dual, loss)
    return loss, clipfrac


def compute_cispo_loss(
    ppo_kl: torch.Tensor,
    log_probs: torch.Tensor,
    advantages: torch.Tensor,
    eps_clip: float,
    eps_clip_high: float,
):
    """CISPO (MiniMax-M1): ``-sg(clip(ratio)) * A * logp``; gradient flows through
    ``log_probs`` only, so clipped tokens still contribute."""
    ratio = torch.exp(-ppo_kl)
    trunc = ratio.clamp(1.0 - eps_clip, 1.0 + eps_clip_high)
    loss = -trunc.detach() * advantages * log_probs
    return loss, (trunc != ratio).float()


# ------------------------------------------- vocab-parallel logprob / entropy
def _group_size_rank(group) -> tuple[int, int]:
    if group is None or not (dist.is_available() and dist.is_initialized()):
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


def _all_reduce_(t: torch.Tensor, op, group) -> None:
    if group is not None and dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=op, group=group)


class VocabParallelLogProbEntropy(torch.autograd.Function):
    """log p(target) and entropy from vocab-sharded logits ``[T, V/tp]``.

    Forward does TP reductions of ``[T]`` vectors only (max, sum-exp,
    sum p*logit, target logit); backward is analytic:
    ``d logp/d z = onehot - p`` and ``d H/d z = -p * (log p + H)``.

    With a keep-mask (top-p replay) the log-prob uses the masked distribution
    (target force-kept) while the entropy always uses the unmasked one.
    """

    @staticmethod
    def forward(ctx, logits, tokens, keep_mask, group, with_entropy, with_entropy_grad):
        tp, rank = _group_size_rank(group)
        z = logits.float()
        T, Vp = z.shape
        lo = rank * Vp
        local = tokens - lo
        owned = (local >= 0) & (local < Vp)
        local_c = local.clamp(0, Vp - 1)

        # ---- unmasked distribution (entropy, and logprob when no mask) ----
        zmax = z.max(dim=-1).values
        _all_reduce_(zmax, dist.ReduceOp.MAX, group)
        ez = torch.exp(z - zmax[:, None])
        denom = ez.sum(-1)
        _all_reduce_(denom, dist.ReduceOp.SUM, group)
        p = ez / denom[:, None]
        log_denom = denom.log() + zmax  # logsumexp

        tgt = torch.where(owned, z.gather(-1, local_c[:, None]).squeeze(-1), torch.zeros_like(zmax))
        _all_reduce_(tgt, dist.ReduceOp.SUM, group)

        entropy = None
        if with_entropy:
            pz = (p * z).sum(-1)
            _all_reduce_(pz, dist.ReduceOp.SUM, group)
            entropy = log_denom - pz

        if keep_mask is None:
            logp = tgt - log_denom
            p_lp = p
        else:
            km = keep_mask.clone()
            rows = torch.nonzero(owned, as_tuple=True)[0]
            km[rows, local_c[rows]] = True  # the sampled token is always kept
            zm = z.masked_fill(~km, float("-inf"))
            mmax = zm.max(dim=-1).values
            _all_reduce_(mmax, dist.ReduceOp.MAX, group)
            em = torch.exp(zm - mmax[:, None])
            mden = em.sum(-1)
            _all_reduce_(mden, dist.ReduceOp.SUM, group)
            p_lp = em / mden[:, None]
            logp = tgt - (mden.log() + mmax)

        ctx.with_entropy = bool(with_entropy and with_entropy_grad)
        ctx.in_dtype = logits.dtype
        saved = [p_lp, owned, local_c]
        if ctx.with_entropy:
            saved += [p, z, entropy, log_denom]
        ctx.save_for_backward(*saved)
        if entropy is None:
            entropy = torch.zeros_like(logp)
        if not ctx.with_entropy:
            ctx.mark_non_differentiable(entropy)
        return logp, entropy

    @staticmethod
    def backward(ctx, g_logp, g_ent):
        saved = ctx.saved_tensors
        p_lp, owned, local_c = saved[:3]
        grad = -p_lp * g_logp[:, None]
        rows = torch.nonzero(owned, as_tuple=True)[0]
        grad[rows, local_c[rows]] += g_logp[rows]
        if ctx.with_entropy and g_ent is not None:
            p, z, entropy, log_denom = saved[3:]
            logp_all = z - log_denom[:, None]
            grad = grad - (p * (logp_all + entropy[:, None])) * g_ent[:, None]
        return grad.to(ctx.in_dtype), None, None, None, None, None


def _logp_entropy_rows(logits, tokens, tp_group, with_entropy, with_entropy_grad, keep_mask):
    logp, ent = VocabParallelLogProbEntropy.apply(logits, tokens, keep_mask, tp_group, with_entropy, with_entropy_grad)
    return logp, (ent if with_entropy else None)


def calculate_log_probs_and_entropy(
    logits,
    tokens,
    tp_group,
    with_entropy: bool = False,
    chunk_size: int = -1,
    log_prob_keep_mask=None,
    with_entropy_grad: bool = True,
):
    """Row-chunked driver around :class:`VocabParallelLogProbEntropy`.

    ``logits`` is ``[T, V/tp]``, ``tokens`` ``[T]``. ``chunk_size > 0`` bounds the
    fp32 scratch to ``chunk_size`` rows at a time.
    """
    logits = logits.contiguous()
    T = logits.size(0)
    if T == 0:
        return logits.new_zeros((0,)), (logits.new_zeros((0,)) if with_entropy else None)
    if chunk_size <= 0 or chunk_size >= T:
        return _logp_entropy_rows(logits, tokens, tp_group, with_entropy, with_entropy_grad, log_prob_keep_mask)
    lps, ents = [], []
    for s in range(0, T, chunk_size):
        e = min(s + chunk_size, T)
        km = None if log_prob_keep_mask is None else log_prob_keep_mask[s:e]
        lp, en = _logp_entropy_rows(logits[s:e], tokens[s:e], tp_group, with_entropy, with_entropy_grad, km)
        lps.append(lp)
        if en is not None:
            ents.append(en)
    return torch.cat(lps), (torch.cat(ents) if ents else None)


# ------------------------------------------------------------ returns / GAE
def get_grpo_returns(rewards: torch.Tensor, kl: list[torch.Tensor]) -> list[torch.Tensor]:
    """GRPO: every response token carries the sample's (already normalised) reward."""
    if not kl:
        return []
    lens = [k.numel() for k in kl]  # one broadcast over the concatenated batch, handed back as per-sample views
    flat = torch.repeat_interleave(rewards.to(kl[0].dtype), torch.as_tensor(lens, device=rewards.device), output_size=sum(lens))
    return list(torch.split(flat, lens))


def _suffix_scan_matrix(width: int, factor: float, device, dtype) -> torch.Tensor:
    """``M[i, j] = factor**(j-i)`` for ``j >= i`` else 0 (upper-triangular Toeplitz)."""
    idx = torch.arange(width, device=device)
    diff = idx[None, :] - idx[:, None]
    pw = torch.pow(torch.tensor(factor, device=device, dtype=torch.float64), diff.clamp_min(0).to(torch.float64))
    return torch.where(diff >= 0, pw, torch.zeros_like(pw)).to(dtype)


def chunked_discounted_returns(rewards: torch.Tensor, gamma: float, chunk: int = 128) -> torch.Tensor:
    """``G_t = r_t + gamma * G_{t+1}`` over ``[B, T]`` as a block scan.

    Each block of ``chunk`` steps is one ``[chunk, chunk]`` matmul; blocks are
    chained right-to-left through a carry, so the sequential depth is
    ``ceil(T / chunk)`` instead of ``T``.
    """
    B, T = rewards.shape
    if T == 0:
        return rewards.clone()
    out = torch.empty_like(rewards)
    M = _suffix_scan_matrix(chunk, gamma, rewards.device, rewards.dtype)
    carry_pw = torch.pow(
        torch.tensor(gamma, dtype=torch.float64, device=rewards.device),
        torch.arange(chunk, 0, -1, device=rewards.device, dtype=torch.float64),
    ).to(rewards.dtype)  # gamma^(chunk - i)
    carry = rewards.new_zeros(B)
    end = T
    while end > 0:
        start = max(0, end - chunk)
        w = end - start
        blk = rewards[:, start:end]
        Mw = M[chunk - w :, chunk - w :] if w < chunk else M
        res = blk @ Mw.T + carry[:, None] * carry_pw[chunk - w :][None, :]
        out[:, start:end] = res
        carry = res[:, 0]
        end = start
    return out


def vanilla_gae(rewards, values, gamma: float, lambd: float):
    """Reference O(T) GAE over padded ``[B, T]``; returns ``(advantages, returns)``."""
    B, T = rewards.shape
    adv = torch.zeros_like(rewards)
    last = rewards.new_zeros(B)
    for t in range(T - 1, -1, -1):
        nxt = values[:, t + 1] if t + 1 < T else rewards.new_zeros(B)
        delta = rewards[:, t] + gamma * nxt - values[:, t]
        last = delta + gamma * lambd * last
        adv[:, t] = last
    return adv, adv + values


def chunked_gae(rewards, values, gamma: float, lambd: float, chunk: int = 128):
    """GAE as a discounted suffix scan of TD residuals with factor ``gamma*lambda``."""
    nxt = torch.cat([values[:, 1:], values.new_zeros(values.size(0), 1)], dim=1)
    deltas = rewards + gamma * nxt - values
    adv = chunked_discounted_returns(deltas, gamma * lambd, chunk)
    return adv, adv + values


def _cp_full(local, total_len, resp_len):
    if mpu.get_context_parallel_world_size() == 1:
        return local
    from slime_b200.backends.train.cp_utils import all_gather_with_cp

    return all_gather_with_cp(local, total_len, resp_len)


def _cp_local(full, total_len, resp_len):
    if mpu.get_context_parallel_world_size() == 1:
        return full
    from slime_b200.backends.train.cp_utils import slice_log_prob_with_cp

    return slice_log_prob_with_cp(full, total_len, resp_len)


def _pad_stack(seqs: list[torch.Tensor]) -> torch.Tensor:
    width = max(s.numel() for s in seqs)
    out = seqs[0].new_zeros(len(seqs), width)
    for i, s in enumerate(seqs):
        out[i, : s.numel()] = s
    return out


def get_reinforce_plus_plus_returns(
    rewards: torch.Tensor,
    kl: list[torch.Tensor],
    loss_masks: list[torch.Tensor],
    response_lengths: list[int],
    total_lengths: list[int],
    kl_coef: float,
    gamma: float,
) -> list[torch.Tensor]:
    """REINFORCE++: token reward ``-kl_coef * kl`` with the scalar reward added at
    the last unmasked token, then discounted returns. CP-aware: works on the
    full response and re-slices to the local chunks."""
    token_rewards = []
    for i, k in enumerate(kl):
        full_kl = _cp_full(k, total_lengths[i], response_lengths[i])
        m = loss_masks[i]
        assert m.sum().item() > 0, f"Sequence at index {i} is fully masked."
        r = -kl_coef * full_kl * m
        last = int(torch.nonzero(m, as_tuple=True)[0][-1])
        r[last] = r[last] + rewards[i]
        token_rewards.append(r)
    if not token_rewards:
        return []
    G = chunked_discounted_returns(_pad_stack(token_rewards), gamma)
    return [
        _cp_local(G[i, : token_rewards[i].numel()], total_lengths[i], response_lengths[i])
        for i in range(len(token_rewards))
    ]


def get_reinforce_plus_plus_baseline_advantages(
    rewards: torch.Tensor,
    kl: list[torch.Tensor],
    loss_masks: list[torch.Tensor],
    kl_coef: float,
) -> list[torch.Tensor]:
    """REINFORCE++-baseline: ``(r - group mean)`` broadcast per token minus the KL penalty."""
    if not kl:
        return []
    lens = [k.numel() for k in kl]
    flat = torch.repeat_interleave(rewards.to(kl[0].dtype), torch.as_tensor(lens, device=rewards.device), output_size=sum(lens))
    return list(torch.split(flat - kl_coef * torch.cat(kl), lens))


def get_advantages_and_returns_batch(
    total_lengths,
    response_lengths,
    values_list,
    rewards_list,
    gamma,
    lambd,
    chunked: bool = True,
):
    """Batched GAE over ragged per-sample tensors (CP-aware)."""
    with torch.no_grad():
        n = len(response_lengths)
        assert n == len(values_list) == len(rewards_list)
        full_v = [_cp_full(v, t, r) for v, t, r in zip(values_list, total_lengths, response_lengths)]
        full_r = [_cp_full(x, t, r) for x, t, r in zip(rewards_list, total_lengths, response_lengths)]
        V, R = _pad_stack(full_v), _pad_stack(full_r)
        # GAE over a padded row is exact because padded rewards/values are zero and
        # lie to the right of the real tokens.
        adv, ret = (chunked_gae if chunked else vanilla_gae)(R, V, gamma, lambd)
        advs, rets = [], []
        for i in range(n):
            L = full_v[i].numel()
            advs.append(_cp_local(adv[i, :L], total_lengths[i], response_lengths[i]))
            rets.append(_cp_local(ret[i, :L], total_lengths[i], response_lengths[i]))
        return advs, rets
