"""BASELINE config 0: CPU-only GRPO loss path, seed 0, against closed-form restatements of the math."""

import math

import torch

from slime_b200.utils.ppo_utils import compute_policy_loss


def _workload(seed=0):
    g = torch.Generator().manual_seed(seed)
    n_prompts, n_samples = 8, 8
    lens = torch.randint(16, 257, (n_prompts * n_samples,), generator=g).tolist()
    old = [(-1.5 + 0.5 * torch.randn(L, generator=g)).clamp(max=0.0) for L in lens]
    new = [o + 0.05 * torch.randn(o.shape, generator=g) for o in old]
    rewards = (torch.rand(n_prompts * n_samples, generator=g) < 0.5).float()
    masks = [torch.ones(L) for L in lens]
    return lens, old, new, rewards, masks, n_samples


def grpo_loss_cpu(seed=0, per_token=False):
    from slime_b200.backends.train.cp_utils import get_sum_of_sample_mean

    lens, old, new, rewards, masks, n = _workload(seed)
    r = rewards.view(-1, n)
    adv_scalar = ((r - r.mean(-1, keepdim=True)) / (r.std(-1, keepdim=True) + 1e-6)).flatten()
    adv = torch.cat([torch.full((L,), float(a)) for L, a in zip(lens, adv_scalar)])
    kl = torch.cat(old) - torch.cat(new)
    loss, clip = compute_policy_loss(kl, adv, 0.2, 0.28)
    reducer = get_sum_of_sample_mean(lens, lens, masks, None, per_token)
    denom = sum(lens) if per_token else len(lens)
    return reducer(loss) / denom, reducer(clip) / denom, reducer(kl) / denom, (lens, old, new, adv_scalar)


def test_config0_matches_manual_loop():
    loss, clipfrac, approx_kl, (lens, old, new, adv) = grpo_loss_cpu(0)
    tot_l = tot_c = tot_k = 0.0
    for L, o, nw, a in zip(lens, old, new, adv.tolist()):
        sl = sc = sk = 0.0
        for t in range(L):
            ratio = math.exp(float(nw[t] - o[t]))
            l1 = -ratio * a
            l2 = -min(max(ratio, 0.8), 1.28) * a
            sl += max(l1, l2)
            sc += 1.0 if l2 > l1 else 0.0
            sk += float(o[t] - nw[t])
        tot_l += sl / L
        tot_c += sc / L
        tot_k += sk / L
    n = len(lens)
    assert abs(loss.item() - tot_l / n) < 1e-5
    assert abs(clipfrac.item() - tot_c / n) < 1e-6
    assert abs(approx_kl.item() - tot_k / n) < 1e-6
    assert 0.0 <= clipfrac.item() < 0.2 and abs(approx_kl.item()) < 0.05


def test_config0_is_deterministic_and_per_token_mode():
    a = grpo_loss_cpu(0)[0].item()
    b = grpo_loss_cpu(0)[0].item()
    assert a == b
    lt, ct, kt, _ = grpo_loss_cpu(0, per_token=True)
    assert torch.isfinite(lt) and 0 <= ct.item() <= 1


def test_group_normalisation_through_train_data():
    """Same numbers through the framework path: Sample -> post_process_rewards."""
    from slime_b200.rollout.train_data import post_process_rewards
    from slime_b200.utils.arguments import namespace_from_dict
    from slime_b200.utils.types import Sample

    lens, old, new, rewards, masks, n = _workload(0)
    args = namespace_from_dict(dict(rollout_batch_size=8, n_samples_per_prompt=8, num_rollout=1))
    samples = [Sample(index=i, reward=float(r), response_length=L, tokens=[0] * (L + 4)) for i, (r, L) in enumerate(zip(rewards, lens))]
    raw, normed = post_process_rewards(args, samples)
    r = rewards.view(-1, n)
    expect = ((r - r.mean(-1, keepdim=True)) / (r.std(-1, keepdim=True) + 1e-6)).flatten()
    assert torch.allclose(torch.tensor(normed), expect, atol=1e-6)
    assert raw == [float(x) for x in rewards]
