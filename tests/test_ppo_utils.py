import pytest
import torch

from slime_b200.utils.ppo_utils import (
    calculate_log_probs_and_entropy,
    chunked_discounted_returns,
    chunked_gae,
    compute_approx_kl,
    compute_cispo_loss,
    compute_gspo_kl,
    compute_opsm_mask,
    compute_policy_loss,
    vanilla_gae,
)


def test_policy_loss_values_and_dual_clip():
    kl = torch.tensor([0.0, -0.5, 0.5, -2.0])
    adv = torch.tensor([1.0, 1.0, -1.0, -1.0])
    loss, clip = compute_policy_loss(kl, adv, 0.2, 0.2)
    ratio = torch.exp(-kl)
    exp = torch.maximum(-ratio * adv, -ratio.clamp(0.8, 1.2) * adv)
    assert torch.allclose(loss, exp)
    assert clip.tolist() == [0.0, 1.0, 1.0, 0.0]
    loss_c, _ = compute_policy_loss(kl, adv, 0.2, 0.2, eps_clip_c=3.0)
    assert loss_c[3].item() == pytest.approx(3.0)  # ratio e^2 ~ 7.39 capped at c * |A|
    assert loss_c[:2].tolist() == loss[:2].tolist()
    with pytest.raises(AssertionError):
        compute_policy_loss(kl, adv, 0.2, 0.2, eps_clip_c=0.5)


def test_cispo_stop_gradient():
    lp = torch.tensor([-1.0, -2.0, -0.5], requires_grad=True)
    old = torch.tensor([-1.2, -1.0, -0.5])
    adv = torch.tensor([1.0, -1.0, 2.0])
    loss, clip = compute_cispo_loss(old - lp, lp, adv, 0.2, 0.3)
    loss.sum().backward()
    ratio = torch.exp(lp.detach() - old).clamp(0.8, 1.3)
    assert torch.allclose(lp.grad, -ratio * adv)  # gradient flows through log-probs only
    assert clip.tolist() == [0.0, 1.0, 0.0]


def test_kl_estimators():
    a, b = torch.tensor([-1.0, -2.0]), torch.tensor([-1.5, -1.0])
    d = a - b
    assert torch.allclose(compute_approx_kl(a, b, "k1"), d)
    assert torch.allclose(compute_approx_kl(a, b, "k2"), d * d / 2)
    assert torch.allclose(compute_approx_kl(a, b, "k3"), torch.exp(-d) - 1 + d)
    assert compute_approx_kl(torch.tensor([-30.0]), torch.tensor([0.0]), "low_var_kl").item() == 10.0
    w = torch.tensor([2.0, 0.5])
    assert torch.allclose(compute_approx_kl(a, b, "k1", importance_ratio=w), w * d)
    with pytest.raises(ValueError):
        compute_approx_kl(a, b, "k9")


def test_gspo_and_opsm():
    lp = [torch.tensor([-1.0, -1.0]), torch.tensor([-2.0, -2.0, -2.0])]
    old = [torch.tensor([-1.5, -0.5]), torch.tensor([-1.0, -1.0, -1.0])]
    masks = [torch.ones(2), torch.tensor([1.0, 1.0, 0.0])]
    kl = compute_gspo_kl(lp, old, lp, masks)
    assert torch.allclose(kl, torch.tensor([0.0, 0.0, 1.0, 1.0, 1.0]))
    from argparse import Namespace

    adv = [torch.tensor([-1.0, 1.0]), torch.tensor([-1.0, -1.0, 1.0])]
    mask, frac = compute_opsm_mask(Namespace(opsm_delta=0.5), lp, old, adv, masks)
    assert mask.tolist() == [1.0, 1.0, 0.0, 0.0, 1.0]
    assert frac.item() == pytest.approx(1.0)


@pytest.mark.parametrize("T", [1, 7, 128, 129, 300])
def test_chunked_scans_match_loops(T):
    torch.manual_seed(T)
    r, v = torch.randn(3, T, dtype=torch.float64), torch.randn(3, T, dtype=torch.float64)
    a, b = vanilla_gae(r, v, 0.97, 0.9)
    c, d = chunked_gae(r, v, 0.97, 0.9)
    assert torch.allclose(a, c, atol=1e-9) and torch.allclose(b, d, atol=1e-9)
    g = chunked_discounted_returns(r, 0.9, chunk=16)
    ref = torch.zeros_like(r)
    run = torch.zeros(3, dtype=torch.float64)
    for t in range(T - 1, -1, -1):
        run = r[:, t] + 0.9 * run
        ref[:, t] = run
    assert torch.allclose(g, ref, atol=1e-9)


def test_logprob_entropy_vs_unfused_reference_with_grads():
    torch.manual_seed(0)
    z = torch.randn(9, 23, dtype=torch.float64, requires_grad=True)
    t = torch.randint(0, 23, (9,))
    lp, ent = calculate_log_probs_and_entropy(z, t, None, with_entropy=True, chunk_size=4)
    z2 = z.detach().clone().requires_grad_(True)
    lsm = torch.log_softmax(z2.float(), -1)
    lp_r = lsm.gather(-1, t[:, None]).squeeze(-1)
    ent_r = -(lsm.exp() * lsm).sum(-1)
    assert torch.allclose(lp, lp_r, atol=1e-6) and torch.allclose(ent, ent_r, atol=1e-6)
    gw, ge = torch.randn(9), torch.randn(9)
    (lp * gw + ent * ge).sum().backward()
    (lp_r * gw + ent_r * ge).sum().backward()
    assert torch.allclose(z.grad, z2.grad, atol=1e-6)


def test_logprob_keep_mask_forces_target_and_keeps_entropy_unmasked():
    torch.manual_seed(1)
    z = torch.randn(4, 10)
    t = torch.tensor([0, 3, 5, 9])
    keep = torch.zeros(4, 10, dtype=torch.bool)
    keep[:, :3] = True  # targets 3, 5, 9 are outside the mask and must be force-kept
    lp, ent = calculate_log_probs_and_entropy(z, t, None, with_entropy=True, log_prob_keep_mask=keep)
    for i in range(4):
        km = keep[i].clone()
        km[t[i]] = True
        ref = torch.log_softmax(z[i].masked_fill(~km, float("-inf")), -1)[t[i]]
        assert lp[i].item() == pytest.approx(ref.item(), abs=1e-6)
    lsm = torch.log_softmax(z, -1)
    assert torch.allclose(ent, -(lsm.exp() * lsm).sum(-1), atol=1e-6)


def test_opd_subtracts_reverse_kl_and_rejects_short_teacher():
    from argparse import Namespace

    from slime_b200.backends.train.loss import apply_opd_kl_to_advantages

    args = Namespace(opd_kl_coef=0.5)
    adv = [torch.zeros(3), torch.ones(2)]
    student = [torch.tensor([-1.0, -2.0, -3.0]), torch.tensor([-0.5, -0.5])]
    data = {"teacher_log_probs": [[-9.0, -1.0, -1.0, -1.0], [-1.5, -0.5]]}  # a longer teacher vector is right-aligned
    apply_opd_kl_to_advantages(args, data, adv, student)
    assert torch.allclose(adv[0], torch.tensor([0.0, 0.5, 1.0])) and torch.allclose(adv[1], torch.tensor([0.5, 1.0]))
    assert torch.allclose(data["opd_reverse_kl"][1], torch.tensor([1.0, 0.0]))
    with pytest.raises(ValueError, match="teacher log-probs cover 1 tokens"):
        apply_opd_kl_to_advantages(args, {"teacher_log_probs": [[-1.0]]}, [torch.zeros(2)], [torch.zeros(2)])
