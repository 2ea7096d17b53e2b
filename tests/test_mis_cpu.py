"""Mismatch-correction weights against a plain per-sequence restatement of the definitions."""

import math
from argparse import Namespace

import pytest
import torch

from slime_b200.utils import mis


def _args(**kw):
    base = dict(use_tis=True, tis_level="token", tis_mode="truncate", tis_lower_bound=0.5, tis_upper_bound=2.0, use_rs=False,
                rs_level="token", rs_lower_bound=None, rs_upper_bound=None, rs_veto_threshold=None, tis_batch_normalize=False)
    base.update(kw)
    return Namespace(**base)


def _data(seed=0):
    g = torch.Generator().manual_seed(seed)
    lens = [5, 1, 9, 4]
    train = [torch.randn(n, generator=g) * 0.5 - 1 for n in lens]
    roll = [t + torch.randn(t.shape, generator=g) * 0.6 for t in train]
    masks = [(torch.rand(n, generator=g) > 0.25).float() for n in lens]
    masks[1][:] = 1
    return train, roll, masks


def _level(d, m, level):
    if level == "token":
        return d
    s = (d * m).sum()
    return (s if level == "sequence" else s / m.sum().clamp_min(1)).expand_as(d)


def _reference(a, train, roll, masks):
    lower = a.tis_lower_bound if a.tis_lower_bound is not None else 1 / a.tis_upper_bound
    rs_lo = a.rs_lower_bound if a.rs_lower_bound is not None else lower
    rs_hi = a.rs_upper_bound if a.rs_upper_bound is not None else a.tis_upper_bound
    ws, ms = [], []
    for t, r, m in zip(train, roll, masks):
        d = t - r
        w = torch.exp(_level(d, m, a.tis_level).clamp(-20, 20))
        nm = m.clone()
        if a.tis_mode == "truncate":
            w = w.clamp(max=a.tis_upper_bound)
        elif a.tis_mode == "clip":
            w = w.clamp(lower, a.tis_upper_bound)
        else:
            nm = nm * ((w >= lower) & (w <= a.tis_upper_bound)).float()
        if a.use_rs:
            rw = torch.exp(_level(d, m, a.rs_level).clamp(-20, 20))
            nm = nm * ((rw >= rs_lo) & (rw <= rs_hi)).float()
            if a.rs_veto_threshold is not None and bool(((d < math.log(a.rs_veto_threshold)) & (m > 0)).any()):
                nm = nm * 0
        ws.append(w)
        ms.append(nm)
    if a.tis_batch_normalize:
        if a.tis_level == "token":
            mean = sum((w * m).sum() for w, m in zip(ws, masks)) / sum(m.sum() for m in masks)
        else:
            mean = sum((w * m).sum() / m.sum().clamp_min(1) for w, m in zip(ws, masks)) / len(ws)
        ws = [w / mean for w in ws]
    return ws, ms


@pytest.mark.parametrize("cfg", [
    dict(), dict(tis_mode="clip"), dict(tis_mode="mask"), dict(tis_level="sequence", tis_batch_normalize=True),
    dict(tis_level="geometric", tis_lower_bound=0.9, tis_upper_bound=1.1, tis_mode="mask"),
    dict(use_rs=True, rs_level="sequence", rs_veto_threshold=0.3, tis_batch_normalize=True),
    dict(use_rs=True, rs_lower_bound=0.8, rs_upper_bound=1.5, tis_lower_bound=None),
])
def test_weights_and_masks_match_definitions(cfg):
    a = _args(**cfg)
    train, roll, masks = _data()
    w, m, metrics = mis.compute_mis_weights(a, train_log_probs=train, rollout_log_probs=roll, loss_masks=masks)
    rw, rm = _reference(a, train, roll, masks)
    for x, y in zip(w, rw):
        torch.testing.assert_close(x, y, rtol=1e-5, atol=1e-6)
    for x, y in zip(m, rm):
        assert torch.equal(x, y)
    assert all(not x.requires_grad for x in w) and all(len(v) == len(train) for v in metrics.values())
    assert all(v[2].shape == train[2].shape for v in metrics.values())


def test_metrics_only_and_cp_entry():
    train, roll, masks = _data(3)
    w, m, metrics = mis.compute_mis_weights(_args(use_tis=False), train_log_probs=train, rollout_log_probs=roll, loss_masks=masks)
    assert w is None and m is masks
    t, r, mk = train[2], roll[2], masks[2]
    torch.testing.assert_close(metrics["kl"][2], r - t)
    torch.testing.assert_close(metrics["training_ppl"][2][0], torch.exp(-(t * mk).sum() / mk.sum()))
    rho = torch.exp(t - r)
    torch.testing.assert_close(metrics["chi2_token"][2][0], (rho**2 * mk).sum() / mk.sum() - 1)
    torch.testing.assert_close(metrics["chi2_seq"][2][0], torch.exp(2 * ((t - r) * mk).sum()) - 1)
    # the loss-side entry (context parallel size 1): flat tensors, prefixed metric names, weights applied to pg_loss
    from slime_b200.parallel import state as mpu

    if not mpu.model_parallel_is_initialized():
        mpu.initialize_model_parallel()
    lens = [x.numel() for x in train]
    pg = torch.ones(sum(lens))
    out, masks2, flat = mis.compute_mis_weights_with_cp(_args(), pg_loss=pg, train_log_probs=train, rollout_log_probs=roll,
                                                        loss_masks=masks, total_lengths=[n + 3 for n in lens], response_lengths=lens)
    torch.testing.assert_close(out, torch.exp(torch.cat(train) - torch.cat(roll)).clamp(max=2.0))
    assert "mis_kl" in flat and flat["mis_kl"].shape == pg.shape and len(masks2) == len(lens)
    import examples.train_infer_mismatch_helper.mis as shim

    assert shim.compute_mis_weights_with_cp is mis.compute_mis_weights_with_cp
