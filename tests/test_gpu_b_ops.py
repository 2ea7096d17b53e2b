"""Fused memory-bound / loss / sampling / paged-attention kernels against fp32 PyTorch references."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def close(a, b, atol, rtol=0.0):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    lim = atol + rtol * b.abs().max().item()
    assert err <= lim, f"max err {err} > {lim}"


@pytest.mark.parametrize("T,H", [(1, 896), (257, 896), (64, 2560), (33, 8192), (100, 128)])
def test_rmsnorm_fwd_bwd(kernels, T, H):
    from slime_b200 import ops
    from slime_b200.ops import reference

    torch.manual_seed(T + H)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    y, h = ops.rmsnorm(x, w, 1e-6, residual=r)
    yr, hr, _ = reference.rmsnorm(x.detach(), w.detach(), 1e-6, r.detach())
    close(y, yr, 2e-2, 1e-2)
    close(h, hr, 1e-2, 1e-2)
    gy, gh = torch.randn_like(y), torch.randn_like(h)
    torch.autograd.backward([y, h], [gy, gh])
    xf, rf, wf = (t.detach().float().requires_grad_(True) for t in (x, r, w))
    hh = xf + rf
    yy = hh * torch.rsqrt(hh.pow(2).mean(-1, keepdim=True) + 1e-6) * wf
    torch.autograd.backward([yy, hh], [gy.float(), gh.float()])
    close(x.grad, xf.grad, 3e-2, 2e-2)
    close(r.grad, rf.grad, 3e-2, 2e-2)
    close(w.grad, wf.grad, 5e-2, 2e-2)
    # without residual
    y2, h2 = ops.rmsnorm(x.detach(), w.detach(), 1e-6)
    close(y2, reference.rmsnorm(x.detach(), w.detach(), 1e-6)[0], 2e-2, 1e-2)


@pytest.mark.parametrize("D,Hq,Hkv,qknorm", [(64, 14, 2, False), (128, 32, 8, True), (128, 4, 4, False)])
def test_rope_qk(kernels, D, Hq, Hkv, qknorm):
    from slime_b200 import ops
    from slime_b200.ops import reference

    torch.manual_seed(D + Hq)
    T = 97
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    pos = torch.randint(0, 500, (T,), device="cuda", dtype=torch.int32)
    cs = ops.rope_cos_sin(512, D, 1e6, device="cuda")
    qn = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16).requires_grad_(True) if qknorm else None
    kn = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16).requires_grad_(True) if qknorm else None
    out = ops.rope_qk(qkv, pos, cs, Hq, Hkv, D, qn, kn, 1e-6)
    xf = qkv.detach().float().requires_grad_(True)
    qnf = qn.detach().float().requires_grad_(True) if qknorm else None
    knf = kn.detach().float().requires_grad_(True) if qknorm else None
    x3 = xf.view(T, Hq + 2 * Hkv, D)
    ref = torch.cat([reference.rope(x3[:, :Hq], pos, cs, qnf), reference.rope(x3[:, Hq:Hq + Hkv], pos, cs, knf),
                     x3[:, Hq + Hkv:]], 1).reshape(T, -1)  # fmt: skip
    close(out, ref, 3e-2, 1e-2)
    g = torch.randn_like(out)
    out.backward(g)
    ref.backward(g.float())
    close(qkv.grad, xf.grad, 5e-2, 2e-2)
    if qknorm:
        close(qn.grad, qnf.grad, 0.5, 3e-2)
        close(kn.grad, knf.grad, 0.5, 3e-2)


def test_swiglu_embedding_add(kernels):
    from slime_b200 import ops
    from slime_b200.ops import reference

    torch.manual_seed(3)
    gu = torch.randn(333, 2 * 4864, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    act = ops.swiglu(gu)
    close(act, reference.swiglu(gu.detach()), 2e-2, 1e-2)
    g = torch.randn_like(act)
    act.backward(g)
    gf = gu.detach().float().requires_grad_(True)
    F = 4864
    (torch.nn.functional.silu(gf[:, :F]) * gf[:, F:]).backward(g.float())
    close(gu.grad, gf.grad, 3e-2, 2e-2)
    table = torch.randn(1000, 896, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, 1000, (77,), device="cuda")
    close(ops.embedding(ids, table), table[ids], 0)
    # vocab-parallel slice: ids outside [lo, hi) give zeros
    out = ops.embedding(ids, table[200:600].contiguous(), 200)
    exp = torch.where(((ids >= 200) & (ids < 600))[:, None], table[ids], torch.zeros_like(table[ids]))
    close(out, exp, 0)


def test_adam_and_sqnorm(kernels):
    from slime_b200.backends.train.buffers import FlatBuffer
    from slime_b200.backends.train.optimizer import DistributedOptimizer
    from slime_b200.ops import reference

    torch.manual_seed(4)
    ps = [torch.nn.Parameter(torch.randn(1000, 37, device="cuda").to(torch.bfloat16)),
          torch.nn.Parameter(torch.randn(513, device="cuda").to(torch.bfloat16))]  # fmt: skip
    buf = FlatBuffer(ps, ["a", "b"], None, 1, 0, "cuda")
    opt = DistributedOptimizer([buf], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, clip_grad=1.0)
    master = [p.detach().float().clone() for p in ps]
    m = [torch.zeros_like(x) for x in master]
    v = [torch.zeros_like(x) for x in master]
    for step in range(1, 4):
        grads = [torch.randn_like(x) * 3 for x in master]
        for p, g in zip(ps, grads):
            p.main_grad.copy_(g)
        norm = torch.sqrt(sum(g.pow(2).sum() for g in grads))
        coef = min(1.0, 1.0 / (norm.item() + 1e-6))
        gn = opt.step()
        assert abs(gn.item() - norm.item()) / norm.item() < 1e-4
        for i in range(2):
            reference.adam_step(master[i], m[i], v[i], grads[i], 1e-2, 0.9, 0.95, 1e-8, 0.1, step, clip_coef=coef)
    for p, ref in zip(ps, master):
        close(p, ref.to(torch.bfloat16), 2e-2, 1e-2)
    s, e = buf.offsets[0]
    close(opt.state[0]["master"][s:e].view(1000, 37), master[0], 1e-4, 1e-4)


def test_logprob_entropy_and_fused_policy_loss(kernels):
    from slime_b200.backends.train import fused_loss

    torch.manual_seed(5)
    R, H, V = 700, 256, 5000
    h = (torch.randn(R, H, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(V, H, device="cuda") * 0.1).to(torch.bfloat16)
    tg = torch.randint(0, V, (R,), device="cuda", dtype=torch.int32)
    lp, ent = fused_loss.logprob_entropy_rows(h, w, tg, inv_temperature=1 / 0.8, chunk=256)
    z = (h.float() @ w.float().t()) / 0.8
    lsm = torch.log_softmax(z, -1)
    close(lp, lsm.gather(-1, tg.long()[:, None]).squeeze(-1), 2e-3)
    close(ent, -(lsm.exp() * lsm).sum(-1), 2e-3)

    # fused forward+backward vs autograd through the fp32 reference
    for cispo, ecoef in ((False, 0.0), (False, 0.01), (True, 0.0)):
        hq = h.clone().requires_grad_(True)
        wq = w.clone().requires_grad_(True)
        old = (lp + 0.3 * torch.randn(R, device="cuda")).contiguous()
        adv = torch.randn(R, device="cuda")
        wt = (torch.rand(R, device="cuda") > 0.2).float() / R
        loss, logp, entropy, metrics = fused_loss.fused_policy_loss(
            hq, wq, tg, old, adv, wt, eps_clip=0.2, eps_clip_high=0.28, eps_clip_c=3.0 if not cispo else None, cispo=cispo,
            entropy_coef=ecoef, temperature=0.8, chunk=256,
        )  # fmt: skip
        loss.backward()
        hr = h.float().clone().requires_grad_(True)
        wr = w.float().clone().requires_grad_(True)
        ref_loss, *_ = fused_loss._reference_policy_loss(hr, wr, tg.long(), old, adv, wt, 0.2, 0.28, 3.0 if not cispo else None,
                                                         cispo, ecoef, 0.8, None, 0)  # fmt: skip
        ref_loss.backward()
        assert abs(loss.item() - ref_loss.item()) < 2e-3 * max(1.0, abs(ref_loss.item())), (loss.item(), ref_loss.item())
        close(hq.grad, hr.grad, 1e-4, 3e-2)
        close(wq.grad, wr.grad, 1e-4, 3e-2)


def test_pg_loss_kernel(kernels):
    from slime_b200.ops import _lib, reference

    torch.manual_seed(6)
    T = 5000
    lp = -torch.rand(T, device="cuda") * 3
    old = lp + 0.4 * torch.randn(T, device="cuda")
    adv = torch.randn(T, device="cuda")
    w = torch.rand(T, device="cuda")
    for mode, eps_c in ((0, 0.0), (0, 3.0), (1, 0.0)):
        g = torch.empty(T, device="cuda")
        acc = torch.zeros(4, device="cuda")
        rc = _lib.lib().sb_pg_loss(lp.data_ptr(), old.data_ptr(), adv.data_ptr(), w.data_ptr(), None, g.data_ptr(), None,
                                   acc.data_ptr(), T, 0.2, 0.28, eps_c, mode, _lib.stream())  # fmt: skip
        assert rc == 0
        tot, clip, kl, ws, gref = reference.pg_loss(lp, old, adv, w, 0.2, 0.28, eps_c if eps_c > 1 else None, mode)
        close(acc[0], tot, 1e-2, 1e-4)
        close(acc[1], clip, 1e-2, 1e-4)
        close(acc[2], kl, 1e-2, 1e-4)
        close(g, gref, 1e-5, 1e-4)


def test_sampling(kernels):
    from slime_b200 import ops
    from slime_b200.ops import reference

    torch.manual_seed(7)
    B, V = 64, 151936
    logits = torch.randn(B, V, device="cuda") * 2
    temp = torch.full((B,), 0.0, device="cuda")
    tok, lp, _, _ = ops.sample(logits, temp)
    assert torch.equal(tok.long(), logits.argmax(-1))
    close(lp, torch.log_softmax(logits, -1).gather(-1, tok.long()[:, None]).squeeze(-1), 1e-4)

    # unfiltered: log-prob is the temperature-scaled log-softmax of the drawn token; draws follow the distribution
    small = torch.randn(1, 50, device="cuda").repeat(4096, 1).contiguous()
    temp = torch.full((4096,), 0.7, device="cuda")
    seeds = torch.arange(4096, device="cuda", dtype=torch.int64) * 7919 + 13
    pos = torch.zeros(4096, device="cuda", dtype=torch.int32)
    tok, lp, _, _ = ops.sample(small, temp, seeds=seeds, positions=pos)
    lsm = torch.log_softmax(small[0] / 0.7, -1)
    close(lp, lsm[tok.long()], 1e-4)
    freq = torch.bincount(tok.long(), minlength=50).float() / 4096
    assert (freq - lsm.exp()).abs().max().item() < 0.03
    tok2, _, _, _ = ops.sample(small, temp, seeds=seeds, positions=pos)
    assert torch.equal(tok, tok2), "same seed and position must reproduce the draw"
    tok3, _, _, _ = ops.sample(small, temp, seeds=seeds, positions=pos + 1)
    assert not torch.equal(tok, tok3)

    # top-k / top-p: kept set equals the reference definition, log-prob renormalised over it
    B = 32
    logits = torch.randn(B, 4000, device="cuda") * 3
    temp = torch.ones(B, device="cuda")
    tk = torch.full((B,), 50, device="cuda", dtype=torch.int32)
    tp = torch.full((B,), 0.9, device="cuda")
    mp = torch.zeros(B, device="cuda")
    tok, lp, kept, cnt = ops.sample(logits, temp, tk, tp, mp, seeds=seeds[:B].contiguous(), positions=pos[:B].contiguous(), kept_cap=4000)
    probs = torch.softmax(logits, -1)
    keep = reference.topp_topk_keep_mask(probs, 50, 0.9)
    for b in range(B):
        ours = set(kept[b, : cnt[b]].tolist())
        ref = set(torch.nonzero(keep[b]).flatten().tolist())
        assert len(ours ^ ref) <= 1, (b, len(ours), len(ref))  # ties at the cut-off may differ by one token
        assert tok[b].item() in ours
        mass = probs[b][list(ours)].sum()
        assert abs(lp[b].item() - math.log(probs[b, tok[b]].item() / mass.item())) < 1e-3


@pytest.mark.parametrize("Hq,Hkv,D", [(14, 2, 64), (32, 8, 128), (16, 4, 128)])
def test_paged_decode_attention(kernels, Hq, Hkv, D):
    from slime_b200 import ops
    from slime_b200.ops import reference

    torch.manual_seed(Hq)
    B, ps, pages = 9, 16, 256
    kc = torch.randn(pages * ps, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(pages * ps, Hkv, D, device="cuda", dtype=torch.bfloat16)
    lens = torch.tensor([1, 15, 16, 17, 100, 333, 64, 257, 300], device="cuda", dtype=torch.int32)
    bt = torch.zeros(B, 24, device="cuda", dtype=torch.int32)
    perm = torch.randperm(pages)[: B * 24].view(B, 24).to(torch.int32).cuda()
    bt.copy_(perm)
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    ref = reference.paged_decode_attention(q, kc, vc, bt, lens, ps)
    for splits in (1, 4):
        out = ops.paged_decode_attention(q, kc, vc, bt, lens, ps, splits=splits)
        close(out, ref, 2e-2, 1e-2)
    # kv_write puts rows where the table says
    k_new = torch.randn(B, Hkv * D, device="cuda", dtype=torch.bfloat16)
    v_new = torch.randn(B, Hkv * D, device="cuda", dtype=torch.bfloat16)
    slots = (bt[:, 0] * ps + 3).to(torch.int32)
    ops.kv_write(k_new, v_new, slots, kc, vc)
    close(kc[slots.long()].reshape(B, -1), k_new, 0)
    close(vc[slots.long()].reshape(B, -1), v_new, 0)


def test_quantisers_and_router(kernels):
    from slime_b200 import ops
    from slime_b200.ops import reference

    torch.manual_seed(8)
    x = torch.randn(300, 520, device="cuda", dtype=torch.bfloat16) * 3
    x[:128, :128] = 0  # an all-zero block must not produce NaN
    q, s = ops.block_fp8_quant(x)
    qr, sr = reference.block_fp8_quant(x)
    close(s, sr, 1e-7, 1e-5)
    assert torch.isfinite(q.float()).all()
    deq = ops.block_fp8_dequant(q, s)
    close(deq, reference.block_fp8_dequant(qr, sr), 1e-2, 7e-2)
    assert deq[:128, :128].abs().max().item() == 0
    assert (deq.float() - x.float()).abs().max().item() <= 0.07 * x.float().abs().max().item()
    q2, s2 = ops.block_fp8_quant(x, pow2_scale=True)
    assert torch.all(torch.log2(s2) == torch.log2(s2).round())

    w = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16)
    for group, sym in (((1, 32), True), ((32, 1), True), ((1, 32), False), ((16, 16), True)):
        y, sc, z = ops.fake_int4_quant(w, group, sym)
        yr, scr, zr = reference.fake_int4(w, group, sym)
        close(sc, scr, 1e-6, 1e-4)
        assert ((y.float() - yr.float()).abs() > 1e-2).float().mean().item() < 0.01  # rare rint ties at bf16 precision

    xr = torch.randn(37, 2048, device="cuda", dtype=torch.bfloat16)
    wr = torch.randn(128, 2048, device="cuda", dtype=torch.bfloat16)
    out = ops.router_gemm(xr, wr)
    close(out, xr.float() @ wr.float().t(), 1e-2, 1e-4)
    # batch invariance: a token's logits do not depend on which other tokens share the launch
    out1 = ops.router_gemm(xr[5:6].contiguous(), wr)
    assert torch.equal(out1[0], out[5])


@pytest.mark.parametrize("Hq,Hkv,D,norm", [(14, 2, 64, False), (8, 2, 128, True)])
def test_rope_kv_write_matches_separate_ops(kernels, Hq, Hkv, D, norm):
    """The fused inference kernel against fp32 PyTorch: rotated q / k in place, k / v rows in their cache slots."""
    from slime_b200 import ops
    from slime_b200.ops import reference

    torch.manual_seed(5)
    T, slots_n = 37, 64
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
    pos = torch.randint(0, 500, (T,), device="cuda", dtype=torch.int32)
    cs = ops.rope_cos_sin(512, D, 10000.0, device="cuda")
    slots = torch.randperm(slots_n, device="cuda")[:T].to(torch.int32)
    slots[3] = -1  # a padding row: rotated in place, not written to the cache
    qw = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16) if norm else None
    kw = (1 + 0.1 * torch.randn(D, device="cuda")).to(torch.bfloat16) if norm else None
    kc = torch.zeros(slots_n, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    x = qkv.float().view(T, Hq + 2 * Hkv, D)
    q_ref = reference.rope(x[:, :Hq], pos, cs, qw.float() if norm else None, 1e-6)
    k_ref = reference.rope(x[:, Hq : Hq + Hkv], pos, cs, kw.float() if norm else None, 1e-6)
    v_ref = x[:, Hq + Hkv :]
    out = ops.rope_kv_write(qkv.clone(), pos, cs, slots, kc, vc, Hq, Hkv, D, qw, kw, 1e-6).view(T, Hq + 2 * Hkv, D)
    torch.cuda.synchronize()
    torch.testing.assert_close(out[:, :Hq].float(), q_ref.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out[:, Hq : Hq + Hkv].float(), k_ref.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out[:, Hq + Hkv :].float(), v_ref)
    ok = slots >= 0
    torch.testing.assert_close(kc[slots[ok].long()].float(), k_ref.float()[ok], rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(vc[slots[ok].long()].float(), v_ref[ok])
    unused = torch.ones(slots_n, dtype=torch.bool, device="cuda")
    unused[slots[ok].long()] = False
    assert (kc[unused] == 0).all() and (vc[unused] == 0).all()
