"""The sm_100a flash-attention kernels (forward, dK/dV pass, dQ pass) against fp32 PyTorch."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, seg, scale):
    from slime_b200.ops.attention import _reference_segments

    return _reference_segments(q.float(), k.float(), v.float(), seg, scale)


def _close(got, want, what, atol, rtol):
    err = (got.float() - want.float()).abs()
    bound = atol + rtol * want.float().abs()
    bad = err > bound
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} elements off, worst {float(err.max()):.4g} (ref scale {float(want.abs().max()):.3g})"


CASES = [
    # lens, Hq, Hkv, D
    ([1, 127, 128, 129, 300], 14, 2, 64),
    ([1, 127, 128, 129, 300], 8, 2, 128),
    ([4097], 4, 1, 128),
    ([515, 64, 2000], 14, 2, 64),
    ([96, 257], 32, 8, 128),
]


@pytest.mark.parametrize("lens,Hq,Hkv,D", CASES)
def test_flash_forward_backward_match_fp32(kernels, lens, Hq, Hkv, D):
    from slime_b200.ops import _lib, attention

    torch.manual_seed(sum(lens) + Hq)
    T = sum(lens)
    pad = (-T) % 128
    Tp = T + pad
    dev = "cuda"
    # one packed qkv buffer, as the trainer has it (q / k / v are strided views)
    qkv = (torch.randn(Tp, (Hq + 2 * Hkv) * D, device=dev) * 0.8).to(torch.bfloat16)
    x3 = qkv.view(Tp, Hq + 2 * Hkv, D)
    q, k, v = x3[:, :Hq], x3[:, Hq : Hq + Hkv], x3[:, Hq + Hkv :]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)) + ([Tp] if pad else []), dtype=torch.int32, device=dev)
    seg = attention.segments_from_cu_seqlens(cu)
    scale = 1.0 / math.sqrt(D)
    out, lse = attention.flash_fwd(q, k, v, seg, scale)
    torch.cuda.synchronize()
    _lib.check_status(dev)
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = _ref(qf, kf, vf, seg.cpu(), scale)
    _close(out, ref, "out", 2e-2, 2e-2)
    # lse against the reference, valid rows only
    for (qo, ql, ko, kl) in seg.tolist():
        s = torch.einsum("thd,shd->hts", qf[qo : qo + ql].detach(), kf[ko : ko + kl].detach().repeat_interleave(Hq // Hkv, 1)) * scale
        m = torch.ones(ql, kl, dtype=torch.bool, device=dev).tril(diagonal=kl - ql)
        want = torch.logsumexp(s.masked_fill(~m, float("-inf")), -1)
        _close(lse[:, qo : qo + ql], want, "lse", 2e-2, 1e-2)
    d_o = (torch.randn(Tp, Hq, D, device=dev) * 0.5).to(torch.bfloat16)
    ref.backward(d_o.float())
    dqkv = torch.zeros_like(qkv)
    d3 = dqkv.view(Tp, Hq + 2 * Hkv, D)
    attention.flash_bwd(q, k, v, out, d_o, lse, seg, scale, dq=d3[:, :Hq], dk=d3[:, Hq : Hq + Hkv], dv=d3[:, Hq + Hkv :])
    torch.cuda.synchronize()
    _lib.check_status(dev)
    # gradients are sums over up to thousands of bf16-rounded products: absolute floor scaled by the tensor's size
    for name, got, want in (("dq", d3[:, :Hq], qf.grad), ("dk", d3[:, Hq : Hq + Hkv], kf.grad), ("dv", d3[:, Hq + Hkv :], vf.grad)):
        _close(got, want, name, 3e-2 * float(want.abs().max()) + 1e-3, 3e-2)


def test_flash_extend_segments_and_autograd(kernels):
    """Queries over a longer key range (prefill over a cached prefix; a context-parallel chunk over gathered keys),
    through the autograd wrapper."""
    from slime_b200.ops import _lib, attention

    torch.manual_seed(3)
    Hq, Hkv, D = 8, 2, 128
    q_lens, k_lens = [5, 130, 64], [200, 130, 1000]
    dev = "cuda"
    q = (torch.randn(sum(q_lens), Hq, D, device=dev) * 0.7).to(torch.bfloat16).requires_grad_()
    k = (torch.randn(sum(k_lens), Hkv, D, device=dev) * 0.7).to(torch.bfloat16).requires_grad_()
    v = (torch.randn(sum(k_lens), Hkv, D, device=dev) * 0.7).to(torch.bfloat16).requires_grad_()
    cu_q = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=dev)
    cu_k = torch.tensor([0] + list(torch.tensor(k_lens).cumsum(0)), dtype=torch.int32, device=dev)
    out = attention.extend_attention(q, k, v, cu_q, cu_k)
    w = torch.randn_like(out)
    (out.float() * w.float()).sum().backward()
    torch.cuda.synchronize()
    _lib.check_status(dev)
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = _ref(qf, kf, vf, attention.segments_extend(cu_q, cu_k).cpu(), 1.0 / math.sqrt(D))
    (ref * w.float()).sum().backward()
    _close(out, ref, "out", 2e-2, 2e-2)
    for name, got, want in (("dq", q.grad, qf.grad), ("dk", k.grad, kf.grad), ("dv", v.grad, vf.grad)):
        _close(got, want, name, 3e-2 * float(want.abs().max()) + 1e-3, 3e-2)


def test_rope_attention_node_matches_reference(kernels):
    """The trainer's fused node (qk-norm + RoPE + attention) on CUDA against the same node on CPU in fp32."""
    from slime_b200 import ops

    torch.manual_seed(5)
    Hq, Hkv, D, lens = 8, 2, 128, [70, 186]
    T = sum(lens)
    qkv = (torch.randn(T, (Hq + 2 * Hkv) * D) * 0.5)
    cu = torch.tensor([0, 70, 256], dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens]).to(torch.int32)
    table = ops.rope_cos_sin(512, D, 1e4)
    qw, kw = 1 + 0.1 * torch.randn(D), 1 + 0.1 * torch.randn(D)
    w = torch.randn(T, Hq * D)

    def run(dev, dt):
        x = qkv.to(dev, dt).requires_grad_()
        a, b = qw.to(dev, dt).requires_grad_(), kw.to(dev, dt).requires_grad_()
        y = ops.rope_attention(x, pos.to(dev), table.to(dev), cu.to(dev), 186, Hq, Hkv, D, a, b, 1e-6)
        (y.float() * w.to(dev)).sum().backward()
        return y.detach().float().cpu(), x.grad.float().cpu(), a.grad.float().cpu(), b.grad.float().cpu()

    got = run("cuda", torch.bfloat16)
    want = run("cpu", torch.float32)
    for name, g, r in zip(("out", "dqkv", "dq_norm_w", "dk_norm_w"), got, want):
        _close(g, r, name, 4e-2 * float(r.abs().max()) + 1e-3, 4e-2)
