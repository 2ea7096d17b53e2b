"""Fused / split paths against plain fp32 PyTorch: split-K GEMM, rope+attention node, vectorised loss reducers."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


@pytest.mark.parametrize("T,O,I,splitk", [(4096, 1152, 896, 4), (1000, 256, 384, 3), (16384, 896, 896, 8), (777, 128, 128, 13)])
def test_wgrad_splitk_accumulates_into_main_grad(kernels, T, O, I, splitk):
    from slime_b200 import ops
    from slime_b200.ops import _lib

    torch.manual_seed(T)
    dy = torch.randn(T, O, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(T, I, device="cuda", dtype=torch.bfloat16)
    ref = dy.float().t() @ x.float()
    acc = torch.full((O, I), 0.5, device="cuda", dtype=torch.float32)
    ops.gemm(dy, x, a_mn=True, b_mn=True, out=acc, accumulate=True, splitk=splitk)
    torch.cuda.synchronize()
    _lib.check_status("cuda")
    assert _rel(acc - 0.5, ref) < 1e-2
    fresh = ops.gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32, splitk=splitk)  # zero-filled output, then summed
    auto = ops.gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32)  # heuristic choice of slices
    torch.cuda.synchronize()
    _lib.check_status("cuda")
    assert _rel(fresh, ref) < 1e-2 and _rel(auto, ref) < 1e-2


@pytest.mark.parametrize("M,N,K", [(256, 896, 4864), (64, 896, 896), (256, 1152, 896)])
def test_skinny_splitk_with_bias(kernels, M, N, K):
    """Decode-shaped projection: few output tiles, long K; the bias must be added exactly once."""
    from slime_b200 import ops

    torch.manual_seed(M + K)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ w.float().t() + b.float()
    for sk in (1, 2, 5):
        out = ops.gemm(a, w, bias=b, out_dtype=torch.float32, splitk=sk)
        torch.cuda.synchronize()
        assert _rel(out, ref) < 1e-2, sk
    with pytest.raises(AssertionError):
        ops.gemm(a, w, out_dtype=torch.bfloat16, splitk=2)


@pytest.mark.parametrize("Hq,Hkv,D,qknorm", [(14, 2, 64, False), (8, 2, 128, True)])
def test_rope_attention_node_matches_reference(kernels, Hq, Hkv, D, qknorm):
    from slime_b200 import ops

    torch.manual_seed(D + Hq)
    lens = [5, 130, 64, 257]
    T = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens]).to(torch.int32)
    qkv = (0.5 * torch.randn(T, (Hq + 2 * Hkv) * D)).to(torch.bfloat16)
    qn = (1 + 0.1 * torch.randn(D)).to(torch.bfloat16) if qknorm else None
    kn = (1 + 0.1 * torch.randn(D)).to(torch.bfloat16) if qknorm else None
    g = torch.randn(T, Hq * D).to(torch.bfloat16)

    def run(dev, dtype):
        x = qkv.to(dev, dtype).requires_grad_(True)
        ws = [None if w is None else w.to(dev, dtype).requires_grad_(True) for w in (qn, kn)]
        cs = ops.rope_cos_sin(512, D, 1e6, device=dev)
        # clone: the CUDA node rotates the projection output in place, exactly as it does inside the model
        out = ops.rope_attention(x.clone(), pos.to(dev), cs, cu.to(dev), max(lens), Hq, Hkv, D, ws[0], ws[1], 1e-6)
        out.backward(g.to(dev, dtype))
        return out.detach().float().cpu(), x.grad.float().cpu(), [None if w is None else w.grad.float().cpu() for w in ws]

    out_c, dx_c, dw_c = run("cuda", torch.bfloat16)
    out_r, dx_r, dw_r = run("cpu", torch.float32)
    assert _rel(out_c, out_r) < 3e-2
    assert _rel(dx_c, dx_r) < 5e-2
    if qknorm:
        assert _rel(dw_c[0], dw_r[0]) < 8e-2 and _rel(dw_c[1], dw_r[1]) < 8e-2


def test_sum_of_sample_mean_matches_per_sample_loop(kernels):
    from slime_b200.backends.train.cp_utils import get_sum_of_sample_mean

    torch.manual_seed(0)
    resp = [7, 1, 30, 12]
    total = [r + 5 for r in resp]
    masks = [(torch.rand(r, device="cuda") > 0.3).int() for r in resp]
    masks[1][:] = 0  # a fully masked sample contributes 0, not NaN
    x = torch.randn(sum(resp), device="cuda", requires_grad=True)
    expect = sum((p * m).sum() / m.sum().clamp_min(1) for p, m in zip(x.detach().split(resp), masks))
    red = get_sum_of_sample_mean(total, resp, masks)
    got = red(x)
    assert torch.allclose(got, expect, atol=1e-5)
    got.backward()
    grad = torch.cat([m.float() / m.sum().clamp_min(1) for m in masks])
    assert torch.allclose(x.grad, grad, atol=1e-6)
    denoms = torch.tensor([10.0, 3.0, 40.0, 40.0], device="cuda")
    got2 = get_sum_of_sample_mean(total, resp, masks, sample_denoms=denoms)(x.detach())
    expect2 = sum((p * m).sum() / d for p, m, d in zip(x.detach().split(resp), masks, denoms))
    assert torch.allclose(got2, expect2, atol=1e-5)
    per_tok = get_sum_of_sample_mean(total, resp, masks, calculate_per_token_loss=True)(x.detach())
    assert torch.allclose(per_tok, sum((p * m).sum() for p, m in zip(x.detach().split(resp), masks)), atol=1e-5)


def test_peer_wait_expiry_sets_status_and_context_survives(kernels):
    """A barrier whose second participant never arrives: the wait runs out (5 ms limit), the kernel returns with
    ERR_WAIT_PEER in the status word, the host check raises, later barriers return at once while the word is set, and
    an ordinary launch afterwards still works."""
    import ctypes
    import time

    from slime_b200 import ops
    from slime_b200.ops import _lib

    lib = _lib.lib()
    pad = torch.zeros(64, dtype=torch.int32, device="cuda")  # stands in for both ranks' signal pads; nobody signals word 1
    pads = (ctypes.c_void_p * 2)(pad.data_ptr(), pad.data_ptr() + 128)
    status = _lib.status_word("cuda")
    status.zero_()
    old = _lib.set_peer_wait_limit(0.005)
    try:
        t0 = time.perf_counter()
        _lib.check(lib.sb_symm_barrier(pads, 0, 2, 1, 0, _lib.ptr(status), _lib.stream()), "sb_symm_barrier")
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 1.0
        assert int(status.item()) & 0xFF == 5
        # sticky word: a second barrier announces itself and returns without waiting
        _lib.check(lib.sb_symm_barrier(pads, 0, 2, 2, 0, _lib.ptr(status), _lib.stream()), "sb_symm_barrier")
        torch.cuda.synchronize()
        with pytest.raises(_lib.KernelWaitExpired) as ei:
            _lib.check_status("cuda")
        assert ei.value.code == 5
    finally:
        _lib.set_peer_wait_limit(old)
    assert int(status.item()) == 0
    a = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(128, 128, device="cuda", dtype=torch.bfloat16)
    out = ops.gemm(a, b)
    torch.cuda.synchronize()
    _lib.check_status("cuda")
    assert _rel(out, a.float() @ b.float().t()) < 2e-2
