"""Block-scaled fp8 GEMM (tcgen05 kind::f8f6f4 with per-K-block promotion) against the dequantised fp32 product."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K,dtype", [(128, 128, 128, torch.float32), (300, 200, 256, torch.bfloat16),
                                          (1024, 1536, 2048, torch.bfloat16), (4096, 768, 7168, torch.float32)])
def test_fp8_block_gemm_matches_dequantised_product(kernels, M, N, K, dtype):
    from slime_b200 import ops
    from slime_b200.ops import _lib

    torch.manual_seed(M + N)
    x = torch.randn(M, K, device="cuda") * 1.5
    w = torch.randn(N, K, device="cuda") * 0.1
    # make the scales differ strongly between blocks so a wrong scale index cannot hide
    x[:, : K // 2] *= 7.0
    w[: N // 2] *= 3.0
    xq, xs = ops.block_fp8_quant(x.to(torch.bfloat16), (1, 128))
    wq, ws = ops.block_fp8_quant(w.to(torch.bfloat16), (128, 128))
    out = ops.fp8_block_gemm(xq, xs, wq, ws, out_dtype=dtype)
    torch.cuda.synchronize()
    _lib.check_status(out.device)
    a = xq.float() * xs.repeat_interleave(128, dim=1)
    b = wq.float() * ws.repeat_interleave(128, dim=0)[:N].repeat_interleave(128, dim=1)
    ref = a @ b.t()
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-3
    assert (out.float() - ref).abs().max() <= tol * ref.abs().max(), float((out.float() - ref).abs().max() / ref.abs().max())
    # and the quantised product is close to the bf16 one (sanity of the whole W8A8 path)
    full = x.to(torch.bfloat16).float() @ w.to(torch.bfloat16).float().t()
    assert (out.float() - full).abs().max() <= 0.08 * full.abs().max()


def test_activation_quant_kernel_matches_block_quant(kernels):
    from slime_b200 import ops
    from slime_b200.ops import reference

    torch.manual_seed(3)
    x = (torch.randn(777, 1024, device="cuda") * torch.rand(777, 1, device="cuda") * 20).to(torch.bfloat16)
    q, s, st = ops.fp8_act_quant(x)
    qr, sr = reference.block_fp8_quant(x.cpu(), (1, 128), False)
    torch.testing.assert_close(s.cpu(), sr, rtol=1e-6, atol=0)
    assert torch.equal(st, s.t())
    # the kernel multiplies by 1/scale where the reference divides: a value on a rounding boundary may land one code off
    same = (q.cpu().view(torch.uint8) == qr.view(torch.uint8)).float().mean().item()
    assert same > 0.999, same
    deq, deq_ref = q.cpu().float() * s.cpu().repeat_interleave(128, 1), qr.float() * sr.repeat_interleave(128, 1)
    assert (deq - deq_ref).abs().max() <= 0.13 * deq_ref.abs().max()
    q2, s2 = ops.block_fp8_quant(x, (1, 128))  # the generic entry point takes the same fast path
    assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8)) and torch.equal(s2, s)
