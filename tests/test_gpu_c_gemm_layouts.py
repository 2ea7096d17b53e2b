"""tcgen05 GEMM with MN-major operands (dgrad / wgrad forms) against fp32 references."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _check(out, ref, tol=2e-2):
    err = (out.float() - ref).abs().max().item()
    assert err / (ref.abs().max().item() + 1e-6) < tol, f"max err {err}"


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 384, 192), (300, 896, 1152), (1000, 200, 520)])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_b_mn_major(kernels, M, N, K, bn):
    """dgrad form: dx[M,N] = dy[M,K] @ W[K,N] with W given row-major [K, N]."""
    from slime_b200 import ops
    from slime_b200.ops import _lib

    torch.manual_seed(M * 3 + N)
    dy = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
    out = ops.gemm(dy, w, b_mn=True, bn=bn)
    torch.cuda.synchronize()
    _lib.check_status("cuda")
    _check(out, dy.float() @ w.float())


@pytest.mark.parametrize("T,O,I", [(64, 128, 128), (520, 256, 384), (1000, 1152, 896), (4096, 896, 4864)])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_both_mn_major(kernels, T, O, I, bn):
    """wgrad form: dW[O,I] = dy[T,O]^T @ x[T,I]."""
    from slime_b200 import ops
    from slime_b200.ops import _lib

    torch.manual_seed(T + O)
    dy = torch.randn(T, O, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(T, I, device="cuda", dtype=torch.bfloat16)
    out = ops.gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32, bn=bn)
    torch.cuda.synchronize()
    _lib.check_status("cuda")
    _check(out, dy.float().t() @ x.float(), 1e-2)


def test_linear_autograd(kernels):
    from slime_b200 import ops

    torch.manual_seed(2)
    x = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(384, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(384, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = ops.linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    (xf @ wf.t() + bf).backward(g.float())
    _check(y, (xf @ wf.t() + bf).detach())
    _check(x.grad, xf.grad)
    _check(w.grad, wf.grad)
    _check(b.grad, bf.grad)
