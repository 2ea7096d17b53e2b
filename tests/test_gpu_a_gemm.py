"""tcgen05 GEMM (K-major operands) against an fp32 PyTorch reference."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, bias=None):
    out = a.float() @ b.float().t()
    return out + bias.float() if bias is not None else out


def _check(out, ref, tol=2e-2, K=None):
    """Per element: |out - ref| <= atol + rtol |ref|. A bf16 result carries one rounding of relative size 2^-9, a fp32
    result only the accumulation-order error; the absolute floor covers elements that cancel to ~0 (their error scales
    with sqrt(K) times the size of one product), so a wrong tile edge of small magnitude cannot hide behind the
    tensor's largest entry. ``tol`` keeps the old global bound as a second, coarser net."""
    err = (out.float() - ref).abs()
    K = K if K is not None else 1024
    rtol, atol = (1e-2, 2e-3 * K**0.5) if out.dtype == torch.bfloat16 else (2e-3, 5e-4 * K**0.5)
    bad = err > atol + rtol * ref.abs()
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} elements off; worst {float(err.max()):.4g} at |ref| {float(ref.abs()[err.argmax() // ref.shape[1], err.argmax() % ref.shape[1]]):.4g}"
    assert err.max().item() / (ref.abs().max().item() + 1e-6) < tol


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 128), (128, 256, 512), (384, 896, 896), (1000, 1152, 896),
                                   (77, 200, 72), (4096, 4864, 896), (130, 151936 // 16, 896)])  # fmt: skip
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_nt_bf16(kernels, M, N, K, bn):
    from slime_b200 import ops
    from slime_b200.ops import _lib

    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    out = ops.gemm(a, b, bn=bn)
    torch.cuda.synchronize()
    _lib.check_status("cuda")
    _check(out, _ref(a, b), K=K)


def test_gemm_fp32_out_bias_accumulate(kernels):
    from slime_b200 import ops
    from slime_b200.ops import _lib

    torch.manual_seed(0)
    M, N, K = 300, 512, 256
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    out = ops.gemm(a, b, bias=bias, out_dtype=torch.float32)
    _check(out, _ref(a, b, bias), 5e-3, K=K)
    acc = torch.ones(M, N, device="cuda", dtype=torch.float32)
    ops.gemm(a, b, out=acc, accumulate=True)
    _check(acc, _ref(a, b) + 1.0, 5e-3, K=K)
    # strided output rows (a column block of a wider buffer)
    wide = torch.zeros(M, N + 64, device="cuda", dtype=torch.bfloat16)
    ops.gemm(a, b, out=wide[:, :N])
    _check(wide[:, :N], _ref(a, b), K=K)
    assert wide[:, N:].abs().max().item() == 0
    torch.cuda.synchronize()
    _lib.check_status("cuda")


def test_gemm_matches_cublas_closely(kernels):
    """Same bf16 inputs, fp32 accumulate: results should agree with cuBLAS to bf16 rounding."""
    from slime_b200 import ops

    torch.manual_seed(1)
    a = torch.randn(2048, 1024, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(1536, 1024, device="cuda", dtype=torch.bfloat16)
    ours = ops.gemm(a, b, out_dtype=torch.float32)
    ref = _ref(a, b)
    assert (ours - ref).abs().max().item() < 1e-2 * ref.abs().max().item()
