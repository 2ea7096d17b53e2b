"""RMSNorm backward with library-owned scratch (``sb_rmsnorm_bwd_static``), called through its exported C symbol.

The file name sorts last on purpose: the entry point shares one scratch array per device with every earlier
call in the process, so it has to pass both on its own and after the rest of the GPU suite has run.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_CTAS, MAX_H = 148, 8192  # SB_RMSNORM_STATIC_MAX_CTAS / SB_RMSNORM_STATIC_MAX_H in csrc/rmsnorm_bwd_static.h


@pytest.fixture(scope="module")
def clib(kernels):
    """The raw shared object, bound here by hand so the test goes through the C ABI and nothing else."""
    from slime_b200.ops import build

    lib = ctypes.CDLL(build.OUT)
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.sb_rmsnorm_bwd_static_setup.argtypes, lib.sb_rmsnorm_bwd_static_setup.restype = [], I
    lib.sb_rmsnorm_bwd_static.argtypes, lib.sb_rmsnorm_bwd_static.restype = [P, P, P, P, P, P, P, I, I, I, P], I
    lib.sb_rmsnorm_bwd.argtypes, lib.sb_rmsnorm_bwd.restype = [P, P, P, P, P, P, P, P, I, I, I, I, P], I
    lib.sb_last_error.argtypes, lib.sb_last_error.restype = [], ctypes.c_char_p
    return lib


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _inputs(T, H, seed, with_res):
    g = torch.Generator(device="cuda").manual_seed(seed)
    dy = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    h = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)
    rstd = torch.rsqrt(h.float().pow(2).mean(-1) + 1e-6).contiguous()
    dres = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16) if with_res else None
    return dy, h, w, rstd, dres


def _reference(dy, h, w, rstd, dres):
    xhat = h.float() * rstd[:, None]
    dyw = dy.float() * w.float()
    dh = rstd[:, None] * (dyw - xhat * (dyw * xhat).mean(-1, keepdim=True))
    if dres is not None:
        dh = dh + dres.float()
    return dh, (dy.float() * xhat).sum(0)


def _close(a, b, rtol, atol):
    torch.testing.assert_close(a.float(), b.float(), rtol=rtol, atol=atol)


@pytest.mark.parametrize("T,H,with_res", [(1000, 896, True), (37, 4096, False), (4096, 8192, True)])
def test_static_matches_regular_twice(clib, T, H, with_res):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert clib.sb_rmsnorm_bwd_static_setup() == 0, clib.sb_last_error()
    n = min(MAX_CTAS, T)
    # everything the two calls need exists before the allocation check starts
    cases = [_inputs(T, H, seed, with_res) for seed in (T + H, T + H + 1)]
    outs = [(torch.empty(T, H, device="cuda", dtype=torch.bfloat16), torch.empty(H, device="cuda")) for _ in cases]
    refs = [(torch.empty(T, H, device="cuda", dtype=torch.bfloat16), torch.empty(H, device="cuda")) for _ in cases]
    part = torch.empty(n, H, device="cuda")
    # one untimed call first: the driver loads a kernel's code at its first launch, which is part of set-up
    dy, h, w, rstd, dres = cases[0]
    assert clib.sb_rmsnorm_bwd_static(_ptr(dy), _ptr(h), _ptr(w), _ptr(rstd), _ptr(dres), _ptr(refs[0][0]), _ptr(refs[0][1]),
                                      T, H, 0, stream) == 0, clib.sb_last_error()  # fmt: skip
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    reserved_before = torch.cuda.memory_reserved()
    for (dy, h, w, rstd, dres), (dh, dw) in zip(cases, outs):  # two calls in a row on the shared scratch
        rc = clib.sb_rmsnorm_bwd_static(_ptr(dy), _ptr(h), _ptr(w), _ptr(rstd), _ptr(dres), _ptr(dh), _ptr(dw), T, H, 0, stream)
        assert rc == 0, clib.sb_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_reserved() == reserved_before
    for (dy, h, w, rstd, dres), (dh, dw), (dh_r, dw_r) in zip(cases, outs, refs):
        rc = clib.sb_rmsnorm_bwd(_ptr(dy), _ptr(h), _ptr(w), _ptr(rstd), _ptr(dres), _ptr(dh_r), _ptr(part), _ptr(dw_r),
                                 T, H, n, 0, stream)
        assert rc == 0, clib.sb_last_error()
        torch.cuda.synchronize()
        _close(dh, dh_r, 3e-2, 2e-2)  # the tolerances of the regular entry point's own test
        _close(dw, dw_r, 5e-2, 2e-2)
        dh_f, dw_f = _reference(dy, h, w, rstd, dres)  # and both against plain fp32 PyTorch
        _close(dh, dh_f, 3e-2, 2e-2)
        _close(dw, dw_f, 5e-2, 5e-2)


def test_static_accumulates_into_dw(clib):
    T, H = 300, 1024
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    dy, h, w, rstd, _ = _inputs(T, H, 7, False)
    dh = torch.empty_like(dy)
    dw = torch.full((H,), 2.0, device="cuda")
    assert clib.sb_rmsnorm_bwd_static(_ptr(dy), _ptr(h), _ptr(w), _ptr(rstd), None, _ptr(dh), _ptr(dw), T, H, 1, stream) == 0
    torch.cuda.synchronize()
    _close(dw, _reference(dy, h, w, rstd, None)[1] + 2.0, 5e-2, 5e-2)


@pytest.mark.parametrize("H", [MAX_H + 8, 900, 0])
def test_static_rejects_sizes_beyond_the_scratch(clib, H):
    """Too wide, not a multiple of 8, or empty: nothing is launched and the reason is readable."""
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    t = torch.zeros(8, device="cuda")
    rc = clib.sb_rmsnorm_bwd_static(_ptr(t), _ptr(t), _ptr(t), _ptr(t), None, _ptr(t), _ptr(t), 4, H, 0, stream)
    assert rc == 1  # cudaErrorInvalidValue
    msg = clib.sb_last_error().decode()
    assert "sb_rmsnorm_bwd_static" in msg and str(MAX_H) in msg
    torch.cuda.synchronize()


def test_static_rejects_misaligned_pointers(clib):
    """A base pointer off the 16-byte boundary the kernels load from is refused on the host; nothing is launched."""
    T, H = 16, 64
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    dy, h, w, rstd, _ = _inputs(T, H, 3, False)
    dh, dw = torch.empty_like(dy), torch.empty(H, device="cuda")
    odd = torch.empty(T * H + 8, device="cuda", dtype=torch.bfloat16)[1:]  # starts 2 bytes past an aligned address
    for args in [(odd, h, w, rstd, None, dh, dw), (dy, h, w, rstd, None, odd, dw), (dy, h, w, rstd, odd, dh, dw)]:
        rc = clib.sb_rmsnorm_bwd_static(*[_ptr(a) for a in args], T, H, 0, stream)
        assert rc == 1
        assert "misaligned" in clib.sb_last_error().decode()
    assert clib.sb_rmsnorm_bwd_static(_ptr(dy), _ptr(h), _ptr(w), _ptr(rstd), None, _ptr(dh), _ptr(dw), T, H, 0, stream) == 0
    torch.cuda.synchronize()
