"""tcgen05 paged decode attention against a plain fp32 PyTorch reference (and against the CUDA-core kernel)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(q, kc, vc, bt, lens, ps, scale):
    B, Hq, D = q.shape
    Hkv = kc.shape[1]
    G = Hq // Hkv
    out = torch.zeros(B, Hq, D, dtype=torch.float32, device=q.device)
    for b in range(B):
        n = int(lens[b])
        if n == 0:
            continue
        t = torch.arange(n, device=q.device)
        slots = bt[b, t // ps].long() * ps + t % ps
        k = kc[slots].float()  # [n, Hkv, D]
        v = vc[slots].float()
        for h in range(Hq):
            s = (k[:, h // G] @ q[b, h].float()) * scale
            out[b, h] = torch.softmax(s, 0) @ v[:, h // G]
    return out


@pytest.mark.parametrize("Hq,Hkv,D,ps", [(14, 2, 64, 16), (32, 8, 128, 16), (16, 4, 128, 64), (32, 4, 128, 32), (16, 1, 64, 128),
                                         (2, 2, 64, 16)])  # fmt: skip
@pytest.mark.parametrize("ws", ["0", "1"])
def test_decode_attention_tc(kernels, monkeypatch, Hq, Hkv, D, ps, ws):
    from slime_b200 import ops

    if ws == "1" and (D != 64 or Hq // Hkv > 8):
        pytest.skip("the warp-specialised kernel covers head dim 64, group size <= 8")
    monkeypatch.setenv("SLIME_B200_DECODE_ATTN_WS", ws)
    from slime_b200.ops import _lib

    torch.manual_seed(Hq * 7 + D)
    lens_list = [1, 15, 16, 17, 100, 128, 129, 333, 64, 257, 300, 640, 0]
    B = len(lens_list)
    max_pages = -(-700 // ps)
    pages = B * max_pages + 1
    kc = torch.randn(pages * ps, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(pages * ps, Hkv, D, device="cuda", dtype=torch.bfloat16)
    lens = torch.tensor(lens_list, device="cuda", dtype=torch.int32)
    bt = (1 + torch.randperm(pages - 1)[: B * max_pages]).view(B, max_pages).to(torch.int32).cuda()
    # poison every slot a sequence does not own yet: the kernel must never let them reach the output
    owned = torch.zeros(pages * ps, dtype=torch.bool, device="cuda")
    for b, n in enumerate(lens_list):
        t = torch.arange(n, device="cuda")
        owned[bt[b, t // ps].long() * ps + t % ps] = True
    kc[~owned] = float("nan")
    vc[~owned] = float("nan")
    q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
    scale = D**-0.5
    ref = _reference(q, kc, vc, bt, lens, ps, scale)
    for splits in (1, 3):
        out = ops.paged_decode_attention(q, kc, vc, bt, lens, ps, splits=splits, use_tensor_cores=True)
        torch.cuda.synchronize()
        _lib.check_status("cuda")
        assert torch.isfinite(out.float()).all()
        torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=1e-2)
    if Hq // Hkv in (1, 2, 4, 5, 7, 8):  # group sizes the CUDA-core kernel is built for
        legacy = ops.paged_decode_attention(q, kc, vc, bt, lens, ps, splits=1, use_tensor_cores=False)
        torch.testing.assert_close(out.float(), legacy.float(), rtol=2e-2, atol=1.5e-2)


@pytest.mark.parametrize("ws", ["0", "1"])
def test_decode_attention_tc_strided_q_and_long_context(kernels, monkeypatch, ws):
    """q as a view into a packed qkv row (the engine's layout) and a context that spans many tiles."""
    from slime_b200 import ops

    monkeypatch.setenv("SLIME_B200_DECODE_ATTN_WS", ws)
    from slime_b200.ops import _lib

    torch.manual_seed(3)
    Hq, Hkv, D, ps, B = 14, 2, 64, 16, 5
    lens_list = [4096, 3000, 1, 2049, 777]
    max_pages = 4096 // ps
    pages = B * max_pages + 1
    kc = torch.randn(pages * ps, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(pages * ps, Hkv, D, device="cuda", dtype=torch.bfloat16)
    lens = torch.tensor(lens_list, device="cuda", dtype=torch.int32)
    bt = (1 + torch.randperm(pages - 1)[: B * max_pages]).view(B, max_pages).to(torch.int32).cuda()
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
    q = qkv.view(B, Hq + 2 * Hkv, D)[:, :Hq]
    ref = _reference(q, kc, vc, bt, lens, ps, D**-0.5)
    for splits in (1, 8):
        out = ops.paged_decode_attention(q, kc, vc, bt, lens, ps, splits=splits)
        torch.cuda.synchronize()
        _lib.check_status("cuda")
        torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=1e-2)
