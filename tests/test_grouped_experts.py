"""Grouped expert MLP: the padded-layout path against the per-expert loop (CPU), and against fp32 math on a GPU."""

import pytest
import torch

from slime_b200.ops import grouped


def _loop_reference(x, counts, w1, w2):
    outs, s = [], 0
    for e, n in enumerate(counts):
        xe = x[s : s + n].float()
        h = xe @ w1[e].float().t()
        g, u = h.chunk(2, dim=-1)
        outs.append((torch.nn.functional.silu(g) * u) @ w2[e].float().t())
        s += n
    return torch.cat(outs)


def test_padded_layout_and_stacked_view():
    lay = grouped.PaddedLayout([3, 0, 130, 128], "cpu")
    assert lay.padded == [128, 0, 256, 128] and lay.rows == 261 and lay.rows_padded == 512
    assert lay.tile_expert.tolist() == [0, 2, 2, 3] and lay.dest[:4].tolist() == [0, 1, 2, 128]
    x = torch.arange(261.0)[:, None].repeat(1, 2)
    assert torch.equal(lay.unpad(lay.pad(x)), x) and lay.pad(x)[3:128].abs().sum() == 0
    flat = torch.randn(3 * 4 * 5)
    views = [flat[i * 20 : (i + 1) * 20].view(4, 5) for i in range(3)]
    st = grouped.stacked_view(views)
    assert st is not None and st.data_ptr() == flat.data_ptr() and torch.equal(st[2], views[2])
    assert grouped.stacked_view([views[0], views[2]]) is None
    assert grouped.stacked_view([torch.randn(4, 5), torch.randn(4, 5).t().contiguous().t()]) is None


def test_grouped_experts_module_matches_loop_on_cpu():
    from slime_b200.models.config import get_preset
    from slime_b200.models.moe import GroupedExperts
    from slime_b200.parallel import state as mpu

    if not mpu.model_parallel_is_initialized():
        mpu.initialize_model_parallel()
    cfg = get_preset("tiny-moe")
    torch.manual_seed(0)
    m = GroupedExperts(cfg, torch.float32, "cpu", 4)
    counts = [5, 0, 9, 2]
    x = torch.randn(sum(counts), cfg.hidden_size, requires_grad=True)
    y = m(x, counts)
    y.pow(2).sum().backward()
    gx, gw = x.grad.clone(), [p.grad.clone() for p in m.parameters()]
    x.grad = None
    for p in m.parameters():
        p.grad = None
    m.use_grouped_gemm = False
    y2 = m(x, counts)
    y2.pow(2).sum().backward()
    torch.testing.assert_close(y, y2, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(gx, x.grad, rtol=1e-4, atol=1e-5)
    for a, p in zip(gw, m.parameters()):
        torch.testing.assert_close(a, p.grad if p.grad is not None else torch.zeros_like(p), rtol=1e-4, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("counts", [[300, 0, 77, 129, 1, 128], [4096, 1000, 2, 3000]])
def test_grouped_gemm_gpu_matches_fp32(kernels, counts):
    from slime_b200 import ops

    torch.manual_seed(len(counts))
    E, H, F = len(counts), 512, 384
    dev = "cuda"
    flat1 = (torch.randn(E * 2 * F * H, device=dev) * 0.05).to(torch.bfloat16)  # adjacent experts: the no-copy path
    w1 = [flat1[e * 2 * F * H : (e + 1) * 2 * F * H].view(2 * F, H).requires_grad_() for e in range(E)]
    w2 = [(torch.randn(H, F, device=dev) * 0.05).to(torch.bfloat16).requires_grad_() for _ in range(E)]  # stacked by copy
    x = torch.randn(sum(counts), H, device=dev).to(torch.bfloat16).requires_grad_()
    lay = grouped.PaddedLayout(counts, dev)
    assert grouped.stacked_view([w.detach() for w in w1]) is not None
    h = grouped.grouped_linear(lay.pad(x), lay, w1)
    y = lay.unpad(grouped.grouped_linear(ops.swiglu(h), lay, w2))
    ref = _loop_reference(x.detach(), counts, [w.detach() for w in w1], [w.detach() for w in w2])
    assert (y.float() - ref).abs().max() <= 0.03 * ref.abs().max() + 1e-3
    gy = torch.randn_like(y)
    y.backward(gy)
    xr = x.detach().float().requires_grad_()
    w1r = [w.detach().float().requires_grad_() for w in w1]
    w2r = [w.detach().float().requires_grad_() for w in w2]
    outs, s = [], 0
    for e, n in enumerate(counts):
        hh = xr[s : s + n] @ w1r[e].t()
        g, u = hh.chunk(2, dim=-1)
        outs.append((torch.nn.functional.silu(g) * u) @ w2r[e].t())
        s += n
    torch.cat(outs).backward(gy.float())

    def close(a, b, what):
        assert (a.float() - b).abs().max() <= 0.04 * b.abs().max() + 1e-3, what

    close(x.grad, xr.grad, "dx")
    for e in range(E):
        close(w1[e].grad if w1[e].grad is not None else torch.zeros_like(w1[e]), w1r[e].grad if w1r[e].grad is not None else torch.zeros_like(w1r[e]), f"dw1[{e}]")
        close(w2[e].grad if w2[e].grad is not None else torch.zeros_like(w2[e]), w2r[e].grad if w2r[e].grad is not None else torch.zeros_like(w2r[e]), f"dw2[{e}]")


def _moe_reference(x, idx, probs, w13, w2):
    out = torch.zeros(x.shape[0], x.shape[1])
    for t in range(x.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            h = x[t].float() @ w13[e].float().t()
            g, u = h.chunk(2)
            out[t] += float(probs[t, j]) * ((torch.nn.functional.silu(g) * u) @ w2[e].float().t())
    return out


def test_device_layout_moe_matches_per_token_reference():
    from slime_b200 import ops

    torch.manual_seed(1)
    T, k, E, H, F = 37, 2, 5, 16, 24
    x = torch.randn(T, H)
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(T)])
    idx[:, 0] = torch.where(idx[:, 0] == 3, torch.tensor(0), idx[:, 0])  # expert 3 gets fewer tokens
    probs = torch.rand(T, k)
    w13, w2 = torch.randn(E, 2 * F, H) * 0.2, torch.randn(E, H, F) * 0.2
    lay = grouped.DeviceLayout(idx, E)
    assert lay.rows_padded % 128 == 0 and lay.rows_padded >= T * k
    act = ops.swiglu(grouped.grouped_gemm(lay.pad(x), w13, lay))
    y = lay.combine(grouped.grouped_gemm(act, w2, lay), probs, T)
    torch.testing.assert_close(y, _moe_reference(x, idx, probs, w13, w2), rtol=1e-4, atol=1e-5)


def test_moe_engine_decodes_consistently_on_cpu():
    """tiny-moe through the engine: decode log-probs equal teacher-forced ones (prefill and decode share the MoE path)."""
    import numpy as np

    from slime_b200.engine.engine import Engine
    from slime_b200.engine.server_args import ServerArgs
    from slime_b200.models.config import get_preset

    e = Engine(get_preset("tiny-moe"), ServerArgs(page_size=4, max_running_requests=4, context_length=64, disable_cuda_graph=True),
               device="cpu", num_pages=64)
    e.weights.init_random(0)
    r = e.generate([[1, 2, 3, 4, 5]], [dict(max_new_tokens=6, ignore_eos=True)])[0]
    rq = e.generate([r.input_ids + r.output_ids], [dict(max_new_tokens=0)], logprob_start_len=0)[0]
    assert np.abs(np.array(rq.input_logprobs[5:]) - np.array(r.output_logprobs)).max() < 1e-4


def _perm_case(device, dtype):
    torch.manual_seed(4)
    T, k, H, R = 33, 3, 64, 150
    x = torch.randn(T, H, device=device).to(dtype)
    dest = torch.randperm(R, device=device)[: T * k].to(torch.int32)
    dest[5] = -1  # a dropped route
    w = torch.rand(T, k, device=device)
    return x, dest, w, T, k, H, R


def test_route_permutation_ops_and_gradients_cpu():
    x, dest, w, T, k, H, R = _perm_case("cpu", torch.float32)
    x.requires_grad_()
    w.requires_grad_()
    rows = grouped.permute_tokens(x, dest, k, R)
    assert torch.equal(rows[dest[7].long()], x[7 // k].detach()) and rows.abs().sum(1).ne(0).sum() == T * k - 1
    y = grouped.combine_routes(rows * 2.0, dest, w, k)
    d = dest.view(T, k).long()
    ok = (d >= 0).float()
    want = (2.0 * x.detach()[:, None, :] * (w.detach() * ok)[:, :, None]).sum(1)
    torch.testing.assert_close(y, want, rtol=1e-5, atol=1e-6)
    gy = torch.randn_like(y)
    y.backward(gy)
    # d/dx sum_j 2 w_j x = 2 * sum_j w_j * gy ; d/dw_j = <2 x, gy>
    torch.testing.assert_close(x.grad, 2.0 * (w.detach() * ok).sum(1, keepdim=True) * gy, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(w.grad, ok * (2.0 * x.detach() * gy).sum(-1, keepdim=True), rtol=1e-5, atol=1e-5)


@pytest.mark.gpu
def test_route_permutation_kernels_match_cpu_reference_and_are_deterministic(kernels):
    x, dest, w, T, k, H, R = _perm_case("cuda", torch.bfloat16)
    rows = grouped.scatter_rows(x, dest, k, R)
    assert torch.equal(rows.cpu(), grouped.scatter_rows(x.cpu(), dest.cpu(), k, R))
    y = grouped.gather_sum(rows, dest, w, k)
    ref = grouped.gather_sum(rows.cpu(), dest.cpu(), w.cpu(), k)
    assert (y.cpu().float() - ref.float()).abs().max() <= 2e-2 * ref.float().abs().max()
    assert torch.equal(grouped.gather_sum(rows, dest, w, k), y)  # same bits every time
    y2 = grouped.gather_sum(rows, dest, w, k, round_each=True)
    ref2 = grouped.gather_sum(rows.cpu(), dest.cpu(), w.cpu(), k, round_each=True)
    assert (y2.cpu().float() - ref2.float()).abs().max() <= 2e-2 * ref2.float().abs().max()
    dy = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    dw = grouped.route_weight_grad(rows, dest, dy, k)
    torch.testing.assert_close(dw.cpu(), grouped.route_weight_grad(rows.cpu(), dest.cpu(), dy.cpu(), k), rtol=2e-3, atol=2e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("E,k", [(128, 8), (8, 2), (160, 6), (512, 32)])
def test_route_topk_kernel_matches_torch(kernels, E, k):
    torch.manual_seed(E)
    T = 301
    logits = torch.randn(T, E, device="cuda") * 3
    bias = torch.randn(E, device="cuda") * 0.5
    cases = [dict(), dict(pre_softmax=True), dict(renorm=False), dict(score="sigmoid", bias=bias, scale=2.5),
             dict(score="sigmoid", renorm=False)]
    for kw in cases:
        w, idx = grouped.route_topk(logits, k, **kw)
        kw_cpu = {a: (b.cpu() if torch.is_tensor(b) else b) for a, b in kw.items()}
        w_ref, idx_ref = grouped.route_topk(logits.cpu(), k, **kw_cpu)
        assert torch.equal(idx.cpu(), idx_ref), kw  # random logits: no ties, the order of the picks is the same
        torch.testing.assert_close(w.cpu(), w_ref, rtol=1e-4, atol=1e-6)


@pytest.mark.gpu
def test_moe_engine_decode_in_cuda_graphs_matches_eager_launches(kernels):
    """The MoE decode step is captured like the dense one (its layout is built on the device with static shapes): the
    replayed step draws the same tokens, log-probs and expert choices as eager launches of the same kernels."""
    from slime_b200.engine.engine import Engine
    from slime_b200.engine.server_args import ServerArgs
    from slime_b200.models.config import get_preset

    prompts = [[(5 * i + 3 * j) % 500 for j in range(6 + i)] for i in range(4)]
    got = []
    for graphs in (False, True):
        e = Engine(get_preset("tiny-moe"), ServerArgs(page_size=16, max_running_requests=4, context_length=128,
                                                      disable_cuda_graph=not graphs, enable_return_routed_experts=True),
                   device="cuda", num_pages=64)  # fmt: skip
        e.weights.init_random(0, std=0.2)
        reqs = e.generate(prompts, dict(max_new_tokens=10, temperature=0, ignore_eos=True), return_routed_experts=True)
        assert bool(e.runner.graphs) == graphs
        for r in reqs:
            routed = torch.cat(r.routed_experts)
            assert routed.shape == (len(r.input_ids) + len(r.output_ids) - 1, 2, 2)
        got.append(([r.output_ids for r in reqs], [r.output_logprobs for r in reqs], [torch.cat(r.routed_experts) for r in reqs]))
        e.shutdown()
    assert got[0][0] == got[1][0]
    assert max(abs(a - b) for x, y in zip(got[0][1], got[1][1]) for a, b in zip(x, y)) < 1e-3
    assert all(torch.equal(a, b) for a, b in zip(got[0][2], got[1][2]))
