"""Grouped (per-expert) linear layers on the tcgen05 GEMM: the MoE expert MLP without a Python loop over experts.

Layout ("M-contiguous"): the tokens routed to this rank's experts arrive sorted by expert; ``PaddedLayout`` places each
expert's rows at a multiple of 128 (the GEMM's row tile), so every tile belongs to exactly one expert and the kernel
only needs a per-tile row offset into the stacked weights (``csrc/gemm_sm100.cu``: ``sb_gemm_bf16_grouped``).

    lay = PaddedLayout(counts, device)              # counts: rows per local expert (host ints)
    xp = lay.pad(x)                                 # [M_pad, H], padding rows are zero
    h = grouped_linear(xp, lay, fc1_weights)        # fc1_weights: list of E parameters [N, K]
    y = lay.unpad(grouped_linear(swiglu(h), lay, fc2_weights))

Forward ``y_e = x_e W_e^T`` and the input gradient ``dx_e = dy_e W_e`` are one grouped launch each; the weight
gradients are one ``dy_e^T x_e`` GEMM per expert over that expert's row range (accumulated straight into
``main_grad`` when the parameter has one). The experts' weights are used in place when they are adjacent in memory (the
flat parameter buffer lays them out that way); otherwise they are stacked with a copy.
On CPU the same functions run a per-expert fp32 loop (the numerics oracle of the GPU path).
"""

from __future__ import annotations

import torch

from slime_b200.ops import _checks, _lib

TILE = 128
P = _lib.ptr


def route_topk(logits: torch.Tensor, k: int, *, score: str = "softmax", pre_softmax: bool = False, renorm: bool = True,
               bias: torch.Tensor | None = None, scale: float | None = None):
    """Router logits [T, E] (fp32) -> ``(weights [T, k] fp32, indices [T, k] int64)`` in one kernel.

    ``score="softmax"`` with ``renorm`` and not ``pre_softmax``: softmax over the k picked logits; with ``pre_softmax``
    or ``renorm=False``: full softmax, pick k, keep the probabilities. ``score="sigmoid"``: sigmoid scores, ``bias``
    steers the choice only, weights are the picked scores (normalised when ``renorm``). ``scale`` multiplies the result.
    """
    T, E = logits.shape
    mode = 2 if score == "sigmoid" else (1 if (pre_softmax or not renorm) else 0)
    if logits.is_cuda and E <= 512 and k <= 32:
        lg = logits.float().contiguous()
        idx = torch.empty(T, k, dtype=torch.int32, device=lg.device)
        w = torch.empty(T, k, dtype=torch.float32, device=lg.device)
        b = None if bias is None else bias.float().contiguous()
        rc = _lib.lib().sb_moe_topk(P(lg), P(b), P(idx), P(w), T, E, k, mode, int(renorm), float(scale or 1.0), _lib.stream())
        _lib.check(rc, "sb_moe_topk")
        return w, idx.long()
    lg = logits.float()
    if mode == 2:
        scores = torch.sigmoid(lg)
        idx = torch.topk(scores + bias.float() if bias is not None else scores, k, dim=-1).indices
        w = scores.gather(-1, idx)
        if renorm:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
    elif mode == 1:
        w, idx = torch.topk(torch.softmax(lg, -1), k, dim=-1)
    else:
        top, idx = torch.topk(lg, k, dim=-1)
        w = torch.softmax(top, -1)
    return w * (scale or 1.0), idx


def scatter_rows(x: torch.Tensor, dest: torch.Tensor, k: int, num_rows: int) -> torch.Tensor:
    """``out[dest[s]] = x[s // k]`` for every route slot ``s`` with ``dest[s] >= 0``; other rows of ``out`` are zero."""
    _checks.index_range("scatter_rows", "dest", dest, upper=num_rows, lower=-(1 << 31))
    out = x.new_zeros(num_rows, x.shape[-1])
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        rc = _lib.lib().sb_moe_scatter_rows(P(x.contiguous()), P(dest), P(out), dest.numel(), k, x.shape[-1], _lib.stream())
        _lib.check(rc, "sb_moe_scatter_rows")
        return out
    keep = dest >= 0
    src = torch.arange(dest.numel(), device=dest.device)[keep] // k
    out[dest[keep].long()] = x[src]
    return out


def gather_sum(rows: torch.Tensor, dest: torch.Tensor, weights: torch.Tensor | None, k: int, round_each: bool = False):
    """``y[t] = sum_j weights[t*k+j] * rows[dest[t*k+j]]`` in route order ``j = 0..k-1`` (fp32 accumulation, one writer
    per element: deterministic). Routes with ``dest < 0`` are skipped."""
    _checks.index_range("gather_sum", "dest", dest, upper=rows.shape[0], lower=-(1 << 31))
    T, H = dest.numel() // k, rows.shape[-1]
    if rows.is_cuda and rows.dtype == torch.bfloat16 and H % 8 == 0:
        y = torch.empty(T, H, dtype=rows.dtype, device=rows.device)
        w = None if weights is None else weights.reshape(-1).float().contiguous()
        rc = _lib.lib().sb_moe_gather_sum(P(rows.contiguous()), P(dest), P(w), P(y), T, k, H, int(round_each), _lib.stream())
        _lib.check(rc, "sb_moe_gather_sum")
        return y
    d = dest.view(T, k).long()
    w = torch.ones(T, k, device=rows.device) if weights is None else weights.reshape(T, k).float()
    acc = torch.zeros(T, H, dtype=torch.float32, device=rows.device)
    for j in range(k):
        ok = (d[:, j] >= 0).float()[:, None]
        acc = acc + ok * w[:, j, None] * rows[d[:, j].clamp_min(0)].float()
        if round_each:
            acc = acc.to(rows.dtype).float()
    return acc.to(rows.dtype)


def route_weight_grad(rows: torch.Tensor, dest: torch.Tensor, dy: torch.Tensor, k: int) -> torch.Tensor:
    """``dw[s] = <rows[dest[s]], dy[s // k]>`` (0 where ``dest[s] < 0``)."""
    if rows.is_cuda and rows.dtype == torch.bfloat16 and rows.shape[-1] % 8 == 0:
        dw = torch.empty(dest.numel(), dtype=torch.float32, device=rows.device)
        rc = _lib.lib().sb_moe_route_weight_grad(P(rows.contiguous()), P(dest), P(dy.contiguous()), P(dw), dest.numel(), k,
                                                 rows.shape[-1], _lib.stream())  # fmt: skip
        _lib.check(rc, "sb_moe_route_weight_grad")
        return dw
    tok = torch.arange(dest.numel(), device=dest.device) // k
    return (rows[dest.clamp_min(0).long()].float() * dy[tok].float()).sum(-1) * (dest >= 0).float()


class _ScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dest, k, num_rows):
        ctx.save_for_backward(dest)
        ctx.k = k
        return scatter_rows(x, dest, k, num_rows)

    @staticmethod
    def backward(ctx, g):
        (dest,) = ctx.saved_tensors
        return gather_sum(g.contiguous(), dest, None, ctx.k), None, None, None


class _GatherSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows, dest, weights, k):
        ctx.save_for_backward(rows, dest, weights)
        ctx.k = k
        return gather_sum(rows, dest, weights, k)

    @staticmethod
    def backward(ctx, dy):
        rows, dest, weights = ctx.saved_tensors
        dy = dy.contiguous()
        # d rows[dest[s]] = w[s] * dy[s // k]: a scatter of the scaled token gradients (each slot owns its row)
        scaled = (dy.float().repeat_interleave(ctx.k, dim=0) * weights.reshape(-1, 1).float()).to(dy.dtype)
        d_rows = scatter_rows(scaled, dest, 1, rows.shape[0])
        return d_rows, None, route_weight_grad(rows, dest, dy, ctx.k).view_as(weights).to(weights.dtype), None


def permute_tokens(x, dest, k: int, num_rows: int):
    """Differentiable ``scatter_rows`` (gradient: route-ordered ``gather_sum``)."""
    return _ScatterRows.apply(x, dest, k, num_rows)


def combine_routes(rows, dest, weights, k: int):
    """Differentiable weighted ``gather_sum`` (gradients for the rows and for the routing weights)."""
    return _GatherSum.apply(rows, dest, weights, k)


class PaddedLayout:
    """Row bookkeeping for ``counts[e]`` rows per expert, each segment starting at a multiple of 128."""

    def __init__(self, counts: list[int], device):
        self.counts = [int(c) for c in counts]
        self.padded = [-(-c // TILE) * TILE for c in self.counts]
        self.num_experts, self.rows, self.rows_padded = len(counts), sum(self.counts), sum(self.padded)
        starts, pstarts, s, ps = [], [], 0, 0
        for c, pc in zip(self.counts, self.padded):
            starts.append(s)
            pstarts.append(ps)
            s, ps = s + c, ps + pc
        self.starts, self.padded_starts = starts, pstarts
        cnt = torch.tensor(self.counts, dtype=torch.long)
        shift = torch.repeat_interleave(torch.tensor([p - q for p, q in zip(pstarts, starts)], dtype=torch.long), cnt)
        self.dest = (torch.arange(self.rows, dtype=torch.long) + shift).to(device)  # sorted row -> padded row
        tiles = torch.tensor([pc // TILE for pc in self.padded], dtype=torch.long)
        self.tile_expert = torch.repeat_interleave(torch.arange(self.num_experts), tiles).to(device=device, dtype=torch.int32)

    def pad(self, x: torch.Tensor) -> torch.Tensor:
        return x.new_zeros(self.rows_padded, x.shape[-1]).index_copy(0, self.dest, x)

    def unpad(self, xp: torch.Tensor) -> torch.Tensor:
        return xp.index_select(0, self.dest)


class DeviceLayout:
    """The same padded layout built entirely on the device from the router's choices: no host synchronisation, static
    shapes (the row count is the worst case ``T*k + E*127`` rounded up to a tile), so it can live inside a CUDA graph.

    ``idx``: [T, k] expert ids. Rows of the padded buffer hold token ``order // k`` for the sorted assignment ``order``;
    tiles past the last used row are zero rows attached to the last expert (they cost a little compute, nothing else).
    """

    def __init__(self, idx: torch.Tensor, num_experts: int, first_expert: int = 0):
        """``num_experts`` experts live here, global ids ``first_expert ...``; routes to other experts get no row
        (``slot_dest = -1``: the permutation kernels skip them), which is all expert parallelism needs when the
        activations are replicated over the group and the outputs are summed over it afterwards."""
        T, k = idx.shape
        dev = idx.device
        flat = idx.reshape(-1).long() - first_expert
        here = (flat >= 0) & (flat < num_experts)
        key = torch.where(here, flat, torch.full_like(flat, num_experts))  # routes served elsewhere sort to the end
        self.k, self.num_experts = k, num_experts
        self.order = torch.argsort(key, stable=True)  # assignments grouped by expert, token order kept inside a group
        sorted_e = key.index_select(0, self.order)
        # counts by scatter-add: fixed output size, no host synchronisation (bincount reads its maximum on the host)
        counts = torch.zeros(num_experts + 1, dtype=torch.long, device=dev).scatter_add_(0, key, torch.ones_like(key))[:num_experts]
        padded = (counts + (TILE - 1)) // TILE * TILE
        pend = torch.cumsum(padded, 0)
        shift = torch.cat([(pend - padded) - (torch.cumsum(counts, 0) - counts), torch.zeros(1, dtype=torch.long, device=dev)])
        dest = torch.arange(flat.numel(), device=dev) + shift.index_select(0, sorted_e)
        self.dest = torch.where(sorted_e < num_experts, dest, torch.full_like(dest, -1))
        # the same destinations in slot order (slot s = token s // k, route s % k): what the permutation kernels index by
        self.slot_dest = torch.empty(flat.numel(), dtype=torch.int32, device=dev)
        self.slot_dest[self.order] = self.dest.to(torch.int32)
        self.rows_padded = -(-(flat.numel() + num_experts * (TILE - 1)) // TILE) * TILE
        tiles = torch.arange(self.rows_padded // TILE, device=dev) * TILE
        self.tile_expert = torch.searchsorted(pend, tiles, right=True).clamp_(max=num_experts - 1).to(torch.int32)
        self.token = self.order // k

    def pad(self, x: torch.Tensor) -> torch.Tensor:
        """[T, H] token activations -> [rows_padded, H] expert-sorted, zero padded."""
        return scatter_rows(x, self.slot_dest, self.k, self.rows_padded)

    def combine(self, y_padded: torch.Tensor, probs: torch.Tensor, T: int) -> torch.Tensor:
        """Weighted sum of each token's k expert outputs, in route order with fp32 accumulation -> [T, H]."""
        return gather_sum(y_padded, self.slot_dest, probs, self.k)


def stacked_view(tensors: list[torch.Tensor]) -> torch.Tensor | None:
    """``[E, *shape]`` view over ``tensors`` without a copy when they sit back to back in one storage, else None."""
    t0 = tensors[0]
    if not all(t.is_contiguous() and t.shape == t0.shape and t.dtype == t0.dtype for t in tensors):
        return None
    step = t0.numel() * t0.element_size()
    base = t0.data_ptr()
    if any(t.data_ptr() != base + i * step for i, t in enumerate(tensors)):
        return None
    try:
        return torch.empty(0, dtype=t0.dtype, device=t0.device).set_(
            t0.untyped_storage(), t0.storage_offset(), (len(tensors), *t0.shape))  # fmt: skip
    except RuntimeError:  # the storage ends before the last tensor: the tensors do not share it after all
        return None


def _stack(weights: list[torch.Tensor]) -> torch.Tensor:
    datas = [w.detach() for w in weights]
    v = stacked_view(datas)
    return v if v is not None else torch.stack(datas)


def grouped_gemm(a: torch.Tensor, w: torch.Tensor, lay, *, b_mn: bool = False, out_dtype=None) -> torch.Tensor:
    """``out[rows of e] = a[rows of e] @ w[e]^T`` (``b_mn`` False, w [E, N, K]) or ``@ w[e]`` (``b_mn`` True, w [E, K, N])."""
    E, R, C = w.shape
    M, K = a.shape
    N = C if b_mn else R
    assert M == lay.rows_padded and E == lay.num_experts and K == (R if b_mn else C)
    _checks.index_range("grouped_gemm", "tile_expert", lay.tile_expert, upper=E)
    out_dtype = out_dtype or a.dtype
    if not a.is_cuda:
        out = torch.zeros(M, N, dtype=torch.float32)
        for t, e in enumerate(lay.tile_expert.tolist()):  # tile by tile: all a layout has to provide is tile -> expert
            we = w[e].float()
            out[t * TILE : (t + 1) * TILE] = a[t * TILE : (t + 1) * TILE].float() @ (we if b_mn else we.t())
        return out.to(out_dtype)
    a = a.contiguous()
    w = w.contiguous()
    out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    if M == 0:
        return out
    boff = lay.tile_expert * R  # first row of the tile's expert in the [E * R, C] stack
    from slime_b200.ops import _pick_bn

    rc = _lib.lib().sb_gemm_bf16_grouped(
        P(a), P(w), P(out), P(boff), M, N, K, E, a.stride(0), w.stride(1), out.stride(0), int(b_mn),
        int(out_dtype == torch.float32), _pick_bn(M, N), P(_lib.status_word(a.device)), _lib.sm_count(a.device), _lib.stream(),
    )  # fmt: skip
    _lib.check(rc, "sb_gemm_bf16_grouped")
    return out


def grouped_gemm_fp8(a: torch.Tensor, w_q: torch.Tensor, w_scale: torch.Tensor, lay, out_dtype=torch.bfloat16) -> torch.Tensor:
    """``out[rows of e] = a[rows of e] @ dequant(w_q[e], w_scale[e])^T`` for block-quantised expert weights.

    ``a`` [rows_padded, K] bf16 is quantised here to e4m3 with one scale per row and 128-wide K group; ``w_q`` [E, N, K]
    e4m3 with ``w_scale`` [E, ceil(N/128), K/128] (128 x 128 blocks, as block-fp8 checkpoints store them). One launch
    of the tcgen05 fp8 kernel over all experts; on CPU the dequantised fp32 product per tile. Same role as the grouped
    fp8 GEMM of the reference's rollout engines (slime/backends/megatron_utils/alignment/deepgemm_moe_forward.py:371-468).
    """
    from slime_b200 import ops

    E, N, K = w_q.shape
    M = a.shape[0]
    assert M == lay.rows_padded and E == lay.num_experts and a.shape[1] == K and K % 128 == 0
    a_q, a_s, a_st = ops.fp8_act_quant(a)
    if not a.is_cuda:
        out = torch.zeros(M, N, dtype=torch.float32)
        a_f = a_q.float() * a_s.repeat_interleave(128, 1)
        for t, e in enumerate(lay.tile_expert.tolist()):
            we = ops.reference.block_fp8_dequant(w_q[e], w_scale[e], (128, 128), torch.float32)
            out[t * TILE : (t + 1) * TILE] = a_f[t * TILE : (t + 1) * TILE] @ we.t()
        return out.to(out_dtype)
    out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    if M == 0:
        return out
    boff = lay.tile_expert * N
    rc = _lib.lib().sb_gemm_fp8_grouped(
        P(a_q), P(w_q), P(a_st), P(w_scale), P(out), P(boff), M, N, K, E, a_q.stride(0), w_q.stride(1), out.stride(0),
        int(out_dtype == torch.float32), P(_lib.status_word(a.device)), _lib.sm_count(a.device), _lib.stream(),
    )  # fmt: skip
    _lib.check(rc, "sb_gemm_fp8_grouped")
    return out


class _GroupedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, lay, *weights):
        ctx.lay, ctx.weights = lay, weights
        ctx.save_for_backward(x)
        return grouped_gemm(x, _stack(list(weights)), lay)

    @staticmethod
    def backward(ctx, dy):
        from slime_b200.ops import gemm

        (x,) = ctx.saved_tensors
        lay, weights = ctx.lay, ctx.weights
        dy = dy.contiguous()
        dx = grouped_gemm(dy, _stack(list(weights)), lay, b_mn=True) if ctx.needs_input_grad[0] else None
        dws = []
        for e, w in enumerate(weights):
            if not ctx.needs_input_grad[2 + e]:
                dws.append(None)
                continue
            s, n = lay.padded_starts[e], lay.counts[e]
            main_grad = getattr(w, "main_grad", None)
            if n == 0:
                dws.append(None if main_grad is not None else torch.zeros_like(w))
            elif main_grad is not None:
                gemm(dy[s : s + n], x[s : s + n], a_mn=True, b_mn=True, out=main_grad, accumulate=True)
                w.grad_added_to_main_grad = True
                dws.append(None)
            else:
                dws.append(gemm(dy[s : s + n], x[s : s + n], a_mn=True, b_mn=True, out_dtype=w.dtype))
        return (dx, None, *dws)


def grouped_linear(x_padded: torch.Tensor, lay: PaddedLayout, weights: list[torch.Tensor]) -> torch.Tensor:
    """Differentiable ``y[rows of e] = x[rows of e] @ weights[e]^T`` on the padded layout."""
    return _GroupedLinear.apply(x_padded, lay, *weights)
