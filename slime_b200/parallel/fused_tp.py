"""Tensor-parallel all-reduce + residual add + RMSNorm as one kernel over NVLink peer memory (``csrc/tp_fused.cu``).

In a decoder layer every row-parallel projection (attention output, MLP down) is followed by the same three steps:
sum the partial products over the tensor-parallel ranks, add the residual stream, normalise for the next block.
``FusedAllReduceNorm`` does them in one launch and without NCCL:

    ar = FusedAllReduceNorm(tp_group, max_tokens, hidden, device)
    ar.begin_forward()                        # once per forward pass (one bounded barrier)
    out = ar.partial(T)                       # [T, hidden] bf16 view: the GEMM writes its partial product here
    ops.gemm(x, w_row_parallel, out=out)
    normed, residual = ar(T, residual, norm_weight, eps)

The partial products live in two alternating symmetric buffers; a kernel reads the peers' rows directly (plain P2P
loads summed in rank order, or NVSwitch ``multimem.ld_reduce``), so every rank ends up with identical values. The launch
arguments never change between calls with the same ``T`` (epochs live in device memory), hence a decode step that
contains these calls can be captured in a CUDA graph; ``begin_forward`` restarts the alternation, so any number of
calls per forward pass works. ``usable()`` says whether the fast path exists here; callers fall back to
``dist.all_reduce`` + ``ops.rmsnorm``.
"""

from __future__ import annotations

import ctypes
import logging
import os

import torch

from slime_b200.parallel.fused_dp import SymmetricStorage, symmetric_memory_usable

logger = logging.getLogger(__name__)
MAX_BLOCKS = 148


def usable(group_size: int, device, hidden: int) -> bool:
    if os.environ.get("SLIME_B200_DISABLE_FUSED_TP") == "1" or os.environ.get("SLIME_B200_LIBRARY_OPS") == "1":
        return False
    return symmetric_memory_usable(group_size, device) and hidden % 8 == 0 and hidden <= 8192


class FusedAllReduceNorm:
    def __init__(self, group, max_tokens: int, hidden: int, device):
        from slime_b200.ops import _lib

        self._lib = _lib
        self.hidden, self.max_tokens, self.device = hidden, max_tokens, torch.device(device)
        self.bufs = [SymmetricStorage(max_tokens * hidden, torch.bfloat16, device, group) for _ in range(2)]
        self.flags = SymmetricStorage(MAX_BLOCKS * 8, torch.int32, device, group)
        self.world, self.rank = self.flags.world, self.flags.rank
        self.epochs = torch.zeros(MAX_BLOCKS, dtype=torch.int32, device=device)
        self.use_mc = all(b.mc_ptr for b in self.bufs) and os.environ.get("SLIME_B200_DISABLE_MULTIMEM") != "1"
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*self.flags.ptrs)
        self._pads = (ctypes.c_void_p * self.world)(*self.flags.pad_ptrs)
        self._pad_base = self.flags.pad_words - 32  # away from the data-parallel barrier's words and torch's own
        self._barrier_counter = torch.zeros(1, dtype=torch.int32, device=device)  # device-side epoch: graph-safe
        self._which = 0
        torch.cuda.synchronize(self.device)
        import torch.distributed as dist

        dist.barrier(group=group)  # every rank's flags and epochs are zero before anyone raises one
        logger.info("fused tensor-parallel all-reduce+norm: %d ranks, %s", self.world,
                    "NVSwitch multimem" if self.use_mc else "P2P loads")  # fmt: skip

    def begin_forward(self) -> None:
        """All ranks have finished the previous forward pass: both partial buffers are free again."""
        lib, P = self._lib.lib(), self._lib.ptr
        rc = lib.sb_symm_barrier_dev(self._pads, self.rank, self.world, P(self._barrier_counter), self._pad_base,
                                     P(self._lib.status_word(self.device)), self._lib.stream())  # fmt: skip
        self._lib.check(rc, "sb_symm_barrier_dev")
        self._which = 0

    def partial(self, T: int) -> torch.Tensor:
        assert T <= self.max_tokens, f"{T} tokens exceed the buffer ({self.max_tokens})"
        return self.bufs[self._which].tensor[: T * self.hidden].view(T, self.hidden)

    def __call__(self, T: int, residual, weight, eps: float, out=None, res_out=None):
        """(normed, new_residual) from the partial products in the current buffer; then switches buffers."""
        lib, P = self._lib.lib(), self._lib.ptr
        buf = self.bufs[self._which]
        y = out if out is not None else torch.empty(T, self.hidden, dtype=torch.bfloat16, device=self.device)
        r = res_out if res_out is not None else torch.empty(T, self.hidden, dtype=torch.bfloat16, device=self.device)
        rc = lib.sb_tp_ar_add_rmsnorm(buf.c_ptrs(self.use_mc), self._flag_ptrs, P(self.epochs), P(residual), P(weight), P(y),
                                      P(r), T, self.hidden, float(eps), self.rank, self.world, int(self.use_mc),
                                      P(self._lib.status_word(self.device)), self._lib.stream())  # fmt: skip
        self._lib.check(rc, "sb_tp_ar_add_rmsnorm")
        self._which ^= 1
        return y, r


class _SymmBarrier:
    """Bounded device-side barrier over a symmetric allocation's signal pad (epoch kept on the device: graph safe)."""

    def __init__(self, storage: SymmetricStorage, word_offset_from_top: int, device):
        from slime_b200.ops import _lib

        self._lib = _lib
        self.world, self.rank = storage.world, storage.rank
        self._pads = (ctypes.c_void_p * self.world)(*storage.pad_ptrs)
        self._base = storage.pad_words - word_offset_from_top
        self._counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.device = device

    def __call__(self):
        lib, P = self._lib.lib(), self._lib.ptr
        rc = lib.sb_symm_barrier_dev(self._pads, self.rank, self.world, P(self._counter), self._base,
                                     P(self._lib.status_word(self.device)), self._lib.stream())  # fmt: skip
        self._lib.check(rc, "sb_symm_barrier_dev")


class GatherGemm:
    """All-gather fused into the GEMM: ``gather_rows(x_0 .. x_{n-1}) @ op(W)`` in one kernel (``GatherA`` in
    ``csrc/gemm_sm100.cu``).

    Sequence-parallel column-parallel linears (QKV, gate/up) and the input-gradient GEMM of row-parallel ones take an
    operand that is sharded by rows over the tensor-parallel ranks. Each rank puts its shard into a symmetric buffer;
    after one bounded barrier the GEMM kernel on every rank starts on its own rows while a dedicated warp in each CTA
    pulls the peers' rows once into local memory (plain loads over NVLink) and releases them to the tile loop block by
    block. Returns the product and the gathered operand (the backward's weight-gradient GEMM reads it again).

    ``rows`` (per rank) must be a multiple of 128. Two shard buffers alternate, so a rank may refill its shard for the
    next call while slower ranks still read the previous one; the barrier at the start of every call keeps two calls
    apart.
    """

    def __init__(self, group, max_rows_per_rank: int, k: int, device):
        from slime_b200.ops import _lib

        self._lib = _lib
        self.k, self.max_rows, self.device = k, max_rows_per_rank, torch.device(device)
        self.bufs = [SymmetricStorage(max_rows_per_rank * k, torch.bfloat16, device, group) for _ in range(2)]
        self.world, self.rank = self.bufs[0].world, self.bufs[0].rank
        self._barrier = _SymmBarrier(self.bufs[0], 48, self.device)
        self._which = 0
        torch.cuda.synchronize(self.device)
        import torch.distributed as dist

        dist.barrier(group=group)

    def fits(self, rows: int, k: int) -> bool:
        return k == self.k and rows <= self.max_rows and rows % 128 == 0

    def __call__(self, x_local: torch.Tensor, weight: torch.Tensor, bias=None, b_mn: bool = False):
        """``x_local`` [rows, K] bf16 -> (``[world * rows, N]`` bf16, gathered ``[world * rows, K]``). ``weight`` is
        [N, K] (``b_mn`` False) or [K, N] (``b_mn`` True: the product is with the transpose-free stored matrix)."""
        from slime_b200.ops import _pick_bn

        lib, P = self._lib.lib(), self._lib.ptr
        rows, k = x_local.shape
        assert self.fits(rows, k), f"shard [{rows}, {k}] does not fit (max rows {self.max_rows}, K {self.k}, rows % 128)"
        buf = self.bufs[self._which]
        buf.tensor[: rows * k].view(rows, k).copy_(x_local)
        m = rows * self.world
        n = weight.shape[1] if b_mn else weight.shape[0]
        gathered = torch.empty(m, k, dtype=torch.bfloat16, device=self.device)
        gathered[self.rank * rows : (self.rank + 1) * rows].copy_(x_local)
        counters = torch.zeros(m // 128, dtype=torch.int32, device=self.device)
        out = torch.empty(m, n, dtype=torch.bfloat16, device=self.device)
        self._barrier()  # every rank's shard is complete
        peers = (ctypes.c_void_p * self.world)(*buf.ptrs)
        fn = self._lib.bind("sb_gemm_bf16_gather_a", [self._lib.P, self._lib.I, self._lib.I, self._lib.I, self._lib.P, self._lib.P,
                                                      ctypes.c_uint, self._lib.P, self._lib.P, self._lib.P] + [self._lib.I] * 6
                            + [self._lib.P, self._lib.I, self._lib.P])  # fmt: skip
        rc = fn(peers, self.world, self.rank, rows, P(gathered), P(counters), 128 // 4, P(weight), P(out), P(bias), n, k,
                weight.stride(0), out.stride(0), int(b_mn), _pick_bn(m, n), P(self._lib.status_word(self.device)),
                self._lib.sm_count(self.device), self._lib.stream())  # fmt: skip
        self._lib.check(rc, "sb_gemm_bf16_gather_a")
        self._which ^= 1
        return out, gathered


class GemmReduceScatter:
    """GEMM fused with the reduce-scatter of its output rows (``ScatterC`` in ``csrc/gemm_sm100.cu``).

    Sequence-parallel row-parallel linears (attention output, MLP down) and the input-gradient GEMM of column-parallel
    ones produce a full ``[M, N]`` partial product on every rank, of which rank ``o`` needs the sum of rows
    ``[o * M / n, (o + 1) * M / n)``. The kernel's epilogue stores every tile straight into the owning rank's receive
    buffer (TMA stores over NVLink for the peers' tiles, which are computed first) and, once its share of the GEMM is
    done, sums the slots of the tiles it owns as their flags arrive. One launch, no NCCL, rank-order summation.
    Two receive buffers alternate: a rank may be one call ahead of its peers, never two (it needs their tiles to finish).
    """

    def __init__(self, group, max_rows_per_rank: int, n: int, device):
        from slime_b200.ops import _lib

        self._lib = _lib
        self.group = group
        self.n, self.max_rows, self.device = n, max_rows_per_rank, torch.device(device)
        probe = SymmetricStorage(8, torch.int32, device, group)
        self.world, self.rank = probe.world, probe.rank
        self.recv = [SymmetricStorage(self.world * max_rows_per_rank * n, torch.bfloat16, device, group) for _ in range(2)]
        nflags = (max_rows_per_rank // 128) * (-(-n // 128)) * self.world * 4
        self.flags = [SymmetricStorage(nflags, torch.int32, device, group) for _ in range(2)]
        self.epochs = [0, 0]
        self._which = 0
        torch.cuda.synchronize(self.device)
        import torch.distributed as dist

        dist.barrier(group=group)  # every rank's flags are zero before anyone raises one

    def fits(self, m: int, n: int) -> bool:
        return n == self.n and m % (self.world * 128) == 0 and m // self.world <= self.max_rows

    def profitable(self, k: int) -> bool:
        """Whether the single-kernel path beats GEMM + NCCL reduce-scatter for an inner dimension ``k`` (see __call__)."""
        if os.environ.get("SLIME_B200_FORCE_FUSED_RS") == "1":
            return True
        return self.world == 2 and k >= 4096

    def __call__(self, a: torch.Tensor, weight: torch.Tensor, b_mn: bool = False):
        """``a`` [M, K] bf16, ``weight`` [N, K] (or [K, N] with ``b_mn``) -> this rank's ``[M / world, N]`` bf16 rows of the
        sum over ranks of ``a @ op(weight)``."""
        from slime_b200.ops import _pick_bn

        lib, P = self._lib.lib(), self._lib.ptr
        m, k = a.shape
        n = weight.shape[1] if b_mn else weight.shape[0]
        assert self.fits(m, n), f"product [{m}, {n}] does not fit (max rows per rank {self.max_rows}, N {self.n})"
        if a.stride(-1) != 1 or a.stride(0) % 8:
            a = a.contiguous()
        if not self.profitable(k):
            # Measured at M 9216, N 2560 (device time, max over ranks): 2 GPUs, K 4864: fused 213 us, GEMM + NCCL
            # reduce-scatter 238 us; K 2048: 177 vs 150 us. 4 GPUs, K 2432: 202 vs 171 us; K 1024: 285 vs 130 us. A short K
            # leaves too little GEMM to hide the tile stores and the owner's reduction behind, so those shapes keep NCCL.
            import torch.distributed as dist

            from slime_b200 import ops

            part = ops.gemm(a, weight, b_mn=b_mn)
            out = torch.empty(m // self.world, n, dtype=torch.bfloat16, device=self.device)
            dist.reduce_scatter_tensor(out, part, group=self.group)
            return out
        w = self._which
        self.epochs[w] += 1
        out = torch.empty(m // self.world, n, dtype=torch.bfloat16, device=self.device)
        recv = (ctypes.c_void_p * self.world)(*self.recv[w].ptrs)
        flags = (ctypes.c_void_p * self.world)(*self.flags[w].ptrs)
        fn = self._lib.bind("sb_gemm_bf16_scatter_c", [self._lib.P, self._lib.P] + [self._lib.I] * 6 + [self._lib.P, self._lib.P,
                                                       self._lib.I, self._lib.I, self._lib.P, self._lib.I, ctypes.c_uint, self._lib.I,
                                                       self._lib.P, self._lib.I, self._lib.P])  # fmt: skip
        rc = fn(P(a), P(weight), m, n, k, a.stride(0), weight.stride(0), int(b_mn), recv, flags, self.world, self.rank, P(out),
                out.stride(0), self.epochs[w], _pick_bn(m, n), P(self._lib.status_word(self.device)),
                self._lib.sm_count(self.device), self._lib.stream())  # fmt: skip
        self._lib.check(rc, "sb_gemm_bf16_scatter_c")
        self._which ^= 1
        return out


class FusedSequenceParallelLinears:
    """The two fused collectives a sequence-parallel transformer layer needs, shared by every layer of a model (all
    gathered operands and scattered products have ``hidden`` columns), with their autograd rules:

        column(x_local, W, b)   = gather(x) @ W^T + b        backward: dx = reduce_scatter(dy @ W), dW += dy^T gather(x)
        row(x, W)               = reduce_scatter(x @ W^T)     backward: dx = gather(dy) @ W,        dW += gather(dy)^T x
    """

    def __init__(self, group, max_tokens: int, hidden: int, device):
        import torch.distributed as dist

        world = dist.get_world_size(group)
        rows = -(-(max_tokens + world * 128) // (world * 128)) * 128
        self.ag = GatherGemm(group, rows, hidden, device)
        self.rs = GemmReduceScatter(group, rows, hidden, device)
        self.world = world

    def fits(self, rows_local: int, hidden: int) -> bool:
        return self.ag.fits(rows_local, hidden) and self.rs.fits(rows_local * self.world, hidden)

    def column(self, x_local, weight, bias=None):
        return _FusedColumn.apply(x_local, weight, bias, self)

    def row(self, x, weight):
        return _FusedRow.apply(x, weight, self)


def _wgrad(dy, x, weight):
    """dW += dy^T x, straight into the fp32 main-grad buffer when the parameter has one."""
    from slime_b200 import ops

    main_grad = getattr(weight, "main_grad", None)
    if main_grad is not None:
        ops.gemm(dy, x, a_mn=True, b_mn=True, out=main_grad, accumulate=True)
        weight.grad_added_to_main_grad = True
        return None
    return ops.gemm(dy, x, a_mn=True, b_mn=True, out_dtype=weight.dtype)


class _FusedColumn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, weight, bias, fused):
        y, gathered = fused.ag(x_local, weight, bias)
        ctx.save_for_backward(gathered, weight)
        ctx.fused, ctx.has_bias = fused, bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        gathered, weight = ctx.saved_tensors
        dy = dy if dy.stride(-1) == 1 and dy.stride(0) % 8 == 0 else dy.contiguous()
        dx = ctx.fused.rs(dy, weight, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = _wgrad(dy, gathered, weight) if ctx.needs_input_grad[1] else None
        db = dy.float().sum(0).to(dy.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db, None


class _FusedRow(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, fused):
        ctx.save_for_backward(x, weight)
        ctx.fused = fused
        return fused.rs(x, weight)

    @staticmethod
    def backward(ctx, dy_local):
        x, weight = ctx.saved_tensors
        dx, dy = ctx.fused.ag(dy_local.contiguous(), weight, None, b_mn=True)
        dw = _wgrad(dy, x, weight) if ctx.needs_input_grad[1] else None
        return (dx if ctx.needs_input_grad[0] else None), dw, None


_LINEARS: dict = {}
_MAX_TOKENS = 16384  # capacity (packed tokens of a micro-batch) the shared buffers are sized for


def set_max_tokens(n: int) -> None:
    """Called by the trainer with ``--max-tokens-per-gpu`` before the first forward pass."""
    global _MAX_TOKENS
    _MAX_TOKENS = max(int(n), 256)


def sequence_parallel_linears(group, hidden: int, device, max_tokens: int | None = None):
    """The shared ``FusedSequenceParallelLinears`` of a tensor-parallel group (created on first use), or None where the
    fused path does not exist (CPU, one rank, no symmetric memory, SLIME_B200_DISABLE_FUSED_TP=1)."""
    import torch.distributed as dist

    if group is None or torch.device(device).type != "cuda" or not usable(dist.get_world_size(group), device, hidden):
        return None
    if os.environ.get("SLIME_B200_DISABLE_FUSED_TP_LINEAR") == "1":
        return None
    max_tokens = max_tokens or _MAX_TOKENS
    key = (id(group), hidden, torch.device(device).index)
    cur = _LINEARS.get(key)
    if cur is None or cur.ag.max_rows * cur.world < max_tokens:
        try:
            cur = FusedSequenceParallelLinears(group, max_tokens, hidden, device)
        except Exception as e:  # noqa: BLE001
            logger.warning("fused sequence-parallel linears unavailable (%r): using NCCL", e)
            return None
        _LINEARS[key] = cur
    return cur
