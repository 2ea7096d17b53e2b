"""Block-fp8 (e4m3, 128 x 128 scale blocks) weight buffers of the rollout engine.

``--sglang-quantization fp8`` keeps the large matrices (fused qkv, attention output, MLP / expert projections) as e4m3
bytes plus one fp32 ``scale_inv`` per 128 x 128 block, the format of block-fp8 checkpoints
(tools/convert_hf_to_fp8.py:41-77 in the reference) and of the fp8 weight-sync branch
(slime/backends/megatron_utils/megatron_to_hf/processors/quantizer_fp8.py in the reference). A buffer accepts

* bf16 rows (a bf16 checkpoint or a bf16 weight sync: quantised on arrival, "online" quantisation), or
* e4m3 rows and, under the ``*.weight_scale_inv`` name, their scale rows (already quantised by the sender).

Row ranges written separately (q / k / v into the fused qkv buffer, gate / up, one expert of a stack) must start on a
multiple of 128 so that no scale block straddles two of them; ``supported`` says whether a buffer of a given shape can
be kept in fp8 at all (the engine keeps the others in bf16). Activations are quantised per row and 128-wide K group
right before the GEMM (``ops.fp8_act_quant``), the product runs on the tcgen05 fp8 kernel with per-K-block promotion.
"""

from __future__ import annotations

import torch

from slime_b200 import ops

BLOCK = 128


def supported(rows: int, cols: int, row_parts: tuple[int, ...] = ()) -> bool:
    """A [rows, cols] matrix whose separately written row ranges start at ``row_parts`` can live in fp8."""
    return cols % BLOCK == 0 and all(r % BLOCK == 0 for r in row_parts)


class Fp8Weight:
    """``[..., N, K]`` e4m3 with ``[..., ceil(N/128), K/128]`` fp32 inverse scales (a leading expert dimension is allowed)."""

    def __init__(self, *shape: int, device):
        *lead, n, k = shape
        assert k % BLOCK == 0
        self.q = torch.zeros(*shape, dtype=torch.float8_e4m3fn, device=device)
        self.scale = torch.ones(*lead, -(-n // BLOCK), k // BLOCK, dtype=torch.float32, device=device)

    # tensor-like surface used by the engine's bookkeeping
    @property
    def shape(self):
        return self.q.shape

    def dim(self) -> int:
        return self.q.dim()

    def tensors(self):
        return (self.q, self.scale)

    def __getitem__(self, e: int) -> "Fp8Weight":
        """Expert ``e`` of a stack, sharing storage."""
        out = object.__new__(Fp8Weight)
        out.q, out.scale = self.q[e], self.scale[e]
        return out

    def load_rows(self, r0: int, t: torch.Tensor):
        """Rows ``[r0, r0 + t.shape[0])`` from a bf16 / fp32 tensor (quantised here) or from e4m3 bytes (copied; their
        scales arrive through ``load_scale_rows``)."""
        assert r0 % BLOCK == 0, "separately written row ranges must start on a scale-block boundary"
        n = t.shape[0]
        if t.dtype == torch.float8_e4m3fn:
            self.q[r0 : r0 + n].copy_(t)
            return
        t = t.to(self.q.device)
        if t.is_cuda:
            t = t.to(torch.bfloat16)  # what the quantisation kernel reads
        b0 = r0 // BLOCK
        ops.block_fp8_quant(t, (BLOCK, BLOCK), out=(self.q[r0 : r0 + n], self.scale[b0 : b0 + -(-n // BLOCK)]))

    def load_scale_rows(self, r0: int, s: torch.Tensor):
        assert r0 % BLOCK == 0
        self.scale[r0 // BLOCK : r0 // BLOCK + s.shape[0]].copy_(s.to(self.scale.device, torch.float32))

    def copy_(self, t: torch.Tensor):
        self.load_rows(0, t)
        return self

    def dequant(self, dtype=torch.bfloat16) -> torch.Tensor:
        if self.q.dim() == 2:
            return ops.block_fp8_dequant(self.q, self.scale, (BLOCK, BLOCK), dtype)
        return torch.stack([ops.block_fp8_dequant(q, s, (BLOCK, BLOCK), dtype) for q, s in zip(self.q, self.scale)])

    def fill_random_(self, std: float, generator=None):
        """Random-init (``load_format=dummy``): quantise a normal draw block by block, 4096 rows at a time."""
        flat_q = self.q.view(-1, *self.q.shape[-2:])
        flat_s = self.scale.view(-1, *self.scale.shape[-2:])
        for q, s in zip(flat_q, flat_s):
            for r in range(0, q.shape[0], 4096):
                n = min(4096, q.shape[0] - r)
                w = torch.empty(n, q.shape[1], dtype=torch.float32, device=q.device).normal_(0, std, generator=generator)
                w = w.to(torch.bfloat16) if w.is_cuda else w
                ops.block_fp8_quant(w, (BLOCK, BLOCK), out=(q[r : r + n], s[r // BLOCK : r // BLOCK + -(-n // BLOCK)]))


def linear(x: torch.Tensor, w, bias=None, out_dtype=None, out=None) -> torch.Tensor:
    """``x @ w^T (+ bias)`` for a bf16 tensor or an ``Fp8Weight``."""
    if not isinstance(w, Fp8Weight):
        return ops.gemm(x, w, bias=bias, out_dtype=out_dtype, out=out)
    q, s, st = ops.fp8_act_quant(x)
    y = ops.fp8_block_gemm(q, s, w.q, w.scale, out_dtype=out_dtype or x.dtype, a_scale_t=st)
    if bias is not None:
        y = y + bias.to(y.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y
