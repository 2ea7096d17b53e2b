"""Vision inputs: the image / video encoder, multi-axis rotary positions and their rotary tables.

``VisionTower`` is the Qwen3-VL / Qwen3.5 style encoder: every image (or video frame pair) arrives as rows of flattened
``temporal_patch x patch x patch`` pixel blocks with its grid ``(t, h, w)``; a linear patch embedding, a learned
position grid interpolated bilinearly to the image's size, ``depth`` pre-LayerNorm blocks of full (non-causal) attention
inside each frame with 2-D rotary embedding (first half of the rotary channels by row, second half by column), and a
merger that joins every ``merge x merge`` neighbourhood into one vector of the language model's width. The rows arrive
already ordered so that the ``merge**2`` patches of a neighbourhood are consecutive (that is how the image processor
emits them). Parameter names are those of the checkpoints (``patch_embed.proj``, ``pos_embed``,
``blocks.N.{norm1,norm2,attn.qkv,attn.proj,mlp.linear_fc1,mlp.linear_fc2}``, ``merger.{norm,linear_fc1,linear_fc2}``),
so tensors load by name. The tower is replicated over tensor-parallel ranks.

``mrope_position_ids`` gives the three position streams (temporal, height, width) of a packed token stream: text
tokens advance all three together, the tokens of an image keep the temporal index and spread over its merged grid, and
the text after an image continues from the largest index used so far. ``mrope_band_axes`` says which stream drives which
rotary frequency band (sections laid out one after another as in Qwen2-VL, or interleaved as in Qwen3-VL / Qwen3.5).

Same role as slime_plugins/models/qwen3_5_vl.py:18-133 and qwen3_5_vl_utils.py:60-157 in the reference, which wrap the
Transformers vision class; this tower is checked against that class in the tests.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class VisionConfig:
    depth: int = 2
    hidden_size: int = 64
    num_heads: int = 4
    intermediate_size: int = 128
    in_channels: int = 3
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 64
    num_position_embeddings: int = 2304
    hidden_act: str = "gelu_pytorch_tanh"
    deepstack_visual_indexes: list = field(default_factory=list)

    @classmethod
    def from_dict(cls, d: dict) -> "VisionConfig":
        names = {f.name for f in cls.__dataclass_fields__.values()}
        return cls(**{k: v for k, v in d.items() if k in names})

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size


def _replicated(t: torch.Tensor) -> nn.Parameter:
    p = nn.Parameter(t)
    p.tensor_model_parallel, p.partition_dim, p.partition_stride = False, -1, 1
    return p


class _Affine(nn.Module):
    """weight (+ bias) holder with the checkpoint's attribute names."""

    def __init__(self, *shape, bias=True, dtype, device, std=0.02, ones=False):
        super().__init__()
        w = torch.ones(*shape, dtype=dtype, device=device) if ones else torch.randn(*shape, dtype=dtype, device=device) * std
        self.weight = _replicated(w)
        self.bias = _replicated(torch.zeros(shape[0], dtype=dtype, device=device)) if bias else None


def _act(name: str):
    if name in ("gelu_pytorch_tanh", "gelu_tanh"):
        return lambda x: F.gelu(x, approximate="tanh")
    if name == "gelu":
        return F.gelu
    if name in ("silu", "swish"):
        return F.silu
    if name == "quick_gelu":
        return lambda x: x * torch.sigmoid(1.702 * x)
    raise ValueError(f"unknown activation {name!r}")


class VisionBlock(nn.Module):
    def __init__(self, c: VisionConfig, dtype, device):
        super().__init__()
        d = c.hidden_size
        self.norm1 = _Affine(d, dtype=dtype, device=device, ones=True)
        self.norm2 = _Affine(d, dtype=dtype, device=device, ones=True)
        self.attn = nn.Module()
        self.attn.qkv = _Affine(3 * d, d, dtype=dtype, device=device)
        self.attn.proj = _Affine(d, d, dtype=dtype, device=device)
        self.mlp = nn.Module()
        self.mlp.linear_fc1 = _Affine(c.intermediate_size, d, dtype=dtype, device=device)
        self.mlp.linear_fc2 = _Affine(d, c.intermediate_size, dtype=dtype, device=device)
        self.heads, self.act = c.num_heads, _act(c.hidden_act)

    def forward(self, x, cos, sin, frames: list[int]):
        T, d = x.shape
        h = F.layer_norm(x, (d,), self.norm1.weight, self.norm1.bias, 1e-6)
        q, k, v = F.linear(h, self.attn.qkv.weight, self.attn.qkv.bias).view(T, 3, self.heads, d // self.heads).unbind(1)
        q, k = _rotate(q, cos, sin), _rotate(k, cos, sin)
        outs, a = [], 0
        for n in frames:  # full attention inside a frame, none across frames
            qs, ks, vs = (t[a : a + n].transpose(0, 1) for t in (q, k, v))
            outs.append(F.scaled_dot_product_attention(qs, ks, vs).transpose(0, 1))
            a += n
        ctx = torch.cat(outs).reshape(T, d)
        x = x + F.linear(ctx, self.attn.proj.weight, self.attn.proj.bias)
        h = F.layer_norm(x, (d,), self.norm2.weight, self.norm2.bias, 1e-6)
        return x + F.linear(self.act(F.linear(h, self.mlp.linear_fc1.weight, self.mlp.linear_fc1.bias)),
                            self.mlp.linear_fc2.weight, self.mlp.linear_fc2.bias)  # fmt: skip


def _rotate(x, cos, sin):
    """Half-split rotary over the whole head width: x [T, H, D], cos / sin [T, D]."""
    xf = x.float()
    a, b = xf[..., : xf.shape[-1] // 2], xf[..., xf.shape[-1] // 2 :]
    return (xf * cos[:, None, :] + torch.cat([-b, a], dim=-1) * sin[:, None, :]).to(x.dtype)


class VisionTower(nn.Module):
    def __init__(self, c: VisionConfig, dtype=torch.float32, device="cpu"):
        super().__init__()
        self.c = c
        d = c.hidden_size
        self.patch_embed = nn.Module()
        self.patch_embed.proj = _Affine(d, c.in_channels, c.temporal_patch_size, c.patch_size, c.patch_size, dtype=dtype, device=device)
        self.pos_embed = _Affine(c.num_position_embeddings, d, bias=False, dtype=dtype, device=device)
        self.blocks = nn.ModuleList([VisionBlock(c, dtype, device) for _ in range(c.depth)])
        self.merger = nn.Module()
        big = d * c.spatial_merge_size**2
        self.merger.norm = _Affine(d, dtype=dtype, device=device, ones=True)
        self.merger.linear_fc1 = _Affine(big, big, dtype=dtype, device=device)
        self.merger.linear_fc2 = _Affine(c.out_hidden_size, big, dtype=dtype, device=device)
        # "deepstack" (Qwen3-VL): the outputs of some intermediate blocks, each through a merger of its own (normalised
        # after the neighbourhoods are joined), are added to the language model's stream after its first layers
        self.deepstack_merger_list = nn.ModuleList()
        for _ in c.deepstack_visual_indexes:
            m = nn.Module()
            m.norm = _Affine(big, dtype=dtype, device=device, ones=True)
            m.linear_fc1 = _Affine(big, big, dtype=dtype, device=device)
            m.linear_fc2 = _Affine(c.out_hidden_size, big, dtype=dtype, device=device)
            self.deepstack_merger_list.append(m)
        self.side = int(math.isqrt(c.num_position_embeddings))

    @property
    def dtype(self):
        return self.pos_embed.weight.dtype

    def _merge_order(self, t: torch.Tensor, h: int, w: int) -> torch.Tensor:
        """Rows of an ``h x w`` grid (row-major) re-ordered so that each ``merge x merge`` neighbourhood is consecutive."""
        m = self.c.spatial_merge_size
        return t.view(h // m, m, w // m, m, -1).permute(0, 2, 1, 3, 4).reshape(h * w, -1)

    def _positions(self, grid: list[list[int]], device):
        """Per patch row: interpolated learned position vector and the (row, column) rotary angles."""
        c, side = self.c, self.side
        head = c.hidden_size // c.num_heads
        inv = 1.0 / (10000.0 ** (torch.arange(0, head // 2, 2, dtype=torch.float32, device=device) / (head // 2)))
        pos, ang = [], []
        table = self.pos_embed.weight
        for t, h, w in grid:
            ys, xs = torch.linspace(0, side - 1, h, device=device), torch.linspace(0, side - 1, w, device=device)
            y0, x0 = ys.floor().long(), xs.floor().long()
            y1, x1 = (y0 + 1).clamp_max(side - 1), (x0 + 1).clamp_max(side - 1)
            fy, fx = (ys - y0).to(table.dtype)[:, None, None], (xs - x0).to(table.dtype)[None, :, None]
            g = lambda yy, xx: table[(yy[:, None] * side + xx[None, :])]  # noqa: E731  [h, w, d]
            img = (g(y0, x0) * (1 - fy) * (1 - fx) + g(y0, x1) * (1 - fy) * fx + g(y1, x0) * fy * (1 - fx) + g(y1, x1) * fy * fx)
            pos.append(self._merge_order(img.reshape(h * w, -1), h, w).repeat(t, 1))
            rc = torch.stack(torch.meshgrid(torch.arange(h, device=device), torch.arange(w, device=device), indexing="ij"), -1)
            rc = self._merge_order(rc.reshape(h * w, 2), h, w).float()  # [h*w, 2] (row, column)
            a = torch.cat([rc[:, :1] * inv, rc[:, 1:] * inv], dim=-1)  # [h*w, head/2]
            ang.append(a.repeat(t, 1))
        ang = torch.cat(ang)
        ang = torch.cat([ang, ang], dim=-1)
        return torch.cat(pos), ang.cos(), ang.sin()

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor, with_deepstack: bool = False):
        """``pixel_values`` [patches, C * tp * p * p], ``grid_thw`` [images, 3] -> [patches / merge**2, out_hidden]; with
        ``with_deepstack`` also the list of same-shaped vectors for the language model's first layers."""
        c = self.c
        grid = [[int(v) for v in row] for row in grid_thw.tolist()]
        assert pixel_values.shape[0] == sum(t * h * w for t, h, w in grid), "pixel rows do not match the grids"
        x = F.linear(pixel_values.to(self.dtype).reshape(-1, c.patch_dim), self.patch_embed.proj.weight.reshape(c.hidden_size, -1),
                     self.patch_embed.proj.bias)  # fmt: skip
        pos, cos, sin = self._positions(grid, x.device)
        x = x + pos
        frames = [h * w for t, h, w in grid for _ in range(t)]
        big = c.hidden_size * c.spatial_merge_size**2
        extras = []
        for i, blk in enumerate(self.blocks):
            x = blk(x, cos, sin, frames)
            if i in c.deepstack_visual_indexes:
                m = self.deepstack_merger_list[c.deepstack_visual_indexes.index(i)]
                y = F.layer_norm(x.reshape(-1, big), (big,), m.norm.weight, m.norm.bias, 1e-6)
                y = F.gelu(F.linear(y, m.linear_fc1.weight, m.linear_fc1.bias))
                extras.append(F.linear(y, m.linear_fc2.weight, m.linear_fc2.bias))
        x = F.layer_norm(x, (c.hidden_size,), self.merger.norm.weight, self.merger.norm.bias, 1e-6)
        x = x.reshape(-1, big)
        x = F.gelu(F.linear(x, self.merger.linear_fc1.weight, self.merger.linear_fc1.bias))
        out = F.linear(x, self.merger.linear_fc2.weight, self.merger.linear_fc2.bias)
        return (out, extras) if with_deepstack else out


# ----------------------------------------------------------------------------------------- multi-axis rotary positions
def mrope_position_ids(input_ids: torch.Tensor, cu_seqlens, image_grid_thw=None, video_grid_thw=None, *, image_token_id: int,
                       video_token_id: int | None = None, spatial_merge_size: int = 2):  # fmt: skip
    """Position streams ``[3, T]`` (temporal, height, width) of a packed token stream and, per sequence, the amount by
    which the position of the next token exceeds... falls short of its index (``delta`` <= 0: decode positions are
    ``index + delta`` on all three axes). Every sequence restarts at 0. A run of ``image_token_id`` (or
    ``video_token_id``) tokens takes the next grid; a video grid with ``t`` frames is consumed as ``t`` one-frame runs
    (each frame sits between its own markers)."""
    ids = input_ids.reshape(-1)
    bounds = [int(v) for v in (cu_seqlens.tolist() if torch.is_tensor(cu_seqlens) else cu_seqlens)]
    dev = ids.device
    m = spatial_merge_size
    images = [] if image_grid_thw is None else [[int(v) for v in g] for g in image_grid_thw.tolist()]
    videos = []
    if video_grid_thw is not None:
        for t, h, w in video_grid_thw.tolist():
            videos += [[1, int(h), int(w)]] * int(t)
    images, videos = iter(images), iter(videos)
    out = torch.zeros(3, ids.numel(), dtype=torch.long, device=dev)
    deltas = []
    host = ids.tolist()
    for a, b in zip(bounds[:-1], bounds[1:]):
        nxt, i = 0, a  # next free position, cursor
        while i < b:
            tok = host[i]
            if tok == image_token_id or (video_token_id is not None and tok == video_token_id):
                try:
                    t, h, w = next(images if tok == image_token_id else videos)
                except StopIteration:
                    raise ValueError("more vision token runs than grids") from None
                gh, gw = h // m, w // m
                n = t * gh * gw
                if i + n > b or any(x != tok for x in host[i : i + n]):
                    raise ValueError(f"a vision run at token {i} is shorter than its grid ({t} x {gh} x {gw})")
                out[0, i : i + n] = torch.arange(t, device=dev).repeat_interleave(gh * gw) + nxt
                out[1, i : i + n] = torch.arange(gh, device=dev).repeat_interleave(gw).repeat(t) + nxt
                out[2, i : i + n] = torch.arange(gw, device=dev).repeat(gh * t) + nxt
                nxt += max(t, gh, gw) if t > 1 else max(gh, gw)
                i += n
            else:
                j = i
                while j < b and host[j] != image_token_id and host[j] != video_token_id:
                    j += 1
                out[:, i:j] = torch.arange(nxt, nxt + (j - i), device=dev)
                nxt += j - i
                i = j
        deltas.append(nxt - (b - a))
    if next(images, None) is not None or next(videos, None) is not None:
        raise ValueError("more grids than vision token runs")
    return out, deltas


def mrope_band_axes(section: list[int], half: int, interleaved: bool, device=None) -> torch.Tensor:
    """``[half]`` long: which position stream (0 temporal, 1 height, 2 width) drives each rotary frequency band.
    Consecutive layout: the first ``section[0]`` bands temporal, the next ``section[1]`` height, then width.
    Interleaved layout: bands 1, 4, 7, ... below ``3 * section[1]`` height, bands 2, 5, 8, ... below ``3 * section[2]``
    width, everything else temporal."""
    ax = torch.zeros(half, dtype=torch.long, device=device)
    if interleaved:
        ax[1 : 3 * section[1] : 3] = 1
        ax[2 : 3 * section[2] : 3] = 2
    else:
        ax[section[0] : section[0] + section[1]] = 1
        ax[section[0] + section[1] : section[0] + section[1] + section[2]] = 2
    return ax


def mrope_cos_sin(table: torch.Tensor, positions: torch.Tensor, axes: torch.Tensor):
    """``table`` [max_pos, rot] = [cos | sin], ``positions`` [3, T], ``axes`` [rot / 2] -> (cos, sin) [T, 1, rot / 2]: band f
    is looked up at the position of stream ``axes[f]``."""
    half = table.shape[-1] // 2
    cs = table[positions.long()]  # [3, T, rot]
    pick = axes[None, None, :].expand(1, cs.shape[1], half)
    cos = cs[..., :half].gather(0, pick)[0]
    sin = cs[..., half:].gather(0, pick)[0]
    return cos[:, None, :], sin[:, None, :]
