"""Images -> the pixel rows a vision tower reads.

An image is resized so that both sides are multiples of ``patch_size * merge_size`` and its area lies within
``[min_pixels, max_pixels]`` (aspect ratio kept as far as rounding allows), normalised per channel, repeated
``temporal_patch_size`` times along time (a still image is one temporal patch), and cut into patches. Rows are ordered so
that the ``merge_size x merge_size`` patches that the tower later joins into one vector are consecutive, and each row is
the flattened ``[channel, time, patch row, patch column]`` block. Returns the rows and the ``(t, h, w)`` patch grid per
image: the ``pixel_values`` / ``image_grid_thw`` pair of Qwen2-VL style processors. The rollout engine uses this when
a request carries images and no processor directory is available; the count of placeholder tokens of an image is
``t * h * w / merge_size**2``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(height: int, width: int, factor: int, min_pixels: int, max_pixels: int) -> tuple[int, int]:
    if max(height, width) / min(height, width) > 200:
        raise ValueError(f"aspect ratio of a {height} x {width} image is beyond 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h, w = math.ceil(height * beta / factor) * factor, math.ceil(width * beta / factor) * factor
    return h, w


@dataclass
class ImageProcessor:
    patch_size: int = 16
    temporal_patch_size: int = 2
    merge_size: int = 2
    min_pixels: int = 56 * 56
    max_pixels: int = 28 * 28 * 1280
    mean: tuple = CLIP_MEAN
    std: tuple = CLIP_STD

    @classmethod
    def from_vision_config(cls, v: dict, **kw) -> "ImageProcessor":
        return cls(patch_size=v.get("patch_size", 16), temporal_patch_size=v.get("temporal_patch_size", 2),
                   merge_size=v.get("spatial_merge_size", 2), **kw)  # fmt: skip

    def tokens_for(self, grid) -> int:
        t, h, w = (int(x) for x in grid)
        return t * h * w // self.merge_size**2

    def one(self, image) -> tuple[torch.Tensor, list[int]]:
        from PIL import Image

        if not hasattr(image, "convert"):
            image = Image.fromarray(np.asarray(image))
        image = image.convert("RGB")
        p, m, tp = self.patch_size, self.merge_size, self.temporal_patch_size
        h, w = smart_resize(image.height, image.width, p * m, self.min_pixels, self.max_pixels)
        if (h, w) != (image.height, image.width):
            image = image.resize((w, h), resample=Image.BICUBIC)
        x = torch.from_numpy(np.asarray(image, dtype=np.float32) / 255.0).permute(2, 0, 1)  # [C, H, W]
        x = (x - torch.tensor(self.mean)[:, None, None]) / torch.tensor(self.std)[:, None, None]
        gh, gw = h // p, w // p
        x = x[None].expand(tp, -1, -1, -1)  # [tp, C, H, W]: a still image fills one temporal patch
        x = x.reshape(tp, 3, gh // m, m, p, gw // m, m, p)
        x = x.permute(2, 5, 3, 6, 1, 0, 4, 7)  # block row, block col, in-block row, in-block col, C, tp, p, p
        return x.reshape(gh * gw, 3 * tp * p * p).contiguous(), [1, gh, gw]

    def video(self, frames) -> tuple[torch.Tensor, list[int]]:
        """Frames of one clip -> rows of flattened patches, each spanning ``temporal_patch_size`` consecutive frames (the
        last frame repeats to fill the final group), and the grid [frame groups, patch rows, patch columns]. Every frame
        takes the size chosen for the first one."""
        from PIL import Image

        frames = [f if hasattr(f, "convert") else Image.fromarray(np.asarray(f)) for f in frames]
        if not frames:
            raise ValueError("a video needs at least one frame")
        p, m, tp = self.patch_size, self.merge_size, self.temporal_patch_size
        h, w = smart_resize(frames[0].height, frames[0].width, p * m, self.min_pixels, self.max_pixels)
        frames = frames + [frames[-1]] * (-len(frames) % tp)
        xs = []
        for f in frames:
            f = f.convert("RGB")
            if (h, w) != (f.height, f.width):
                f = f.resize((w, h), resample=Image.BICUBIC)
            xs.append(torch.from_numpy(np.asarray(f, dtype=np.float32) / 255.0).permute(2, 0, 1))
        x = (torch.stack(xs) - torch.tensor(self.mean)[:, None, None]) / torch.tensor(self.std)[:, None, None]  # [T, C, H, W]
        gt, gh, gw = len(frames) // tp, h // p, w // p
        x = x.reshape(gt, tp, 3, gh // m, m, p, gw // m, m, p)
        x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)  # group, block row, block col, in-block row, in-block col, C, tp, p, p
        return x.reshape(gt * gh * gw, 3 * tp * p * p).contiguous(), [gt, gh, gw]

    def __call__(self, images=None, videos=None) -> dict:
        out = {}
        if images:
            rows, grids = zip(*(self.one(im) for im in images))
            out.update(pixel_values=torch.cat(rows), image_grid_thw=torch.tensor(grids, dtype=torch.long))
        if videos:
            rows, grids = zip(*(self.video(v) for v in videos))
            out.update(pixel_values_videos=torch.cat(rows), video_grid_thw=torch.tensor(grids, dtype=torch.long))
        return out


def expand_image_placeholders(ids: list[int], token: int, counts: list[int]) -> list[int]:
    """Give the i-th run of ``token`` in ``ids`` the length ``counts[i]`` (a chat template writes one placeholder per image;
    a processor-expanded prompt already has the right lengths and passes through unchanged)."""
    out, i, k = [], 0, 0
    while i < len(ids):
        if ids[i] != token:
            out.append(ids[i])
            i += 1
            continue
        j = i
        while j < len(ids) and ids[j] == token:
            j += 1
        if k >= len(counts):
            raise ValueError(f"more image placeholder runs than images ({len(counts)})")
        if j - i not in (1, counts[k]):
            raise ValueError(f"image {k} needs {counts[k]} placeholder tokens, the prompt has a run of {j - i}")
        out += [token] * counts[k]
        i, k = j, k + 1
    if k != len(counts):
        raise ValueError(f"{len(counts)} images for {k} placeholder runs")
    return out
