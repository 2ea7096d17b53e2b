"""Named host snapshots of a model's parameters (actor / ref / teacher / old_actor / rollout_actor).

One set of device parameters is re-pointed at different weight sets by copying from
pinned-host snapshots (parity: slime/utils/tensor_backper.py:12-104). When HBM allows, a
snapshot can stay on the device instead (``device_resident=True``): 180 GB per B200 makes
that the default for models up to a few billion parameters, removing the H2D copy per switch.
"""

from __future__ import annotations

from collections.abc import Callable, Iterable

import torch


class TensorBackuper:
    def __init__(self, source_getter: Callable[[], Iterable[tuple[str, torch.Tensor]]], device_resident: bool = False):
        self._source_getter = source_getter
        self._backups: dict[str, dict[str, torch.Tensor]] = {}
        self.device_resident = device_resident

    @property
    def backup_tags(self):
        return list(self._backups)

    def _alloc_like(self, t: torch.Tensor):
        if self.device_resident or not t.is_cuda:
            return torch.empty_like(t)
        return torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)

    @torch.no_grad()
    def backup(self, tag: str):
        store = self._backups.setdefault(tag, {})
        for name, t in self._source_getter():
            if name not in store:
                store[name] = self._alloc_like(t)
            store[name].copy_(t.detach(), non_blocking=True)
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()

    @torch.no_grad()
    def restore(self, tag: str):
        store = self._backups[tag]
        for name, t in self._source_getter():
            assert name in store, f"no backup of {name} under tag {tag}"
            t.copy_(store[name], non_blocking=True)
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()

    @torch.no_grad()
    def copy(self, src_tag: str, dst_tag: str):
        dst = self._backups.setdefault(dst_tag, {})
        for name, t in self._backups[src_tag].items():
            if name not in dst:
                dst[name] = torch.empty_like(t, pin_memory=t.is_pinned()) if not t.is_cuda else torch.empty_like(t)
            dst[name].copy_(t)

    def get(self, tag: str) -> dict[str, torch.Tensor]:
        return self._backups[tag]

    def drop(self, tag: str):
        self._backups.pop(tag, None)
