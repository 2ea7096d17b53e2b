"""Node-local object store: rollout -> trainer payloads travel as references to files in shared memory.

``put(obj)`` pickles (torch tensors through ``torch.save``) into ``/dev/shm`` and returns a small
``StoreRef``; ``get(ref)`` loads it in whichever process asks. This is the stand-in for the Ray object
store the reference uses for per-DP-rank rollout data (slime/ray/rollout.py:817-823).
"""

from __future__ import annotations

import os
import uuid
from dataclasses import dataclass

import torch

_DIR = os.environ.get("SLIME_B200_STORE_DIR") or ("/dev/shm" if os.path.isdir("/dev/shm") else "/tmp")


@dataclass(frozen=True)
class StoreRef:
    path: str
    nbytes: int

    def __repr__(self):
        return f"StoreRef({os.path.basename(self.path)}, {self.nbytes} B)"


def put(obj) -> StoreRef:
    path = os.path.join(_DIR, f"slb200-obj-{uuid.uuid4().hex}.pt")
    torch.save(obj, path)
    return StoreRef(path, os.path.getsize(path))


def get(ref):
    if isinstance(ref, StoreRef):
        return torch.load(ref.path, weights_only=False, mmap=False)
    if hasattr(ref, "result"):
        return ref.result()
    return ref


def free(ref) -> None:
    if isinstance(ref, StoreRef):
        try:
            os.unlink(ref.path)
        except OSError:
            pass
