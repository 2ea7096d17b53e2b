"""Small host-side helpers shared by every layer.

Parity: slime/utils/misc.py (load_function :39, Box :131,
should_run_periodic_action :107, decode_int32_meta_array :13).
"""

from __future__ import annotations

import base64
import importlib
import socket
import subprocess
import threading
from collections.abc import Callable, Iterable
from typing import Any

import numpy as np
import torch

_FN_CACHE: dict[str, Any] = {}
_FN_LOCK = threading.Lock()


def load_function(path: str):
    """Resolve ``"pkg.mod.attr"`` (or ``"pkg.mod:attr"``) to the object it names.

    Results are memoised so a hook resolved on every sample costs one dict hit.
    """
    with _FN_LOCK:
        hit = _FN_CACHE.get(path)
    if hit is not None:
        return hit
    if ":" in path:
        mod_name, attr = path.split(":", 1)
    else:
        mod_name, _, attr = path.rpartition(".")
    if not mod_name:
        raise ValueError(f"'{path}' is not a dotted path to a module attribute")
    obj = importlib.import_module(mod_name)
    for part in attr.split("."):
        obj = getattr(obj, part)
    with _FN_LOCK:
        _FN_CACHE[path] = obj
    return obj


def decode_int32_meta_array(meta_info: dict[str, Any], keys: str | Iterable[str]) -> torch.Tensor | None:
    """Fetch an int32 array from engine ``meta_info``.

    The wire form is base64 of little-endian int32; lists, numpy arrays, bytes
    and tensors are accepted too. Returns a flat CPU int32 tensor or ``None``
    when no key is present.
    """
    names = (keys,) if isinstance(keys, str) else tuple(keys)
    raw = None
    for name in names:
        if name in meta_info:
            raw = meta_info[name]
            break
    if raw is None:
        return None
    if isinstance(raw, str):
        raw = base64.b64decode(raw.encode("ascii"))
    if isinstance(raw, (bytes, bytearray, memoryview)):
        arr = np.frombuffer(bytes(raw), dtype="<i4").copy()
        return torch.from_numpy(arr)
    if torch.is_tensor(raw):
        return raw.detach().to("cpu", torch.int32).reshape(-1)
    return torch.as_tensor(np.array(raw, dtype=np.int32, copy=True)).reshape(-1)


def encode_int32_meta_array(values) -> str:
    """Inverse of :func:`decode_int32_meta_array` (base64 little-endian int32)."""
    arr = np.asarray(torch.as_tensor(values).cpu().numpy() if torch.is_tensor(values) else values, dtype="<i4")
    return base64.b64encode(arr.tobytes()).decode("ascii")


class SingletonMeta(type):
    """Metaclass giving each class exactly one instance (``clear_instances`` resets)."""

    _instances: dict[type, Any] = {}

    def __call__(cls, *args, **kwargs):
        inst = SingletonMeta._instances.get(cls)
        if inst is None:
            inst = super().__call__(*args, **kwargs)
            SingletonMeta._instances[cls] = inst
        return inst

    def clear_instances(cls):
        SingletonMeta._instances.pop(cls, None)


class Box:
    """Opaque wrapper so an object-store reference travels through RPC by reference."""

    __slots__ = ("_inner",)

    def __init__(self, inner):
        self._inner = inner

    @property
    def inner(self):
        return self._inner


def should_run_periodic_action(rollout_id, interval, num_rollout_per_epoch=None, num_rollout=None) -> bool:
    """True when a save/eval cadence fires at ``rollout_id`` (0-based).

    Fires every ``interval`` rollouts, at epoch boundaries and on the final rollout.
    """
    if interval is None:
        return False
    if num_rollout is not None and rollout_id == num_rollout - 1:
        return True
    n = rollout_id + 1
    if n % interval == 0:
        return True
    return num_rollout_per_epoch is not None and n % num_rollout_per_epoch == 0


def exec_command(cmd: str, capture_output: bool = False) -> str | None:
    print(f"EXEC: {cmd}", flush=True)
    res = subprocess.run(["bash", "-c", cmd], check=True, capture_output=capture_output, text=capture_output)
    return res.stdout if capture_output else None


def is_port_available(port: int, host: str = "127.0.0.1") -> bool:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            s.bind((host, port))
            return True
        except OSError:
            return False


def get_free_port(start_port: int = 10000, consecutive: int = 1) -> int:
    port = start_port
    while not all(is_port_available(port + i) for i in range(consecutive)):
        port += 1
    return port


def get_current_node_ip() -> str:
    import os

    if os.environ.get("SLIME_HOST_IP"):
        return os.environ["SLIME_HOST_IP"]
    try:
        with socket.socket(socket.AF_INET, socket.SOCK_DGRAM) as s:
            s.connect(("10.255.255.255", 1))
            return s.getsockname()[0]
    except OSError:
        return "127.0.0.1"


def group_by(items: Iterable, key: Callable) -> dict:
    out: dict = {}
    for it in items:
        out.setdefault(key(it), []).append(it)
    return out


def chunk_named_params_by_size(named: Iterable[tuple[str, torch.Tensor]], limit_bytes: int):
    """Greedy contiguous bucketing of ``(name, tensor)`` pairs under a byte cap."""
    bucket, used = [], 0
    for name, t in named:
        nbytes = t.numel() * t.element_size()
        if bucket and used + nbytes > limit_bytes:
            yield bucket
            bucket, used = [], 0
        bucket.append((name, t))
        used += nbytes
    if bucket:
        yield bucket
