"""Engine-host side of the disk transports: keep a local Hugging Face checkpoint directory at a requested version.

``pull_weights(local_dir, source_dir, target_version, base_dir)`` brings ``local_dir`` to ``target_version``:

* version 0 (or an empty ``local_dir``): copy the base checkpoint (``base_dir``, the engine's model path).
* a published *full* version (``source_dir/weight_vNNNNNN`` without delta metadata): copy it over as-is.
* published *deltas*: apply ``weight_v(cur+1) .. weight_v(target)`` in order. Each delta file holds, per changed tensor,
  a compressed byte diff (xor against the previous bytes, or an overwrite list); the tensor is patched in place inside
  the local safetensors file and the result is verified against the checksum the trainer recorded.

``local_dir/weight_version.txt`` records what the directory currently holds, so a restarted engine catches up from
wherever it was. Writes are in place (memory-mapped) because a checkpoint can be hundreds of GB; the version stamp is
written last and atomically. The trainer-side producer is ``slime_b200/weight_sync/disk_delta.py``.
Parity: the ``/pull_weights`` contract of slime/backends/sglang_utils/sglang_engine.py:344-356.
"""

from __future__ import annotations

import glob
import json
import logging
import os
import shutil
import struct

import numpy as np

from slime_b200.weight_sync import delta_codec

logger = logging.getLogger(__name__)
_STAMP = "weight_version.txt"


def version_dir(source_dir: str, version: int) -> str:
    return os.path.join(source_dir, f"weight_v{version:06d}")


def current_version(local_dir: str) -> int | None:
    try:
        with open(os.path.join(local_dir, _STAMP)) as f:
            return int(f.read().strip())
    except (OSError, ValueError):
        return None


def _stamp(local_dir: str, version: int) -> None:
    delta_codec.atomic_write(os.path.join(local_dir, _STAMP), str(version).encode())


def tensor_locations(ckpt_dir: str) -> dict[str, tuple[str, int, int]]:
    """name -> (file, absolute byte offset, nbytes), read from every safetensors header in ``ckpt_dir``."""
    out: dict[str, tuple[str, int, int]] = {}
    for path in sorted(glob.glob(os.path.join(ckpt_dir, "*.safetensors"))):
        with open(path, "rb") as f:
            (n,) = struct.unpack("<Q", f.read(8))
            header = json.loads(f.read(n))
        for name, info in header.items():
            if name != "__metadata__":
                lo, hi = info["data_offsets"]
                out[name] = (path, 8 + n + lo, hi - lo)
    return out


def _copy_checkpoint(src: str, dst: str) -> None:
    os.makedirs(dst, exist_ok=True)
    for name in os.listdir(dst):  # drop weights of an older layout, keep nothing stale
        if name.endswith(".safetensors") or name == "model.safetensors.index.json":
            os.unlink(os.path.join(dst, name))
    for name in os.listdir(src):
        p = os.path.join(src, name)
        if os.path.isfile(p) and not name.endswith(".tmp"):
            shutil.copyfile(p, os.path.join(dst, name))


def _read_index(vdir: str) -> dict:
    with open(os.path.join(vdir, "model.safetensors.index.json")) as f:
        return json.load(f)


def apply_delta_dir(local_dir: str, vdir: str) -> int:
    """Patch ``local_dir`` with the delta published in ``vdir``; returns the number of tensors changed."""
    from safetensors import safe_open

    index = _read_index(vdir)
    meta = index["metadata"]
    where = tensor_locations(local_dir)
    by_file: dict[str, list[str]] = {}
    for name, fname in index["weight_map"].items():
        by_file.setdefault(fname, []).append(name)
    n = 0
    for fname, names in by_file.items():
        with safe_open(os.path.join(vdir, fname), framework="np") as f:
            sums = f.metadata() or {}
            for name in names:
                if name not in where:
                    raise KeyError(f"delta {vdir} changes {name}, which the local checkpoint {local_dir} does not have")
                path, off, nbytes = where[name]
                diff = delta_codec.decompress(f.get_tensor(name), meta.get("compression_format", "zlib"))
                mm = np.memmap(path, dtype=np.uint8, mode="r+", offset=off, shape=(nbytes,))
                delta_codec.apply_delta(mm, diff, meta["delta_encoding"])
                got = delta_codec.checksum(meta["checksum_format"], mm)
                if name in sums and got != sums[name]:
                    raise ValueError(f"checksum mismatch after applying {vdir} to {name}: {got} != {sums[name]}")
                mm.flush()
                del mm
                n += 1
    return n


def pull_weights(local_dir: str, source_dir: str, target_version: int, base_dir: str | None = None) -> str:
    """Bring ``local_dir`` to ``target_version`` (see the module docstring). Returns ``local_dir``."""
    cur = current_version(local_dir)
    if cur is None or target_version == 0 or cur > target_version:
        if target_version == 0 or _is_delta(source_dir, target_version):
            if base_dir is None:
                raise ValueError("materialising the base checkpoint needs base_dir (the engine's model path)")
            logger.info("local checkpoint %s <- base %s", local_dir, base_dir)
            _copy_checkpoint(base_dir, local_dir)
            _stamp(local_dir, 0)
            cur = 0
    if target_version == 0:
        return local_dir
    vdir = version_dir(source_dir, target_version)
    if not _is_delta(source_dir, target_version):
        logger.info("local checkpoint %s <- full version %s", local_dir, vdir)
        _copy_checkpoint(vdir, local_dir)
        _stamp(local_dir, target_version)
        return local_dir
    for v in range(cur + 1, target_version + 1):
        step = version_dir(source_dir, v)
        meta = _read_index(step)["metadata"]
        if int(meta["base_version"]) != v - 1:
            raise ValueError(f"{step} is a delta against version {meta['base_version']}, local checkpoint is at {v - 1}")
        n = apply_delta_dir(local_dir, step)
        _stamp(local_dir, v)
        logger.info("local checkpoint %s: version %d applied (%d tensors changed)", local_dir, v, n)
    return local_dir


def _is_delta(source_dir: str, version: int) -> bool:
    try:
        return "delta_encoding" in _read_index(version_dir(source_dir, version)).get("metadata", {})
    except OSError:
        return False
