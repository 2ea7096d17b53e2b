"""Byte-level codec shared by the producer (trainer) and the consumer (engine host) of delta weight updates.

A tensor's delta is computed on its raw bytes against the previous version:
  ``xor``        new ^ old. Mostly zeros when few weights changed, so it compresses extremely well; applying it twice
                 undoes it (an involution), so a delta must be applied exactly once.
  ``overwrite``  little-endian u32 count, then that many u32 byte positions, then the new byte at each position.
                 Idempotent to apply; larger than xor when many bytes change.
The encoded bytes are then compressed (zstd when the ``zstandard`` package is present, zlib otherwise; the format name
is recorded next to the data) and the *new* bytes are checksummed (xxh3-128, blake3 or adler32) so the consumer can
prove that its patched tensor equals the trainer's. Parity: slime/utils/disk_delta.py:16-87.
"""

from __future__ import annotations

import os
import zlib

import numpy as np

NUM_WORKERS = min(32, os.cpu_count() or 8)

try:  # optional, faster and tighter than zlib
    import zstandard as _zstd
except ImportError:  # pragma: no cover - depends on the environment
    _zstd = None

DEFAULT_COMPRESSION = "zstd" if _zstd is not None else "zlib"


# ------------------------------------------------------------------------------ encode / apply
def xor_encode(new: np.ndarray, old: np.ndarray) -> tuple[np.ndarray, int]:
    diff = np.bitwise_xor(new, old)
    return diff, int(np.count_nonzero(diff))


def overwrite_encode(new: np.ndarray, changed_mask: np.ndarray) -> np.ndarray:
    pos = np.flatnonzero(changed_mask).astype("<u4")
    return np.concatenate([np.array([pos.size], "<u4").view(np.uint8), pos.view(np.uint8), new[changed_mask]])


def encode_delta(new: np.ndarray, old: np.ndarray, encoding: str) -> tuple[np.ndarray | None, int]:
    """(encoded bytes or None when nothing changed, number of changed bytes)."""
    if new.shape != old.shape:
        raise ValueError(f"tensor changed size: {old.shape} -> {new.shape}")
    if encoding == "xor":
        diff, changed = xor_encode(new, old)
        return (diff if changed else None), changed
    if encoding == "overwrite":
        mask = new != old
        changed = int(np.count_nonzero(mask))
        return (overwrite_encode(new, mask) if changed else None), changed
    raise ValueError(f"unknown delta encoding {encoding!r}")


def apply_delta(target: np.ndarray, diff: np.ndarray, encoding: str) -> None:
    """Patch ``target`` (uint8, writable, e.g. a memory map of the tensor inside a safetensors file) in place."""
    if encoding == "xor":
        if diff.size != target.size:
            raise ValueError(f"xor delta of {diff.size} bytes for a tensor of {target.size} bytes")
        np.bitwise_xor(target, diff, out=target)
    elif encoding == "overwrite":
        n = int(diff[:4].view("<u4")[0])
        pos = diff[4 : 4 + 4 * n].view("<u4")
        vals = diff[4 + 4 * n : 4 + 5 * n]
        if vals.size != n or (n and int(pos.max()) >= target.size):
            raise ValueError("malformed overwrite delta")
        target[pos] = vals
    else:
        raise ValueError(f"unknown delta encoding {encoding!r}")


# ---------------------------------------------------------------------------------- compression
def compress(buf: np.ndarray, fmt: str = DEFAULT_COMPRESSION) -> np.ndarray:
    raw = np.ascontiguousarray(buf).tobytes()
    if fmt == "zstd":
        if _zstd is None:
            raise RuntimeError("zstd compression requested but the zstandard package is not installed")
        out = _zstd.ZstdCompressor(level=1).compress(raw)
    elif fmt == "zlib":
        out = zlib.compress(raw, 1)
    elif fmt == "none":
        out = raw
    else:
        raise ValueError(f"unknown compression format {fmt!r}")
    return np.frombuffer(out, dtype=np.uint8)


def decompress(buf: np.ndarray, fmt: str) -> np.ndarray:
    raw = np.ascontiguousarray(buf).tobytes()
    if fmt == "zstd":
        if _zstd is None:
            raise RuntimeError("this delta is zstd-compressed but the zstandard package is not installed")
        out = _zstd.ZstdDecompressor().decompress(raw)
    elif fmt == "zlib":
        out = zlib.decompress(raw)
    elif fmt == "none":
        out = raw
    else:
        raise ValueError(f"unknown compression format {fmt!r}")
    return np.frombuffer(out, dtype=np.uint8)


# ------------------------------------------------------------------------------------ checksums
class _Adler32:
    def __init__(self):
        self.v = 1

    def update(self, data):
        self.v = zlib.adler32(data, self.v)

    def hexdigest(self) -> str:
        return f"{self.v:08x}"


def _hasher(algorithm: str):
    if algorithm == "xxh3-128":
        import xxhash

        return xxhash.xxh3_128()
    if algorithm == "blake3":
        import blake3

        return blake3.blake3()
    if algorithm == "adler32":
        return _Adler32()
    raise KeyError(f"unknown checksum algorithm {algorithm!r}")


def checksum(algorithm: str, buf) -> str:
    h = _hasher(algorithm)
    h.update(np.ascontiguousarray(buf))
    return h.hexdigest()


def atomic_write(path: str, data: bytes) -> None:
    """Write-then-rename so a reader never sees half a file (the directory is shared with other hosts)."""
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)
