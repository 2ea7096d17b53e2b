"""Delta weight sync over a shared filesystem (``--update-weight-mode delta --update-weight-transport disk``).

Each sync publishes only what changed since the previous one:

    <update_weight_disk_dir>/weight_vNNNNNN/model-00000-of-0000K.safetensors   one uint8 blob per changed tensor
                                           /model.safetensors.index.json       metadata + weight_map

Metadata: ``version``, ``base_version``, ``delta_encoding`` (xor | overwrite), ``compression_format``,
``checksum_format``; per-file safetensors metadata maps tensor name -> checksum of the *new* bytes. Engines call
``/pull_weights`` (``slime_b200/weight_sync/local_checkpoint.py``) to patch their local checkpoint and then reload it
through the ordinary from-disk path, so multi-host engines and external engines need nothing else.

The producer keeps the previous bytes of every HF tensor (seeded from ``--hf-checkpoint``, which is what the engines
materialise as version 0, so the invariant "snapshot == engine base" holds). The diff runs where the weights are:
on the GPU (xor / compare and a changed-byte count), and only tensors that did change are copied to the host,
compressed by a thread pool, checksummed and written. The first ``update_weights`` call only captures the baseline.
Parity: slime/backends/megatron_utils/update_weight/update_weight_from_disk_delta.py:31-304.
"""

from __future__ import annotations

import json
import logging
import os
import shutil
import time
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import torch
import torch.distributed as dist

from slime_b200.parallel import state as mpu
from slime_b200.utils.misc import load_function
from slime_b200.weight_sync import delta_codec
from slime_b200.weight_sync.local_checkpoint import tensor_locations, version_dir
from slime_b200.weight_sync.updaters import WeightUpdaterBase, iter_hf_buckets

logger = logging.getLogger(__name__)


def _world():
    return (dist.get_rank(), dist.get_world_size()) if dist.is_available() and dist.is_initialized() else (0, 1)


def _barrier():
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def _gather_objects(obj):
    rank, world = _world()
    if world == 1:
        return [obj]
    out = [None] * world
    dist.all_gather_object(out, obj)
    return out


class UpdateWeightFromDiskDelta(WeightUpdaterBase):
    def __init__(self, args, model, weights_backuper=None):
        super().__init__(args, model, weights_backuper)
        self.delta_dir = args.update_weight_disk_dir
        os.makedirs(self.delta_dir, exist_ok=True)
        self.encoding = args.update_weight_delta_encoding
        self.checksum_algorithm = args.update_weight_delta_checksum
        self.compression = delta_codec.DEFAULT_COMPRESSION
        self._snapshot: dict[str, torch.Tensor] = {}  # hf name -> previous bytes (uint8, on snapshot_device)
        self._baseline_captured = False
        hook = getattr(args, "custom_update_weight_post_write_path", None)
        self._post_write_hook = load_function(hook) if hook else None
        self.is_src = False

    def connect_rollout_engines(self, engines, lock=None):
        super().connect_rollout_engines(engines, lock)
        # one writer per pipeline stage: the (dp=0, tp=0) rank owns the gathered tensors of its stage
        self.is_src = mpu.get_data_parallel_rank(with_context_parallel=True) == 0 and mpu.get_tensor_model_parallel_rank() == 0

    # ---------------------------------------------------------------------- public
    @torch.no_grad()
    def update_weights(self):
        t0 = time.time()
        if not self._baseline_captured:
            self._capture_baseline()
            self._baseline_captured = True
            return
        self.weight_version += 1
        delta, sums, changed, total = self._encode()
        wire = self._write(delta, sums)
        self._reload_engines()
        stats = torch.tensor([changed, total, wire], dtype=torch.float64)
        if dist.is_available() and dist.is_initialized():
            stats = stats.to(self.model.device)
            dist.all_reduce(stats)
        changed, total, wire = stats.tolist()
        self.metrics["perf/update_weights_density"] = changed / max(total, 1)
        self.metrics["perf/update_weights_wire_bytes"] = wire
        self.metrics["perf/update_weights_time"] = time.time() - t0
        if _world()[0] == 0:
            logger.info("[disk delta v%d] %.2f%% of bytes changed, %.3f GB on the wire", self.weight_version,
                        100.0 * changed / max(total, 1), wire / 1e9)  # fmt: skip

    # -------------------------------------------------------------------- internals
    def _iter_hf(self):
        for bucket in iter_hf_buckets(self.args, self.model, self.quantization_config):
            yield from bucket

    def _bytes_of(self, t: torch.Tensor) -> torch.Tensor:
        return t.detach().contiguous().view(-1).view(torch.uint8)

    def _capture_baseline(self):
        """Seed the snapshot and make every engine host materialise version 0, without publishing anything."""
        rank, _ = _world()
        pulls = []
        if rank == 0:
            shutil.rmtree(self.delta_dir, ignore_errors=True)  # a stale stream from an earlier run must not be replayed
            os.makedirs(self.delta_dir, exist_ok=True)
            if self._post_write_hook is not None:
                self._post_write_hook(self.args, self.delta_dir, list(self.engines))
            local = self.args.update_weight_local_checkpoint_dir
            pulls = [e.pull_weights(local, self.delta_dir, 0) for e in self.engines if local]
        _barrier()
        hf_dir = self.args.hf_checkpoint
        where = tensor_locations(hf_dir) if hf_dir and os.path.isdir(hf_dir) else {}
        dev = self.model.device
        seeded = 0
        for name, t in self._iter_hf():
            if not self.is_src:
                continue
            cur = self._bytes_of(t)
            if name in where and where[name][2] == cur.numel():
                path, off, n = where[name]
                base = torch.from_numpy(np.fromfile(path, dtype=np.uint8, count=n, offset=off))
                self._snapshot[name] = base.to(dev) if cur.is_cuda else base
                seeded += 1
            else:  # not in the base checkpoint (or a different size): the engines got it from the first full sync
                self._snapshot[name] = cur.clone()
        for p in pulls:
            if hasattr(p, "result"):
                p.result()
        if self.is_src:
            logger.info("[disk delta] baseline of %d tensors captured (%d seeded from %s)", len(self._snapshot), seeded, hf_dir)

    def _encode(self):
        """Diff every gathered HF tensor against the snapshot (on the device), compress the changed ones (host pool)."""
        delta: dict[str, np.ndarray] = {}
        sums: dict[str, str] = {}
        changed = total = 0
        pool = ThreadPoolExecutor(max_workers=delta_codec.NUM_WORKERS)
        jobs = []

        def finish(name, new_np, old_np):
            enc, _ = delta_codec.encode_delta(new_np, old_np, self.encoding)
            return name, delta_codec.compress(enc, self.compression), delta_codec.checksum(self.checksum_algorithm, new_np)

        try:
            for name, t in self._iter_hf():
                if not self.is_src:
                    continue
                new = self._bytes_of(t)
                total += new.numel()
                old = self._snapshot.get(name)
                if old is None or old.numel() != new.numel():
                    raise KeyError(f"{name} has no baseline of matching size; delta sync cannot add or resize tensors")
                n_changed = int(torch.count_nonzero(new != old))  # the only host sync per tensor
                if n_changed == 0:
                    continue
                changed += n_changed
                jobs.append(pool.submit(finish, name, new.cpu().numpy(), old.cpu().numpy()))
                self._snapshot[name] = new.clone()  # becomes the base of the next sync
            for j in jobs:
                name, blob, digest = j.result()
                delta[name], sums[name] = blob, digest
        finally:
            pool.shutdown()
        return delta, sums, changed, total

    def _write(self, delta: dict, sums: dict) -> int:
        """One canonical ``model-NNNNN-of-MMMMM.safetensors`` per writing rank plus the index on rank 0. File numbers
        and the weight map travel over the process group, not the filesystem, which may not show one host's writes
        to another before they are committed."""
        from safetensors.numpy import save as st_save

        rank, world = _world()
        vdir = version_dir(self.delta_dir, self.weight_version)
        if self.is_src:
            os.makedirs(vdir, exist_ok=True)
        counts = _gather_objects(int(bool(delta)))
        offset, n_files = sum(counts[:rank]), sum(counts)
        fname, wire = None, 0
        if delta:
            fname = f"model-{offset:05d}-of-{n_files:05d}.safetensors"
            blob = st_save(delta, metadata=sums)
            wire = len(blob)
            delta_codec.atomic_write(os.path.join(vdir, fname), blob)
        maps = _gather_objects({name: fname for name in delta})
        if rank == 0:
            os.makedirs(vdir, exist_ok=True)
            index = {"metadata": {"version": f"{self.weight_version:06d}", "base_version": f"{self.weight_version - 1:06d}",
                                  "delta_encoding": self.encoding, "compression_format": self.compression,
                                  "checksum_format": self.checksum_algorithm},
                     "weight_map": {n: f for m in maps for n, f in m.items()}}  # fmt: skip
            delta_codec.atomic_write(os.path.join(vdir, "model.safetensors.index.json"), json.dumps(index).encode())
        _barrier()
        return wire

    def _reload_engines(self):
        rank, _ = _world()
        vdir = version_dir(self.delta_dir, self.weight_version)
        if self._post_write_hook is not None and rank == 0:
            self._post_write_hook(self.args, vdir, list(self.engines))
        _barrier()
        if rank == 0 and self.engines:
            local = self.args.update_weight_local_checkpoint_dir
            assert local, "delta sync needs --update-weight-local-checkpoint-dir (where each engine host keeps its copy)"
            pulls = [e.pull_weights(local, self.delta_dir, self.weight_version) for e in self.engines]
            for p in pulls:
                if hasattr(p, "result"):
                    p.result()
            self._pause()
            for e in self.engines:
                e.update_weights_from_disk(local, weight_version=str(self.weight_version))
            self._resume()
            # published deltas stay on disk: an engine that restarts replays them from its base to catch up
        _barrier()
