"""Trainer -> rollout-engine weight synchronisation.

Transport selection (parity: slime/backends/megatron_utils/actor.py:152-183):
  update_weight_mode=delta           -> ``UpdateWeightFromDiskDelta``
  update_weight_transport=disk       -> ``UpdateWeightFromDisk``
  colocated                          -> ``UpdateWeightFromTensor``   (device-to-device, same GPUs)
  otherwise                          -> ``UpdateWeightFromDistributed`` (NCCL broadcast to engine GPUs)

All of them walk the trainer parameters in buckets of at most ``--update-weight-buffer-size``
bytes of *gathered* tensors: TP all-gather (fused qkv / GLU aware) -> Megatron->HF rename and split
-> optional 128x128 block-FP8 quantisation -> hand-off. Engines are paused and their prefix cache
flushed before the first bucket and resumed after the last; every sync bumps ``weight_version``.

When trainer and engine live in the same process and shard identically (the colocated fast path of
``slime_b200.api``), tensors are copied device-to-device into the engine's fused buffers with no
rename/split at all.
"""

from __future__ import annotations

import logging
import os
import time

import torch
import torch.distributed as dist

from slime_b200.parallel import state as mpu
from slime_b200.utils.misc import load_function
from slime_b200.weight_sync import convert
from slime_b200.weight_sync.quantizer import quantize_params

logger = logging.getLogger(__name__)


def named_params_and_buffers(model):
    """(global_name, tensor) for parameters and the buffers that must reach the engine (expert_bias)."""
    from slime_b200.backends.train.checkpoint import global_param_name

    for name, p in model.named_parameters():
        yield global_param_name(name, p), p
    for name, b in model.named_buffers():
        if name.endswith("expert_bias"):
            yield name, b


def all_gather_param(cfg, name: str, p: torch.Tensor) -> torch.Tensor:
    """Full tensor of a TP-sharded parameter on every rank of its TP group."""
    if not getattr(p, "tensor_model_parallel", False):
        return p.data
    is_exp = getattr(p, "is_expert", False)
    tp = mpu.get_expert_tensor_parallel_world_size() if is_exp else mpu.get_tensor_model_parallel_world_size()
    if tp == 1:
        return p.data
    group = mpu.get_expert_tensor_parallel_group() if is_exp else mpu.get_tensor_model_parallel_group()
    shards = [torch.empty_like(p.data) for _ in range(tp)]
    dist.all_gather(shards, p.data.contiguous(), group=group)
    return convert.merge_tp_shards(cfg, name, shards, p.partition_dim, getattr(p, "partition_stride", 1))


def iter_hf_buckets(args, model, quantization_config=None):
    """Yield lists of (hf_name, tensor) bounded by the buffer size (counting gathered bytes)."""
    limit = args.update_weight_buffer_size
    bucket, used = [], 0
    cfg = model.cfg
    for name, p in named_params_and_buffers(model):
        if name == "output_layer.weight" and cfg.tie_word_embeddings:
            continue
        full = all_gather_param(cfg, name, p)
        pairs = convert.convert_to_hf(cfg, name, full)
        pairs = quantize_params(args, name, pairs, quantization_config)
        nbytes = sum(t.numel() * t.element_size() for _n, t in pairs)
        if bucket and used + nbytes > limit:
            yield bucket
            bucket, used = [], 0
        bucket += pairs
        used += nbytes
    if bucket:
        yield bucket


class WeightUpdaterBase:
    def __init__(self, args, model, weights_backuper=None):
        self.args, self.model, self.backuper = args, model, weights_backuper
        self.engines, self.lock = [], None
        self.weight_version = 0
        self.metrics: dict = {}
        self.quantization_config = _load_quant_config(args)

    def connect_rollout_engines(self, engines, lock=None):
        self.engines, self.lock = list(engines), lock

    def pop_metrics(self) -> dict:
        m, self.metrics = self.metrics, {}
        return m

    def _pause(self):
        for e in self.engines:
            e.pause_generation()
            e.flush_cache()

    def _resume(self):
        for e in self.engines:
            e.continue_generation()

    def update_weights(self):
        raise NotImplementedError


def _load_quant_config(args):
    path = getattr(args, "hf_checkpoint", None)
    if getattr(args, "sglang_quantization", None) == "fp8":
        return {"quant_method": "fp8", "weight_block_size": [128, 128]}
    if path and os.path.exists(os.path.join(path, "config.json")):
        import json

        return json.load(open(os.path.join(path, "config.json"))).get("quantization_config")
    return None


class UpdateWeightFromTensor(WeightUpdaterBase):
    """Colocated sync. Engines are in-process objects (or proxies with the same methods)."""

    def update_weights(self):
        t0 = time.time()
        self.weight_version += 1
        is_src = mpu.get_data_parallel_rank(with_context_parallel=True) == 0 or len(self.engines) > 0
        self._pause()
        if self._can_copy_fused():
            self._copy_fused()
        else:
            for bucket in iter_hf_buckets(self.args, self.model, self.quantization_config):
                if is_src:
                    for e in self.engines:
                        e.update_weights(bucket, version=str(self.weight_version), flush_cache=False)
        for e in self.engines:
            if getattr(e, "weights", None) is not None:  # in-process engine object; remote ones get the version per bucket
                e.weights.version = str(self.weight_version)
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()  # consumers' copies retired before generation resumes
        self._resume()
        self.metrics["perf/update_weights_time"] = time.time() - t0

    def _can_copy_fused(self) -> bool:
        if self.quantization_config or not self.engines:
            return False
        e = self.engines[0]
        return (
            getattr(e, "weights", None) is not None and e.weights.tp == mpu.get_tensor_model_parallel_world_size()
            and e.weights.rank == mpu.get_tensor_model_parallel_rank()
            and mpu.get_pipeline_model_parallel_world_size() == 1 and self.model.cfg.num_experts is None
            and self._fused_pairs(e) is not None
        )  # fmt: skip

    # trainer parameter (name inside a layer) -> engine buffer of the same shard shape
    _LAYER_MAP = {
        "self_attention.linear_qkv.weight": "qkv", "self_attention.linear_qkv.bias": "qkv_bias",
        "self_attention.linear_qkv.layer_norm_weight": "ln1", "self_attention.q_layernorm.weight": "q_norm",
        "self_attention.k_layernorm.weight": "k_norm", "self_attention.linear_proj.weight": "o",
        "mlp.linear_fc1.weight": "gate_up", "mlp.linear_fc1.layer_norm_weight": "ln2", "mlp.linear_fc2.weight": "down",
    }  # fmt: skip

    def _fused_pairs(self, e):
        """(trainer shard, engine buffer) for every parameter, or None when a name has no same-shape counterpart."""
        w, pairs = e.weights, []
        for name, p in self.model.named_parameters():
            if name == "embedding.word_embeddings.weight":
                dst = w.embed
            elif name == "output_layer.weight":
                if self.model.cfg.tie_word_embeddings:
                    continue
                dst = w.lm_head
            elif name == "decoder.final_layernorm.weight":
                dst = w.final_norm
            else:
                _, _, i, sub = name.split(".", 3)
                key = self._LAYER_MAP.get(sub)
                dst = w.layers[int(i)].get(key) if key else None
            if dst is None or dst.shape != p.shape:
                return None
            pairs.append((p.data, dst))
        return pairs

    @torch.no_grad()
    def _copy_fused(self):
        """Same sharding on both sides (rank r of the tensor-parallel group holds shard r of the trainer's and of the
        engine's weights, in the same fused layouts): the sync is a device-local copy of every shard, with no gather,
        split or rename. On CUDA all tensors go in one launch of the multi-tensor copy kernel."""
        from slime_b200.weight_sync import device_sync

        for e in self.engines:
            pairs = self._fused_pairs(e)
            assert pairs is not None, "engine and trainer shards differ in shape"
            device_sync.copy_tensors([(s, d) for s, d in pairs if isinstance(d, torch.Tensor)])
            for s, d in pairs:  # block-fp8 engine buffers: quantised on the device straight into the resident bytes and scales
                if not isinstance(d, torch.Tensor):
                    d.load_rows(0, s)


class UpdateWeightFromDistributed(WeightUpdaterBase):
    """Disaggregated sync: the (dp=0, tp=0) rank of every pipeline stage broadcasts each HF tensor to
    all engine GPUs over a dedicated NCCL group ``slime-pp_{pp_rank}``; engines are told names /
    dtypes / shapes through their control API and post the matching receives."""

    def connect_rollout_engines(self, engines, lock=None):
        super().connect_rollout_engines(engines, lock)
        self.is_src = (
            mpu.get_data_parallel_rank(with_context_parallel=True) == 0 and mpu.get_tensor_model_parallel_rank() == 0
        )
        self.group = None
        if self.is_src and engines:
            self.group_name = f"slime-pp_{mpu.get_pipeline_model_parallel_rank()}"
            self.group = connect_rollout_engines_from_distributed(self.args, self.group_name, engines)

    def update_weights(self):
        t0 = time.time()
        self.weight_version += 1
        if self.is_src:
            self._pause()
        for bucket in iter_hf_buckets(self.args, self.model, self.quantization_config):
            if not self.is_src:
                continue
            if self.lock is not None:
                self.lock.acquire()
            try:
                update_weights_from_distributed(self.group_name, self.group, self.weight_version, self.engines, bucket)
            finally:
                if self.lock is not None:
                    self.lock.release()
        if self.is_src:
            self._resume()
        self.metrics["perf/update_weights_time"] = time.time() - t0


def connect_rollout_engines_from_distributed(args, group_name, engines):
    """Create the trainer+engines NCCL world: rank 0 = this trainer rank, then every engine GPU."""
    from slime_b200.utils.distributed_utils import init_extra_process_group
    from slime_b200.utils.misc import get_current_node_ip, get_free_port

    addr, port = get_current_node_ip(), get_free_port(start_port=20000)
    gpus = [getattr(e, "num_gpus", 1) for e in engines]
    world = 1 + sum(gpus)
    off, handles = 1, []
    for e, n in zip(engines, gpus):
        handles.append(e.init_weights_update_group(addr, port, off, world, group_name, backend="nccl"))
        off += n
    group = init_extra_process_group(backend="nccl", init_method=f"tcp://{addr}:{port}", world_size=world, rank=0,
                                     group_name=group_name)  # fmt: skip
    for h in handles:
        if hasattr(h, "result"):
            h.result()
    return group


def update_weights_from_distributed(group_name, group, version, engines, named):
    handles = [
        e.update_weights_from_distributed(
            names=[n for n, _ in named], dtypes=[str(t.dtype).replace("torch.", "") for _, t in named],
            shapes=[list(t.shape) for _, t in named], group_name=group_name, weight_version=str(version),
        )
        for e in engines
    ]  # fmt: skip
    works = [dist.broadcast(t.contiguous(), 0, group=group, async_op=True) for _n, t in named]
    for w in works:
        w.wait()
    for h in handles:
        if hasattr(h, "result"):
            h.result()


class UpdateWeightFromDisk(WeightUpdaterBase):
    """Full checkpoint per version (``weight_v{N:06d}``) on a filesystem both sides can read."""

    def update_weights(self):
        from slime_b200.checkpoint.hf_saver import save_hf_model_to_path

        t0 = time.time()
        self.weight_version += 1
        vdir = os.path.join(self.args.update_weight_disk_dir, f"weight_v{self.weight_version:06d}")
        save_hf_model_to_path(self.args, self.model, vdir)
        hook = getattr(self.args, "custom_update_weight_post_write_path", None)
        rank0 = not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0
        if rank0:
            if hook:
                load_function(hook)(self.args, vdir, self.engines)
            self._pause()
            for e in self.engines:
                if getattr(self.args, "update_weight_local_checkpoint_dir", None) and hasattr(e, "pull_weights"):
                    e.pull_weights(self.args.update_weight_local_checkpoint_dir, self.args.update_weight_disk_dir, self.weight_version)
                e.update_weights_from_disk(vdir, weight_version=str(self.weight_version))
            self._resume()
            if not self.args.update_weight_disk_keep_files and self.weight_version > 1:
                import shutil

                old = os.path.join(self.args.update_weight_disk_dir, f"weight_v{self.weight_version - 1:06d}")
                shutil.rmtree(old, ignore_errors=True)
        self.metrics["perf/update_weights_time"] = time.time() - t0


def make_weight_updater(args, model, weights_backuper=None):
    if args.update_weight_mode == "delta":
        from slime_b200.weight_sync.disk_delta import UpdateWeightFromDiskDelta

        return UpdateWeightFromDiskDelta(args, model, weights_backuper)
    if args.update_weight_transport == "disk":
        return UpdateWeightFromDisk(args, model, weights_backuper)
    if args.colocate:
        return UpdateWeightFromTensor(args, model, weights_backuper)
    return UpdateWeightFromDistributed(args, model, weights_backuper)
