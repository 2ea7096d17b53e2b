"""Write a Hugging Face safetensors checkpoint from the live trainer model.

Every rank converts the tensors it is responsible for (TP-gathered, HF names), shards are
assigned to writer ranks, and rank 0 writes ``model.safetensors.index.json`` + ``config.json``.
Parity: slime/backends/megatron_utils/hf_checkpoint_saver.py:44-311.
"""

from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

from slime_b200.weight_sync import convert

MAX_SHARD_BYTES = 5 * 2**30


def iter_hf_tensors(model):
    """(hf_name, tensor) for every parameter this rank is the designated writer of."""
    from slime_b200.backends.train.checkpoint import _gather_tp, global_param_name
    from slime_b200.parallel import state as mpu

    for name, p in model.named_parameters():
        full = _gather_tp(model, name, p)
        owner = (mpu.get_expert_data_parallel_rank() if getattr(p, "is_expert", False)
                 else mpu.get_data_parallel_rank(with_context_parallel=True)) == 0  # fmt: skip
        if full is None or not owner:
            continue
        if name == "output_layer.weight" and model.cfg.tie_word_embeddings:
            continue
        yield from convert.convert_to_hf(model.cfg, global_param_name(name, p), full)


def save_hf_model_to_path(args, model, path: str, quantizer=None) -> str:
    from safetensors.torch import save_file

    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    os.makedirs(path, exist_ok=True)
    shard, shard_bytes, files, weight_map = {}, 0, [], {}

    def flush():
        nonlocal shard, shard_bytes
        if not shard:
            return
        fn = f"model-rank{rank:03d}-{len(files):05d}.safetensors"
        save_file({k: v.contiguous().cpu() for k, v in shard.items()}, os.path.join(path, fn), metadata={"format": "pt"})
        for k in shard:
            weight_map[k] = fn
        files.append(fn)
        shard, shard_bytes = {}, 0

    for name, t in iter_hf_tensors(model):
        items = quantizer(name, t) if quantizer is not None else [(name, t)]
        for n, x in items:
            shard[n] = x.detach()
            shard_bytes += x.numel() * x.element_size()
            if shard_bytes >= MAX_SHARD_BYTES:
                flush()
    flush()
    maps = [weight_map]
    if world > 1:
        maps = [None] * world
        dist.all_gather_object(maps, weight_map)
    if rank == 0:
        merged = {}
        for m in maps:
            merged.update(m)
        total = sum(os.path.getsize(os.path.join(path, f)) for f in set(merged.values()))
        with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": dict(sorted(merged.items()))}, f, indent=1)
        src_cfg = os.path.join(getattr(args, "hf_checkpoint", None) or "", "config.json")
        if os.path.exists(src_cfg):
            cfg = json.load(open(src_cfg))
        else:
            cfg = model.cfg.to_hf_dict()
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(cfg, f, indent=1)
    if world > 1:
        dist.barrier()
    return path
