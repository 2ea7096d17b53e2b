"""Checkpoint save / load in the Megatron ``torch_dist`` directory layout, plus HF loading.

Layout (parity: docs/en/get_started/usage.md:112-127, tools/convert_torch_dist_to_hf.py:222-228
of the reference): ``{save}/latest_checkpointed_iteration.txt`` holding the iteration (or
``release``), ``{save}/iter_{:07d}/`` (or ``release/``) with PyTorch-DCP shards
(``.metadata`` + ``__{rank}_{k}.distcp``) and ``common.pt`` carrying ``args``.
Model keys are the Megatron module paths with *global* layer and expert indices; fused qkv is
written in the Megatron per-KV-group interleave. Every tensor is written once, TP-gathered, by the
tp-rank-0 of each pipeline stage / expert group, so a checkpoint can be reloaded under any
(tp, pp, ep, dp) factorisation. Optimizer shards are written per data-parallel rank under
``optimizer.*`` keys with the step at top level (placement independent: GPU or CPU-offloaded Adam).

``load_checkpoint`` dispatches: torch_dist if the tracker file / ``iter_*`` dir exists, else a
Hugging Face directory (safetensors) loaded straight into the local shards
(slime/backends/megatron_utils/checkpoint.py:95-142). Missing keys are tolerated (partial load:
new critic heads, MTP layers).
"""

from __future__ import annotations

import logging
import os
import threading

import torch
import torch.distributed as dist

from slime_b200.parallel import state as mpu
from slime_b200.weight_sync import convert

logger = logging.getLogger(__name__)
TRACKER = "latest_checkpointed_iteration.txt"
_async_threads: list[threading.Thread] = []


def checkpoint_dir(base: str, iteration: int | str) -> str:
    return os.path.join(base, "release" if iteration == "release" else f"iter_{int(iteration):07d}")


def read_tracker(base: str):
    path = os.path.join(base, TRACKER)
    if not os.path.exists(path):
        return None
    txt = open(path).read().strip()
    return "release" if txt == "release" else int(txt)


def is_native_checkpoint(path: str | None) -> bool:
    if not path or not os.path.isdir(path):
        return False
    if os.path.exists(os.path.join(path, TRACKER)):
        return True
    return any(n.startswith("iter_") or n == "release" for n in os.listdir(path))


def _world():
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def _gather_tp(model, name, p):
    """Full tensor of a (possibly TP-sharded) parameter on tp-rank 0; None elsewhere."""
    tp = mpu.get_expert_tensor_parallel_world_size() if getattr(p, "is_expert", False) else mpu.get_tensor_model_parallel_world_size()
    if tp == 1 or not getattr(p, "tensor_model_parallel", False):
        return p.detach() if mpu.get_tensor_model_parallel_rank() == 0 or tp == 1 else None
    group = mpu.get_expert_tensor_parallel_group() if getattr(p, "is_expert", False) else mpu.get_tensor_model_parallel_group()
    shards = [torch.empty_like(p) for _ in range(tp)]
    dist.all_gather(shards, p.detach().contiguous(), group=group)
    if dist.get_rank(group) != 0:
        return None
    return convert.merge_tp_shards(model.cfg, name, shards, p.partition_dim, getattr(p, "partition_stride", 1))


def global_param_name(name: str, p) -> str:
    """Apply the expert-parallel index offset so ``weight{e}`` carries the global expert id."""
    if getattr(p, "is_expert", False) and mpu.get_expert_model_parallel_world_size() > 1:
        import re

        m = re.match(r"^(.*\.weight)(\d+)$", name)
        if m:
            per = None
            # local experts per rank = count of weightN siblings; derive from the id space lazily
            per = getattr(p, "num_local_experts", None)
            if per is None:
                return name
            return f"{m.group(1)}{int(m.group(2)) + mpu.get_expert_model_parallel_rank() * per}"
    return name


def model_state_for_save(model) -> dict[str, torch.Tensor]:
    """Tensors this rank is responsible for writing (global names, Megatron layouts)."""
    out = {}
    dp_rank = mpu.get_data_parallel_rank(with_context_parallel=True)
    for name, p in model.named_parameters():
        owner_dp = mpu.get_expert_data_parallel_rank() == 0 if getattr(p, "is_expert", False) else dp_rank == 0
        full = _gather_tp(model, name, p)
        if full is None or not owner_dp:
            continue
        if name.endswith("linear_qkv.weight") or name.endswith("linear_qkv.bias"):
            full = convert.qkv_to_megatron_layout(model.cfg, full)
        out[global_param_name(name, p)] = full.cpu() if not full.is_cuda else full
    for name, b in model.named_buffers():
        if dp_rank == 0 and mpu.get_tensor_model_parallel_rank() == 0:
            out[name] = b.detach()
    return out


def save_checkpoint(args, iteration: int | str, model, save_optimizer: bool = True, async_save: bool = False, base=None):
    import torch.distributed.checkpoint as dcp

    finalize_async_saves()
    base = base or args.save
    path = checkpoint_dir(base, iteration)
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    if rank == 0:
        os.makedirs(path, exist_ok=True)
    if _world():
        dist.barrier()
    state = dict(model_state_for_save(model))
    if save_optimizer and model.optimizer is not None:
        osd = model.optimizer.state_dict()
        for bi, shard in enumerate(osd["shards"]):
            for k, v in shard.items():
                state[f"optimizer.state.buf{bi}.rank{model.buffers[bi].group_rank}.{k}"] = v
    state = {k: (v.detach().cpu() if async_save else v) for k, v in state.items()}
    common = None
    if rank == 0:
        common = {
            "args": args,
            "iteration": iteration,
            "checkpoint_version": 3.0,
            "optimizer_step": model.optimizer.step_count if model.optimizer is not None else 0,
            "opt_param_scheduler": model.scheduler.state_dict() if model.scheduler is not None else None,
            "rng_state": {"torch": torch.get_rng_state()} if not getattr(args, "no_save_rng", False) else None,
            "format": "torch_dist",
        }

    rng = None if getattr(args, "no_save_rng", False) else collect_rng_state()

    def _write():
        writer = dcp.FileSystemWriter(path, single_file_per_rank=True, thread_count=2)
        dcp.save(state, storage_writer=writer, no_dist=not _world())
        if rng is not None:  # every rank keeps its own streams (host, device, model-parallel generators)
            torch.save(rng, os.path.join(path, f"rng_rank{rank:05d}.pt"))
        if rank == 0:
            torch.save(common, os.path.join(path, "common.pt"))
            tmp = os.path.join(base, TRACKER + ".tmp")
            with open(tmp, "w") as f:
                f.write(str(iteration))
            os.replace(tmp, os.path.join(base, TRACKER))

    if async_save and _world():
        logger.warning("async_save: a multi-rank save is collective and runs synchronously")
    if async_save and not _world():
        t = threading.Thread(target=_write, daemon=True)
        t.start()
        _async_threads.append(t)
    else:
        _write()
        if _world():
            dist.barrier()
    return path


def finalize_async_saves():
    while _async_threads:
        _async_threads.pop().join()


# --------------------------------------------------------------------------------- load
def _read_dcp_keys(path: str) -> dict:
    import torch.distributed.checkpoint as dcp

    reader = dcp.FileSystemReader(path)
    return reader.read_metadata().state_dict_metadata


def _dcp_load(path: str, wanted: dict[str, torch.Tensor]):
    import torch.distributed.checkpoint as dcp

    if wanted:
        dcp.load(wanted, storage_reader=dcp.FileSystemReader(path), no_dist=True)
    return wanted


def load_checkpoint(args, model, load_optimizer: bool = True):
    """Returns the loaded iteration (int), ``None`` for HF / fresh init."""
    path = args.load
    if path is None:
        return None
    if is_native_checkpoint(path):
        return _load_native(args, model, path, load_optimizer)
    if os.path.isdir(path) and os.path.exists(os.path.join(path, "config.json")):
        from slime_b200.checkpoint.hf_loader import load_hf_weights

        load_hf_weights(path, model)
        if model.optimizer is not None:
            model.optimizer.reload_model_params()
        return None
    raise FileNotFoundError(f"--load {path} is neither a torch_dist checkpoint nor a Hugging Face directory")


def _load_native(args, model, base, load_optimizer):
    step = getattr(args, "ckpt_step", None)
    iteration = step if step is not None else read_tracker(base)
    if iteration is None:
        its = sorted(int(n[5:]) for n in os.listdir(base) if n.startswith("iter_"))
        iteration = its[-1] if its else "release"
    path = checkpoint_dir(base, iteration)
    meta = _read_dcp_keys(path)
    cfg = model.cfg
    tp, tpr = mpu.get_tensor_model_parallel_world_size(), mpu.get_tensor_model_parallel_rank()
    wanted, plan = {}, []
    for name, p in model.named_parameters():
        key = global_param_name(name, p)
        if key not in meta:
            logger.warning("checkpoint %s has no key %s: keeping the initialised value (partial load)", path, key)
            continue
        full_shape = tuple(meta[key].size)
        wanted[key] = torch.empty(full_shape, dtype=p.dtype)
        plan.append((name, key, p))
    _dcp_load(path, wanted)
    with torch.no_grad():
        for name, key, p in plan:
            full = wanted[key]
            if name.endswith("linear_qkv.weight") or name.endswith("linear_qkv.bias"):
                full = convert.qkv_from_megatron_layout(cfg, full)
            is_exp = getattr(p, "is_expert", False)
            ptp = mpu.get_expert_tensor_parallel_world_size() if is_exp else tp
            prk = mpu.get_expert_tensor_parallel_rank() if is_exp else tpr
            if getattr(p, "tensor_model_parallel", False) and ptp > 1:
                full = convert.shard_for_tp(cfg, name, full, p.partition_dim, getattr(p, "partition_stride", 1), ptp, prk)
            if full.shape != p.shape:
                if "output_layer" in name and getattr(model, "role", "") == "critic":
                    logger.warning("re-initialising critic head %s (checkpoint shape %s)", name, tuple(full.shape))
                    continue
                raise ValueError(f"shape mismatch for {name}: checkpoint {tuple(full.shape)} vs model {tuple(p.shape)}")
            p.copy_(full.to(p.device))
    common_path = os.path.join(path, "common.pt")
    common = torch.load(common_path, weights_only=False) if os.path.exists(common_path) else {}
    opt = model.optimizer
    if opt is not None:
        opt.reload_model_params()
        if load_optimizer and not getattr(args, "finetune", False):
            want = {}
            for bi, st in enumerate(opt.state):
                for k, v in st.items():
                    key = f"optimizer.state.buf{bi}.rank{model.buffers[bi].group_rank}.{k}"
                    if key in meta and tuple(meta[key].size) == tuple(v.shape):
                        want[key] = torch.empty(v.shape, dtype=v.dtype)
            _dcp_load(path, want)
            for bi, st in enumerate(opt.state):
                for k, v in st.items():
                    key = f"optimizer.state.buf{bi}.rank{model.buffers[bi].group_rank}.{k}"
                    if key in want:
                        v.copy_(want[key])
            opt.step_count = common.get("optimizer_step", 0)
            if model.scheduler is not None and common.get("opt_param_scheduler"):
                model.scheduler.load_state_dict(common["opt_param_scheduler"])
    if not getattr(args, "no_load_rng", False) and not getattr(args, "finetune", False):
        rank = dist.get_rank() if _world() else 0
        own = os.path.join(path, f"rng_rank{rank:05d}.pt")
        if os.path.exists(own):
            restore_rng_state(torch.load(own, weights_only=False))
        elif common.get("rng_state"):  # a checkpoint written by another layout (or an older one): rank 0's host stream only
            torch.set_rng_state(common["rng_state"]["torch"])
    return iteration if isinstance(iteration, int) else None


def collect_rng_state() -> dict:
    """This rank's random streams: torch host and device generators, ``random``, numpy, and the model-parallel
    generators parameters and dropout draw from (Megatron checkpoints carry the same per rank)."""
    import random

    import numpy as np

    from slime_b200.parallel import tensor_parallel as tp

    out = {"torch": torch.get_rng_state(), "python": random.getstate(), "numpy": np.random.get_state(),
           "tracker": {k: g.get_state() for k, g in tp.get_rng_tracker().states.items()}}  # fmt: skip
    if torch.cuda.is_available():
        out["cuda"] = torch.cuda.get_rng_state()
    return out


def restore_rng_state(state: dict) -> None:
    import random

    import numpy as np

    from slime_b200.parallel import tensor_parallel as tp

    torch.set_rng_state(state["torch"])
    random.setstate(state["python"])
    np.random.set_state(state["numpy"])
    if "cuda" in state and torch.cuda.is_available():
        torch.cuda.set_rng_state(state["cuda"])
    gens = tp.get_rng_tracker().states
    for k, st in state.get("tracker", {}).items():
        if k in gens:
            gens[k].set_state(st.to(gens[k].get_state().device) if hasattr(st, "to") else st)
