"""GPU memory choreography for colocated train + rollout.

The reference pauses whole CUDA VMM regions through an LD_PRELOAD allocator hook
(torch_memory_saver; slime/backends/megatron_utils/actor.py:206-244). Here the trainer's
state is a handful of flat buffers, so offload is explicit: optimizer shards (fp32 master
and moments) go to pinned host memory, gradient buffers are dropped (they are zeroed at
the start of every step anyway) and bf16 parameters stay (the weight sync reads them).
``tag`` bookkeeping for the engine side lives in ``Engine.release/resume_memory_occupation``.
"""

from __future__ import annotations

import gc

import torch


def available_memory(device=None) -> dict:
    if not torch.cuda.is_available():
        return {"free_GB": 0.0, "total_GB": 0.0}
    free, total = torch.cuda.mem_get_info(device)
    return {"free_GB": free / 2**30, "total_GB": total / 2**30, "allocated_GB": torch.cuda.memory_allocated(device) / 2**30,
            "reserved_GB": torch.cuda.memory_reserved(device) / 2**30}  # fmt: skip


def clear_memory():
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        torch.cuda.empty_cache()


def print_memory(msg: str, device=None) -> dict:
    info = available_memory(device)
    print(f"[memory] {msg}: {info}", flush=True)
    return info


def offload_train_state(model) -> None:
    """Move optimizer shards to pinned host memory and free gradient storage."""
    opt = model.optimizer
    if opt is not None:
        for st in opt.state:
            for k, t in list(st.items()):
                if t.is_cuda:
                    host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
                    host.copy_(t, non_blocking=True)
                    st[k] = host
        torch.cuda.synchronize()
    for b in model.buffers:
        b._grad_numel = b.grad_data.numel()
        b._grad_device = b.grad_data.device
        b.grad_data.data = torch.empty(0, dtype=b.grad_data.dtype, device=b.grad_data.device)
        for p in b.params:
            p.main_grad = None
    clear_memory()


def onload_train_state(model) -> None:
    for b in model.buffers:
        if b.grad_data.numel() == 0:
            b.grad_data = torch.zeros(b._grad_numel, dtype=b.grad_data.dtype, device=b._grad_device)
            for p, (s, e) in zip(b.params, b.offsets):
                p.main_grad = b.grad_data[s:e].view(p.shape)
    opt = model.optimizer
    if opt is not None and not opt.cpu_offload:
        dev = model.device
        for st in opt.state:
            for k, t in list(st.items()):
                if not t.is_cuda and dev.type == "cuda":
                    st[k] = t.to(dev, non_blocking=True)
        if dev.type == "cuda":
            torch.cuda.synchronize()
