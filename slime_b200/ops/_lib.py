"""ctypes binding of the sm_100a kernel library (``_kernels.so``).

The library is built in-tree by ``slime_b200.ops.build``. On a machine with a GPU
the kernels are mandatory: a missing or stale library raises instead of silently
falling back to PyTorch ops. CPU tensors take the PyTorch reference path in
``slime_b200.ops`` (that is what the CPU test-suite exercises).
"""

from __future__ import annotations

import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_kernels.so")
_lock = threading.Lock()
_lib = None
_launches = 0  # number of kernel-library calls issued by this process (bench reports it)

c_void_p, c_int, c_long, c_float, c_ulonglong = (
    ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float, ctypes.c_ulonglong,
)  # fmt: skip

P, I, L, F = c_void_p, c_int, c_long, c_float

_SIGS = {
    "sb_gemm_bf16": [P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, P, I, P],
    "sb_symm_barrier": [P, I, I, ctypes.c_uint, I, P, P],
    "sb_symm_barrier_dev": [P, I, I, P, I, P, P],
    "sb_tp_ar_add_rmsnorm": [P, P, P, P, P, P, P, I, I, F, I, I, I, P, P],
    "sb_dp_reduce_shard": [P, I, I, I, L, L, P, P, P, P, P],
    "sb_dp_adam_bcast": [P, P, P, P, P, I, I, I, L, L, F, F, F, F, F, F, F, F, F, P, I, P],
    "sb_group_fp8_quant_1x128": [P, P, P, P, I, I, L, L, I, P],
    "sb_moe_topk": [P, P, P, P, L, I, I, I, I, F, P],
    "sb_moe_scatter_rows": [P, P, P, L, I, I, P],
    "sb_moe_gather_sum": [P, P, P, P, L, I, I, I, P],
    "sb_moe_route_weight_grad": [P, P, P, P, L, I, I, P],
    "sb_gemm_fp8_block": [P, P, P, P, P, I, I, I, I, I, I, I, P, I, P],
    "sb_gemm_fp8_grouped": [P, P, P, P, P, P, I, I, I, I, I, I, I, I, P, I, P],
    
    "sb_gemm_bf16_grouped": [P, P, P, P, I, I, I, I, I, I, I, I, I, I, P, I, P],
    "sb_gemm_bf16_splitk": [P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, I, P, I, P],
    "sb_rmsnorm_fwd": [P, P, P, P, P, P, I, I, F, P],
    "sb_rmsnorm_fwd_f32x": [P, P, P, P, P, P, I, I, F, P],
    "sb_rmsnorm_bwd": [P, P, P, P, P, P, P, P, I, I, I, I, P],
    "sb_rope": [P, P, P, P, P, P, I, I, I, I, I, I, F, F, P],
    "sb_swiglu_fwd": [P, P, L, I, P],
    "sb_swiglu_bwd": [P, P, P, L, I, P],
    "sb_embedding_fwd": [P, P, P, I, I, I, I, P],
    "sb_embedding_bwd": [P, P, P, I, I, I, I, P],
    "sb_add_bf16": [P, P, P, L, P],
    "sb_sqnorm": [P, L, I, P, I, P, I, P],
    "sb_adam": [P, P, P, P, I, P, L, F, F, F, F, F, F, F, F, F, P, I, P],
    "sb_softmax_stats": [P, P, P, I, I, L, I, F, P],
    "sb_finalize_logprob": [P, P, P, P, I, P],
    "sb_dlogits": [P, P, P, P, P, P, P, I, I, L, L, I, F, P],
    "sb_pg_loss": [P, P, P, P, P, P, P, P, I, F, F, F, I, P],
    "sb_sample": [P, I, L, I, I, P, P, P, P, P, P, P, P, P, P, I, P],
    "sb_kv_write": [P, P, P, P, P, I, I, I, I, P],
    "sb_rope_kv_write": [P, P, P, P, P, P, P, P, I, I, I, I, I, F, P],
    "sb_decode_prepare": [P, P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, P],
    "sb_decode_advance": [P, P, P, P, P, I, P],
    "sb_paged_decode": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, P],
    "sb_paged_decode_tc": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, P, P],
    "sb_paged_decode_ws": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, P, I, L, L, P],
    "sb_paged_decode_ws_load_path_only": [I],
    "sb_block_fp8_quant": [P, P, P, I, I, L, L, I, I, I, P],
    "sb_block_fp8_dequant": [P, P, P, I, I, I, I, P],
    "sb_fake_int4": [P, P, P, P, I, I, I, I, I, P],
    "sb_router_gemm": [P, P, P, I, I, I, P],
}


class KernelLibraryMissing(RuntimeError):
    pass


def available() -> bool:
    return os.path.exists(_SO)


def lib():
    """Load (once) and return the kernel library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(_SO):
                raise KernelLibraryMissing(
                    f"{_SO} not found: build it with `python -m slime_b200.ops.build` (CUDA tensors need the sm_100a kernels)"
                )
            handle = ctypes.CDLL(_SO)
            for name, argtypes in _SIGS.items():
                try:
                    fn = getattr(handle, name)
                except AttributeError:
                    continue  # optional symbol groups are bound by their own modules
                fn.argtypes = argtypes
                fn.restype = c_int
            _lib = handle
    return _lib


def bind(name: str, argtypes, restype=c_int):
    fn = getattr(lib(), name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(rc: int, what: str):
    global _launches
    _launches += 1
    if rc != 0:
        detail = ""
        try:
            fn = lib().sb_last_error
            fn.restype = ctypes.c_char_p
            fn.argtypes = []
            detail = (fn() or b"").decode(errors="replace")
        except Exception:  # noqa: BLE001
            pass
        raise RuntimeError(f"{what} failed with CUDA error {rc} {detail}")


def launch_count() -> int:
    return _launches


_status = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 that kernels with bounded waits write a non-zero code into."""
    key = torch.device(device).index or 0
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[key] = t
    return t


STATUS_NAMES = {1: "ERR_WAIT_FULL", 2: "ERR_WAIT_EMPTY", 3: "ERR_WAIT_TMEM_FULL", 4: "ERR_WAIT_TMEM_EMPTY",
                5: "ERR_WAIT_PEER", 6: "ERR_BOUNDS"}  # fmt: skip


class KernelWaitExpired(RuntimeError):
    """A bounded wait inside a kernel gave up. ``code`` is the low byte of the status word, ``where`` the rest
    (CTA or peer index). The results of the launches since the last check are not to be used."""

    def __init__(self, code: int, where: int):
        super().__init__(f"kernel wait limit expired: {STATUS_NAMES.get(code, code)} (code={code}, where={where})")
        self.code, self.where = code, where


def check_status(device) -> None:
    """Host-side check of the bounded-wait status word (synchronises). Clears the word before raising, so the
    kernels run normally again afterwards."""
    t = status_word(device)
    code = int(t.item())
    if code != 0:
        t.zero_()
        raise KernelWaitExpired(code & 0xFF, code >> 8)


def set_peer_wait_limit(seconds: float | None) -> float:
    """Limit of every wait on another GPU (signal-pad barriers, per-CTA peer flags); ``None`` restores the default.
    Returns the previous limit in seconds."""
    get = bind("sb_get_peer_wait_limit_ns", [], ctypes.c_ulonglong)
    st = bind("sb_set_peer_wait_limit_ns", [ctypes.c_ulonglong], None)
    old = get() / 1e9
    st(0 if seconds is None else max(1, int(seconds * 1e9)))
    return old


_sm_count = {}


def sm_count(device) -> int:
    key = torch.device(device).index or 0
    if key not in _sm_count:
        _sm_count[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _sm_count[key]
