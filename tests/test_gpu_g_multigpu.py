"""Multi-GPU checks, each a torchrun job on one node. Skipped on boxes with fewer GPUs than the check needs."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _torchrun(script, nproc, extra_env=None, timeout=420):
    """One torchrun job with a rendezvous port of its own (jobs run back to back; a port shared between them can
    still be held by the previous job's store when the next one starts)."""
    env = dict(os.environ, **(extra_env or {}))
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, script)]  # fmt: skip
    try:
        return subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=timeout)
    except subprocess.TimeoutExpired as e:
        out = (e.stdout or b"")[-3000:], (e.stderr or b"")[-3000:]
        raise AssertionError(f"{script} still running after {timeout} s; its output so far:\n{out[0]!r}\n{out[1]!r}") from None


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


@pytest.mark.parametrize("multimem", ["1", "0"])
def test_fused_dp_step_matches_nccl(kernels, multimem):
    _need(2)
    n = min(torch.cuda.device_count(), 8)
    r = _torchrun("tests/multigpu/fused_dp_check.py", n, {"SLIME_B200_DISABLE_MULTIMEM": "0" if multimem == "1" else "1"})
    assert r.returncode == 0 and "RESULT ok" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.parametrize("multimem", ["1", "0"])
def test_fused_tp_allreduce_norm_matches_nccl(kernels, multimem):
    _need(2)
    n = min(torch.cuda.device_count(), 8)
    r = _torchrun("tests/multigpu/fused_tp_check.py", n, {"SLIME_B200_DISABLE_MULTIMEM": "0" if multimem == "1" else "1"})
    assert r.returncode == 0 and "RESULT ok" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_tensor_parallel_engine_matches_single_gpu(kernels):
    _need(2)
    r = _torchrun("tests/multigpu/engine_tp_check.py", 2, timeout=300)
    assert r.returncode == 0 and "RESULT ok" in r.stdout and "fused_tp=True" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_fused_sequence_parallel_linears_match_nccl_path(kernels):
    """All-gather -> GEMM and GEMM -> reduce-scatter as single kernels, forward and backward, against NCCL + GEMM."""
    _need(2)
    n = 2 if torch.cuda.device_count() < 4 else 4
    r = _torchrun("tests/multigpu/fused_linear_check.py", n, timeout=300)
    assert r.returncode == 0 and "RESULT ok" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.parametrize("mode", ["tp_sp", "cp"])
def test_trainer_model_parallel_parity_on_gpus(kernels, mode):
    """The trainer model under TP2 + SP (fused linears, own attention kernels) and under CP2 against the fp32 oracle."""
    _need(2)
    r = _torchrun("tests/multigpu/model_parallel_check.py", 2, {"MODE": mode, "DEVICE": "cuda"}, timeout=300)
    assert r.returncode == 0 and "RESULT ok" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_colocated_grpo_with_tensor_parallel_engine(kernels):
    """Two GRPO steps with trainer and rollout engine both TP2 over the same ranks (fused decode all-reduce, fused
    linears, shard-to-shard weight sync)."""
    _need(2)
    r = _torchrun("tests/multigpu/colocated_tp_check.py", 2, {"DEVICE": "cuda"}, timeout=300)
    assert r.returncode == 0 and "RESULT ok" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_colocated_moe_with_fp8_engines_and_routing_replay(kernels):
    """Two GRPO steps on a small MoE: experts of the trainer spread over the two GPUs, one block-fp8 rollout engine per GPU
    (fp8 dense and grouped GEMMs, MoE decode in CUDA graphs), routers replaying the engines' expert choices."""
    _need(2)
    r = _torchrun("tests/multigpu/colocated_moe_check.py", 2, {"DEVICE": "cuda"}, timeout=300)
    assert r.returncode == 0 and "RESULT ok" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_expert_parallel_engine_matches_single_rank(kernels):
    """TP2 + EP2 rollout engine on a small MoE against the single-GPU engine."""
    _need(2)
    r = _torchrun("tests/multigpu/engine_tp_check.py", 2, {"ENGINE_TP_CHECK_MOE": "1"}, timeout=300)
    assert r.returncode == 0 and "RESULT ok" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
