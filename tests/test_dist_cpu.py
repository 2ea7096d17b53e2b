"""Distributed training invariants on CPU: gloo ranks under torchrun (context, data and tensor parallel)."""

import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("mode,world,port", [("cp", 2, 29681), ("cp", 4, 29682), ("dp", 2, 29683), ("dp", 3, 29684), ("tp", 2, 29685), ("reload", 4, 29686)])
def test_invariants(mode, world, port):
    env = dict(os.environ, MODE=mode, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests/multigpu/dist_cpu_check.py")],
                       env=env, cwd=ROOT, capture_output=True, text=True, timeout=280)  # fmt: skip
    assert r.returncode == 0 and f"RESULT ok mode={mode} world={world}" in r.stdout, r.stdout[-1500:] + r.stderr[-3000:]


@pytest.mark.parametrize("mode,world,port", [("tp", 2, 29691), ("tp_sp", 2, 29692), ("pp", 2, 29693), ("pp_vpp", 2, 29694),
                                             ("ep", 2, 29695), ("dp", 2, 29696), ("tp_dp", 4, 29697), ("cp", 2, 29698),
                                             ("tp_sp_moe", 2, 29701), ("tp_ep_moe", 2, 29702)])
def test_model_under_parallel_layout_matches_single_rank_oracle(mode, world, port):
    """4-layer trainer model (qk-norm, GQA, dense or MoE) under each layout: loss, gradient shards and gradient norm
    equal a plain-PyTorch single-rank transformer."""
    env = dict(os.environ, MODE=mode, DEVICE="cpu", MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests/multigpu/model_parallel_check.py")],
                       env=env, cwd=ROOT, capture_output=True, text=True, timeout=280)  # fmt: skip
    assert r.returncode == 0 and f"RESULT ok mode={mode} world={world}" in r.stdout, r.stdout[-1500:] + r.stderr[-3000:]


def test_colocated_moe_with_fp8_engine_and_rollout_routing_replay():
    """Two gloo ranks: expert-parallel trainer, one block-fp8 rollout engine per rank, routers replaying the engine's
    expert choices through forward, log-prob pass and recomputed backward."""
    env = dict(os.environ, DEVICE="cpu", MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                        "127.0.0.1", "--master-port", "29699", os.path.join(ROOT, "tests/multigpu/colocated_moe_check.py")],
                       env=env, cwd=ROOT, capture_output=True, text=True, timeout=400)  # fmt: skip
    assert r.returncode == 0 and "RESULT ok world=2 ep=2" in r.stdout, r.stdout[-1500:] + r.stderr[-3000:]


@pytest.mark.parametrize("kind,port", [("dsa", 29745), ("mla", 29746)])
def test_allgather_context_parallelism_of_latent_attention(kind, port):
    """Two gloo ranks hold the two contiguous halves of a micro-batch's stream; keys, values and indexer keys are gathered
    inside the attention layers. Logits, summed gradients, redistributed response log-probs / entropies / values and the
    rows of a top-p keep mask equal the single-rank run."""
    env = dict(os.environ, ALLGATHER_CP_MODEL=kind, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests/multigpu/allgather_cp_check.py")],
                       env=env, cwd=ROOT, capture_output=True, text=True, timeout=280)  # fmt: skip
    assert r.returncode == 0 and f"RESULT ok world=2 model={kind}" in r.stdout, r.stdout[-1500:] + r.stderr[-3000:]
