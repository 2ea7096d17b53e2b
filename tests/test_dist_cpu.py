"""Distributed training invariants on CPU: gloo ranks under torchrun (context, data and tensor parallel)."""

import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("mode,world,port", [("cp", 2, 29681), ("cp", 4, 29682), ("dp", 2, 29683), ("dp", 3, 29684), ("tp", 2, 29685)])
def test_invariants(mode, world, port):
    env = dict(os.environ, MODE=mode, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests/multigpu/dist_cpu_check.py")],
                       env=env, cwd=ROOT, capture_output=True, text=True, timeout=280)  # fmt: skip
    assert r.returncode == 0 and f"RESULT ok mode={mode} world={world}" in r.stdout, r.stdout[-1500:] + r.stderr[-3000:]
