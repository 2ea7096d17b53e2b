"""Rank-local expert weight routing: the transfer planner (pure function) and one executed plan on gloo ranks."""

import os
import subprocess
import sys

import pytest

from slime_b200.weight_sync.expert_routing import ExpertTensor, expert_shard_targets, plan_expert_transfers, routable

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _tensors(layers, experts, trainer_ep, world):
    out = []
    per = experts // trainer_ep
    for L in range(layers):
        for e in range(experts):
            src = (e // per) % world  # expert-data-parallel rank 0 of the shard
            for fc, nbytes in ((1, 6000), (2, 3000)):
                out.append(ExpertTensor(f"decoder.layers.{L}.mlp.experts.linear_fc{fc}.weight{e}", nbytes, src, (nbytes // 2,)))
    return out


def test_targets_of_two_engines_with_moe_dp():
    t = expert_shard_targets([4, 4], [0, 4], ep_size=2, moe_dp_size=2, world_size=8)
    assert t == [(0, 2, 4, 6), (1, 3, 5, 7)]
    with pytest.raises(ValueError):
        expert_shard_targets([3], [0], 2, 2, 8)


def test_plan_delivers_every_tensor_exactly_to_its_hosts_within_budget():
    world, experts, trainer_ep = 8, 16, 4
    targets = expert_shard_targets([8], [0], ep_size=8, moe_dp_size=1, world_size=world)
    tensors = _tensors(3, experts, trainer_ep, world)
    budget = 20000
    rounds = plan_expert_transfers(tensors, experts, targets, budget)
    seen, last_layer = {}, -1
    for rnd in rounds:
        load = {}
        layers = {t.layer_expert[0] for tr in rnd for t in tr.tensors}
        assert len(layers) == 1 and min(layers) >= last_layer  # one layer per round, layers in order
        last_layer = min(layers)
        for tr in rnd:
            for r in set(tr.dst_ranks) | {tr.src_rank}:
                load[r] = load.get(r, 0) + tr.nbytes
            for t in tr.tensors:
                hosts = set(tr.dst_ranks) | ({tr.src_rank} if tr.src_hosts_it else set())
                assert t.name not in seen
                seen[t.name] = hosts
        assert max(load.values()) <= budget
    assert len(seen) == len(tensors)
    for t in tensors:
        assert seen[t.name] == set(targets[t.layer_expert[1] // (experts // 8)])
    with pytest.raises(ValueError):
        plan_expert_transfers(tensors, experts, targets, 100)


def test_routable_conditions():
    import argparse

    a = argparse.Namespace()
    assert routable(a, engine_pp=1, engine_ep=8, expert_tp=1, engine_gpu_counts=[8])[0]
    assert not routable(a, engine_pp=2, engine_ep=8, expert_tp=1, engine_gpu_counts=[8])[0]
    assert not routable(a, engine_pp=1, engine_ep=1, expert_tp=1, engine_gpu_counts=[8])[0]
    assert not routable(a, engine_pp=1, engine_ep=4, expert_tp=1, engine_gpu_counts=[8])[0]  # engine size != ep * moe-dp


def test_plan_executes_on_gloo_ranks():
    env = dict(os.environ, MODE="expert_route", MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
                        "127.0.0.1", "--master-port", "29688", os.path.join(ROOT, "tests/multigpu/dist_cpu_check.py")],
                       env=env, cwd=ROOT, capture_output=True, text=True, timeout=280)  # fmt: skip
    assert r.returncode == 0 and "RESULT ok mode=expert_route" in r.stdout, r.stdout[-1500:] + r.stderr[-3000:]
