"""GPU placement for trainer and rollout actors on one node (or a fixed list of nodes).

Bundles are ``(node_ip, gpu_id)`` pairs sorted by (ip, gpu id) so rank <-> GPU is deterministic.
Colocated: trainer and rollout share ``max(actor, rollout)`` GPUs starting at offset 0.
Disaggregated: trainer GPUs first, rollout GPUs after them.
Parity: slime/ray/placement_group.py:42-137 (placement) and :140-253 (group/model creation).
"""

from __future__ import annotations

import os
from dataclasses import dataclass

from slime_b200.utils.misc import get_current_node_ip


@dataclass
class Bundle:
    node_ip: str
    gpu_id: int


@dataclass
class PlacementGroup:
    bundles: list[Bundle]
    offset: int  # first bundle of this role
    count: int

    def gpu(self, i: int) -> Bundle:
        return self.bundles[self.offset + i]


def visible_gpus() -> list[int]:
    env = os.environ.get("CUDA_VISIBLE_DEVICES")
    if env:
        return [int(x) for x in env.split(",") if x.strip() != ""]
    try:
        import torch

        return list(range(torch.cuda.device_count()))
    except Exception:  # noqa: BLE001
        return []


def _layout(args) -> tuple[int, int, int]:
    """(total bundles, rollout offset, rollout count)."""
    actor = args.actor_num_nodes * args.actor_num_gpus_per_node
    rollout = args.rollout_num_gpus or 0
    if args.debug_train_only:
        return actor, 0, 0
    if getattr(args, "rollout_external", False):  # engines started elsewhere take no GPU of this placement
        return (actor, 0, 0) if args.debug_rollout_only else (actor, actor, 0)
    if args.debug_rollout_only:
        return rollout, 0, rollout
    if args.colocate:
        return max(actor, rollout), 0, rollout
    return actor + rollout, actor, rollout


def create_placement_groups(args, gpus: list[int] | None = None) -> dict[str, PlacementGroup]:
    total, r_off, r_cnt = _layout(args)
    ip = get_current_node_ip()
    gpus = gpus if gpus is not None else visible_gpus()
    if len(gpus) < total and gpus:
        raise ValueError(f"need {total} GPUs ({'colocated' if args.colocate else 'disaggregated'} placement), found {len(gpus)}")
    ids = gpus[:total] if gpus else list(range(total))  # CPU-only boxes: logical ids
    bundles = sorted((Bundle(ip, g) for g in ids), key=lambda b: (b.node_ip, b.gpu_id))
    actor = args.actor_num_nodes * args.actor_num_gpus_per_node
    groups = {"actor": PlacementGroup(bundles, 0, actor), "rollout": PlacementGroup(bundles, r_off, r_cnt)}
    if getattr(args, "use_critic", False):
        groups["critic"] = PlacementGroup(bundles, 0, actor)  # critic shares the actor's GPUs
    return groups


def validate_server_group_gpu_indices(groups: list[dict], total_rollout_gpus: int) -> None:
    """Every server group's GPU range must fit into the rollout placement group and not overlap."""
    used: set[int] = set()
    for g in groups:
        start, n = g.get("gpu_offset", 0), g["num_gpus"]
        rng = set(range(start, start + n))
        if max(rng, default=-1) >= total_rollout_gpus:
            raise ValueError(f"server group {g.get('name')} uses GPUs {sorted(rng)} but only {total_rollout_gpus} are placed")
        if rng & used:
            raise ValueError(f"server group {g.get('name')} overlaps another group on GPUs {sorted(rng & used)}")
        used |= rng
