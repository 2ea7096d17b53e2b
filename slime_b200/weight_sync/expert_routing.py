"""Rank-local routing of expert weights during weight sync.

With an expert-parallel trainer and colocated expert-parallel engines, gathering every expert on every rank and then
letting each engine rank throw away the experts it does not host moves ``ep`` times more bytes than needed. Instead each
routed-expert tensor travels once, from the trainer rank that owns it to exactly the ranks whose engine shard hosts that
expert, as point-to-point transfers packed into rounds whose staging memory per rank is bounded by
``--update-weight-buffer-size``.

    targets = expert_shard_targets(engine_gpu_counts, engine_gpu_offsets, ep_size, moe_dp_size, world)
    plan    = plan_expert_transfers(expert_tensors, num_experts, targets, buffer_size)
    for rnd in plan:  run_round(rnd, my_rank, fetch, deliver, group)

The plan is a pure function of metadata that every rank holds after one ``all_gather_object`` of the local expert
names, so all ranks build the same rounds without further coordination. Covers the role of
slime/backends/megatron_utils/update_weight/expert_routing.py:221-380 in the reference (there the transfers feed SGLang
engine processes through CUDA IPC; here the engine is an object of the same process and ``deliver`` writes its buffers).
"""

from __future__ import annotations

import dataclasses
import re
from collections import defaultdict

import torch
import torch.distributed as dist

_EXPERT_NAME = re.compile(r"decoder\.layers\.(\d+)\.mlp\.experts\.linear_fc([12])\.weight(\d+)$")


@dataclasses.dataclass(frozen=True)
class ExpertTensor:
    name: str  # global name: ...experts.linear_fc{1,2}.weight{global expert id}
    nbytes: int
    src_rank: int  # trainer rank that holds it (one owner per tensor: expert-data-parallel rank 0 of its EP shard)
    shape: tuple = ()
    dtype: str = "bfloat16"

    @property
    def layer_expert(self) -> tuple[int, int]:
        m = _EXPERT_NAME.search(self.name)
        if m is None:
            raise ValueError(f"not a routed-expert tensor: {self.name}")
        return int(m.group(1)), int(m.group(3))


@dataclasses.dataclass(frozen=True)
class Transfer:
    src_rank: int
    dst_ranks: tuple[int, ...]  # the other ranks that host the expert
    tensors: tuple[ExpertTensor, ...]
    src_hosts_it: bool = False  # the source's own engine shard hosts the expert too: delivered without a transfer

    @property
    def nbytes(self) -> int:
        return sum(t.nbytes for t in self.tensors)


def routable(args, *, engine_pp: int, engine_ep: int, expert_tp: int, engine_gpu_counts, moe_dp_size: int = 1) -> tuple[bool, str]:
    """Whether expert tensors can be sent shard to shard, and if not, why (logged by the caller)."""
    if engine_pp != 1:
        return False, "engine pipeline parallelism"
    if engine_ep <= 1:
        return False, "engine experts are not sharded"
    if expert_tp != 1:
        return False, "trainer experts are tensor-parallel"
    if getattr(args, "sglang_enable_eplb", False) or getattr(args, "sglang_ep_num_redundant_experts", 0):
        return False, "engine relocates or replicates experts at run time"
    if any(n != engine_ep * moe_dp_size for n in engine_gpu_counts):
        return False, "engine experts are tensor-parallel (engine size != ep * moe-dp)"
    return True, ""


def expert_shard_targets(engine_gpu_counts, engine_gpu_offsets, ep_size: int, moe_dp_size: int, world_size: int) -> list[tuple[int, ...]]:
    """``targets[s]``: global ranks (over all engines and their MoE-DP replicas) that host expert shard ``s``."""
    out: list[list[int]] = [[] for _ in range(ep_size)]
    for count, off in zip(engine_gpu_counts, engine_gpu_offsets):
        if count != ep_size * moe_dp_size:
            raise ValueError(f"engine of {count} GPUs is not ep {ep_size} x moe-dp {moe_dp_size}")
        if off < 0 or off + count > world_size:
            raise ValueError("engine GPUs lie outside the trainer world")
        for rep in range(moe_dp_size):
            for s in range(ep_size):
                out[s].append(off + rep * ep_size + s)
    return [tuple(r) for r in out]


def plan_expert_transfers(tensors: list[ExpertTensor], num_experts: int, targets: list[tuple[int, ...]],
                          buffer_size: int) -> list[list[Transfer]]:
    """Rounds of transfers. A transfer bundles the tensors of one (layer, expert) from one source; a round never asks a
    rank to stage more than ``buffer_size`` bytes (as sender plus as receiver). Layers are kept in order, so the engine
    sees complete layers early; inside a layer the largest bundles are placed first (first fit, least-loaded round)."""
    if buffer_size <= 0:
        raise ValueError("the staging budget must be positive")
    per_shard = num_experts // len(targets)
    bundles: dict[tuple[int, int, int], list[ExpertTensor]] = defaultdict(list)
    for t in tensors:
        layer, expert = t.layer_expert
        bundles[(layer, expert, t.src_rank)].append(t)
    by_layer: dict[int, list[Transfer]] = defaultdict(list)
    for (layer, expert, src), ts in bundles.items():
        hosts = targets[expert // per_shard]
        dst = tuple(r for r in hosts if r != src)  # a tensor already on its host rank stays
        by_layer[layer].append(Transfer(src, dst, tuple(sorted(ts, key=lambda x: x.name)), src in hosts))
    rounds: list[list[Transfer]] = []
    for layer in sorted(by_layer):
        todo = sorted(by_layer[layer], key=lambda tr: (-tr.nbytes, tr.dst_ranks, tr.src_rank))
        if todo and todo[0].nbytes > buffer_size:
            raise ValueError(f"one expert bundle ({todo[0].nbytes} B) exceeds the staging budget ({buffer_size} B)")
        layer_rounds: list[list[Transfer]] = []
        load: list[dict[int, int]] = []
        for tr in todo:
            ranks = set(tr.dst_ranks) | {tr.src_rank}
            fit = [i for i, ld in enumerate(load) if all(ld.get(r, 0) + tr.nbytes <= buffer_size for r in ranks)]
            i = min(fit, key=lambda i: (sum(load[i].values()), i)) if fit else len(layer_rounds)
            if not fit:
                layer_rounds.append([])
                load.append({})
            layer_rounds[i].append(tr)
            for r in ranks:
                load[i][r] = load[i].get(r, 0) + tr.nbytes
        rounds += layer_rounds
    return rounds


def collect_expert_tensors(model, group=None) -> list[ExpertTensor]:
    """Metadata of every routed-expert tensor of the trainer world (one ``all_gather_object``), global names."""
    from slime_b200.backends.train.checkpoint import global_param_name
    from slime_b200.parallel import state as mpu

    mine = []
    if mpu.get_expert_data_parallel_rank() == 0:
        for name, p in model.named_parameters():
            if getattr(p, "is_expert", False):
                mine.append(ExpertTensor(global_param_name(name, p), p.numel() * p.element_size(), dist.get_rank(),
                                         tuple(p.shape), str(p.dtype).replace("torch.", "")))  # fmt: skip
    everyone = [None] * dist.get_world_size(group)
    dist.all_gather_object(everyone, mine, group=group)
    return sorted((t for part in everyone for t in part), key=lambda t: (t.layer_expert, t.name))


def run_round(transfers: list[Transfer], my_rank: int, fetch, deliver, group=None, device=None) -> int:
    """Execute one round. ``fetch(name) -> tensor`` on the source, ``deliver(name, tensor)`` on every target (the
    source itself included when it hosts the expert: no copy through the network). Returns the bytes this rank received."""
    ops, incoming = [], []
    for tr in transfers:
        for t in tr.tensors:
            if tr.src_rank == my_rank:
                src = fetch(t.name).contiguous()
                if tr.src_hosts_it:
                    incoming.append((t.name, src))
                for d in tr.dst_ranks:
                    ops.append(dist.P2POp(dist.isend, src, d, group))
            elif my_rank in tr.dst_ranks:
                buf = torch.empty(t.shape, dtype=getattr(torch, t.dtype), device=device)
                ops.append(dist.P2POp(dist.irecv, buf, tr.src_rank, group))
                incoming.append((t.name, buf))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    got = 0
    for name, buf in incoming:
        deliver(name, buf)
        got += buf.numel() * buf.element_size()
    return got
