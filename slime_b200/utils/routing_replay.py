"""Record / replay of MoE top-k routing decisions.

R2 (``--use-routing-replay``): the top-k indices picked in the log-prob forward
are replayed in the training forward and in the backward recompute, so all three
passes route identically. R3 (``--use-rollout-routing-replay``): the indices come
from the rollout engine (``Sample.rollout_routed_experts``) instead.
The stage is selected with ``ROUTING_REPLAY_STAGE`` in {fallthrough, record,
replay_forward, replay_backward}; under ``replay_forward`` a call made from inside the backward pass (a recomputed
layer) reads the backward cursor by itself. Parity: slime/utils/routing_replay.py:81-226.
"""

from __future__ import annotations

import os

import torch


class RoutingReplay:
    all_instances: list["RoutingReplay"] = []
    _by_layer: dict[int, "RoutingReplay"] = {}

    def __init__(self, layer_number: int | None = None):
        self.layer_number = layer_number
        self.forward_index = 0
        self.backward_index = 0
        self.top_indices_list: list[torch.Tensor] = []
        RoutingReplay.all_instances.append(self)

    @classmethod
    def register(cls, layer_number: int) -> "RoutingReplay":
        inst = cls(layer_number)
        cls._by_layer[layer_number] = inst
        return inst

    # ---- storage ----------------------------------------------------------
    def record(self, top_indices: torch.Tensor):
        buf = torch.empty_like(top_indices, device="cpu", pin_memory=torch.cuda.is_available())
        buf.copy_(top_indices)
        self.top_indices_list.append(buf)

    def pop_forward(self) -> torch.Tensor:
        t = self.top_indices_list[self.forward_index]
        self.forward_index += 1
        return t

    def pop_backward(self) -> torch.Tensor:
        t = self.top_indices_list[self.backward_index]
        self.backward_index += 1
        return t

    def clear(self):
        self.forward_index = self.backward_index = 0
        self.top_indices_list = []

    def clear_forward(self):
        self.forward_index = 0

    @classmethod
    def clear_all(cls):
        for r in cls.all_instances:
            r.clear()

    @classmethod
    def clear_all_forward(cls):
        for r in cls.all_instances:
            r.clear_forward()

    # ---- the hook the router calls ---------------------------------------------
    def compute_topk(self, scores: torch.Tensor, k: int) -> torch.Tensor:
        if os.environ.get("ENABLE_ROUTING_REPLAY", "0") != "1":
            return torch.topk(scores, k, dim=-1).indices
        stage = os.environ.get("ROUTING_REPLAY_STAGE", "fallthrough")
        if stage == "fallthrough":
            return torch.topk(scores, k, dim=-1).indices
        if stage == "record":
            idx = torch.topk(scores, k, dim=-1).indices
            self.record(idx)
            return idx
        if stage in ("replay_forward", "replay_backward"):
            # A layer re-run by activation recomputation executes inside the backward pass: it takes the backward
            # cursor, so the forward cursor stays in step with the micro-batches whatever the recompute setting.
            recomputing = stage == "replay_backward" or torch._C._current_graph_task_id() != -1
            idx = (self.pop_backward() if recomputing else self.pop_forward()).to(scores.device, non_blocking=True)
            assert idx.shape[0] == scores.shape[0] and idx.shape[1] == k, (
                f"replayed routing {tuple(idx.shape)} does not match scores {tuple(scores.shape)} (k={k})"
            )
            return idx.long()
        raise ValueError(f"unknown ROUTING_REPLAY_STAGE {stage!r}")


def set_stage(stage: str):
    os.environ["ROUTING_REPLAY_STAGE"] = stage


def fill_from_rollout(routed_experts: list[torch.Tensor], layer_ids: list[int]):
    """R3: load per-micro-batch routed experts ``[T, layers, k]`` into each layer's replay list."""
    for layer in layer_ids:  # the rollout reports one column per layer of the model, dense ones included
        inst = RoutingReplay._by_layer.get(layer)
        if inst is None:
            continue
        for mb in routed_experts:
            inst.top_indices_list.append(mb[:, layer].contiguous())
