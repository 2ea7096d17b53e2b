"""Mixture-of-experts layer: top-k router, expert-parallel dispatch/combine, grouped expert MLPs.

Replaces Megatron's TopKRouter + alltoall token dispatcher + grouped MLP
(configured by scripts/models/qwen3-30B-A3B.sh:40-48 in the reference).
Routing can be recorded and replayed (R2: trainer forward -> backward recompute,
R3: rollout engine -> trainer) through ``slime_b200.utils.routing_replay``.

Expert parallel layout: expert ``e`` lives on EP rank ``e // (E / ep)``. Tokens are
exchanged with an all-to-all whose split sizes come from a first (tiny) all-to-all
of per-expert counts; received rows are already grouped by (local expert) after a
local sort, so each expert runs two dense tcgen05 GEMMs on a contiguous slice.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as nn

from slime_b200 import ops
from slime_b200.ops import grouped
from slime_b200.models.config import ModelConfig
from slime_b200.parallel import state as mpu
from slime_b200.parallel import tensor_parallel as tp
from slime_b200.utils import routing_replay


def _param(shape, dtype, device, std, generator=None):
    t = torch.empty(*shape, dtype=torch.float32, device=device).normal_(0.0, std, generator=generator)
    return nn.Parameter(t.to(dtype))


def group_limited(scores: torch.Tensor, num_groups: int, group_topk: int) -> torch.Tensor:
    """Group-limited routing: experts are split into ``num_groups`` equal groups, a group's score is the sum of its two
    best experts, and only experts of the ``group_topk`` best groups stay eligible (the others get -inf)."""
    T, E = scores.shape
    per = scores.view(T, num_groups, E // num_groups)
    group_score = per.topk(min(2, per.shape[-1]), dim=-1).values.sum(-1)
    keep = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, group_score.topk(group_topk, dim=-1).indices, True)
    return per.masked_fill(~keep[:, :, None], float("-inf")).view(T, E)


class TopKRouter(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_number: int, dtype, device):
        super().__init__()
        self.cfg, self.layer_number = cfg, layer_number
        gen = tp.get_rng_tracker().states.get("default")
        self.weight = tp.set_tp_attrs(_param((cfg.num_experts, cfg.hidden_size), dtype, device, cfg.init_method_std, gen), False)
        if cfg.moe_router_enable_expert_bias:
            self.register_buffer("expert_bias", torch.zeros(cfg.num_experts, dtype=torch.float32, device=device))
        else:
            self.expert_bias = None
        self.replay = routing_replay.RoutingReplay.register(layer_number)

    def forward(self, x):
        """x: [T, H] -> (probs [T, k] fp32, indices [T, k] int64, aux_loss)."""
        cfg = self.cfg
        logits = ops.router_gemm(x.detach(), self.weight.detach()) if not torch.is_grad_enabled() else (
            x.float() @ self.weight.float().t()
        )
        k = cfg.moe_router_topk
        if cfg.moe_router_score_function == "sigmoid":
            scores = torch.sigmoid(logits)
            sel = scores + self.expert_bias if self.expert_bias is not None else scores
            if cfg.moe_router_num_groups and cfg.moe_router_group_topk and cfg.moe_router_num_groups > 1:
                sel = group_limited(sel, cfg.moe_router_num_groups, cfg.moe_router_group_topk)
            idx = self.replay.compute_topk(sel, k)
            probs = scores.gather(-1, idx)
            if cfg.norm_topk_prob:
                probs = probs / (probs.sum(-1, keepdim=True) + 1e-20)
        elif cfg.moe_router_pre_softmax or cfg.norm_topk_prob is False:
            scores = torch.softmax(logits, -1)
            idx = self.replay.compute_topk(scores, k)
            probs = scores.gather(-1, idx)
        else:
            # softmax over the selected logits == renormalised top-k of the full softmax
            idx = self.replay.compute_topk(logits, k)
            probs = torch.softmax(logits.gather(-1, idx), -1)
        if cfg.moe_router_topk_scaling_factor:
            probs = probs * cfg.moe_router_topk_scaling_factor
        aux = None
        if cfg.moe_aux_loss_coeff and torch.is_grad_enabled():
            full = torch.softmax(logits, -1)
            load = torch.zeros(cfg.num_experts, device=x.device).index_add_(
                0, idx.reshape(-1), torch.ones(idx.numel(), device=x.device)
            )
            aux = cfg.moe_aux_loss_coeff * cfg.num_experts * (full.mean(0) * load / max(idx.numel(), 1)).sum()
        return probs, idx, aux


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty((sum(out_splits), *x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.in_splits), *g.shape[1:]))
        dist.all_to_all_single(
            out, g.contiguous(), output_split_sizes=ctx.in_splits, input_split_sizes=ctx.out_splits, group=ctx.group
        )
        return out, None, None, None


class GroupedExperts(nn.Module):
    """Local experts; parameters named ``linear_fc1.weight{e}`` / ``linear_fc2.weight{e}`` (local index)."""

    def __init__(self, cfg: ModelConfig, dtype, device, num_local: int):
        super().__init__()
        self.cfg, self.num_local = cfg, num_local
        etp = mpu.get_expert_tensor_parallel_world_size()
        f = cfg.moe_ffn_hidden_size // etp
        self.f = f
        gen = tp.get_rng_tracker().states.get("ep")
        out_std = cfg.init_method_std / math.sqrt(2.0 * cfg.num_layers)
        self.linear_fc1 = nn.Module()
        self.linear_fc2 = nn.Module()
        for e in range(num_local):
            w1 = tp.set_tp_attrs(_param((2 * f, cfg.hidden_size), dtype, device, cfg.init_method_std, gen), etp > 1, 0, 2, "column")
            w2 = tp.set_tp_attrs(_param((cfg.hidden_size, f), dtype, device, out_std, gen), etp > 1, 1, 1, "row")
            w1.is_expert = w2.is_expert = True
            w1.num_local_experts = w2.num_local_experts = num_local  # global expert id = ep_rank * num_local + e
            self.linear_fc1.register_parameter(f"weight{e}", w1)
            self.linear_fc2.register_parameter(f"weight{e}", w2)
        self.int4_qat_group = 0  # >0: fake-INT4 the expert weights in forward (straight-through backward)
        self.use_grouped_gemm = True  # False: one GEMM pair per expert (kept as the oracle of the grouped path)

    def _w(self, mod, e):
        w = getattr(mod, f"weight{e}")
        if self.int4_qat_group > 0:
            return ops.FakeInt4STE.apply(w, self.int4_qat_group)
        return w

    def forward(self, x, counts: list[int]):
        """x: [sum(counts), H] rows grouped by local expert."""
        if self.int4_qat_group == 0 and x.shape[0] > 0 and self.use_grouped_gemm:
            # one grouped launch per projection instead of a loop over experts (rows padded to the GEMM's row tile)
            lay = grouped.PaddedLayout(counts, x.device)
            w1 = [getattr(self.linear_fc1, f"weight{e}") for e in range(self.num_local)]
            w2 = [getattr(self.linear_fc2, f"weight{e}") for e in range(self.num_local)]
            act = ops.swiglu(grouped.grouped_linear(lay.pad(x), lay, w1))
            return lay.unpad(grouped.grouped_linear(act, lay, w2))
        outs, start = [], 0
        for e, n in enumerate(counts):
            if n == 0:
                continue
            xe = x[start : start + n]
            act = ops.swiglu(ops.linear(xe, self._w(self.linear_fc1, e)))
            outs.append(ops.linear(act, self._w(self.linear_fc2, e)))
            start += n
        if not outs:
            return x.new_zeros((0, x.shape[-1]))
        return torch.cat(outs, dim=0)


class MoELayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_number: int, dtype, device, sequence_parallel: bool):
        super().__init__()
        self.cfg, self.sp = cfg, sequence_parallel
        self.ep = mpu.get_expert_model_parallel_world_size()
        self.ep_rank = mpu.get_expert_model_parallel_rank()
        assert cfg.num_experts % self.ep == 0
        self.num_local = cfg.num_experts // self.ep
        self.pre_mlp_layernorm = nn.Module()
        self.pre_mlp_layernorm.weight = tp.set_tp_attrs(
            nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device)), False
        )
        self.router = TopKRouter(cfg, layer_number, dtype, device)
        # replicated parameters that only see this rank's rows under sequence parallelism: their gradients are partial
        # sums and must be added up over the tensor-parallel group
        self.pre_mlp_layernorm.weight.sequence_parallel = sequence_parallel
        self.router.weight.sequence_parallel = sequence_parallel
        self.experts = GroupedExperts(cfg, dtype, device, self.num_local)
        if cfg.moe_shared_expert_intermediate_size:
            from slime_b200.models.gpt import MLP

            self.shared_experts = MLP(cfg, dtype, device, sequence_parallel, ffn=cfg.moe_shared_expert_intermediate_size,
                                      with_norm=False)  # fmt: skip
            if cfg.moe_shared_expert_gate:
                self.shared_experts.gate_weight = tp.set_tp_attrs(_param((1, cfg.hidden_size), dtype, device, cfg.init_method_std), False)
                self.shared_experts.gate_weight.sequence_parallel = sequence_parallel
        else:
            self.shared_experts = None
        self.aux_loss = None

    def forward(self, x, residual):
        cfg = self.cfg
        normed, residual = ops.rmsnorm(x, self.pre_mlp_layernorm.weight, cfg.norm_epsilon, residual)
        T, H = normed.shape
        probs, idx, self.aux_loss = self.router(normed)
        k = idx.shape[1]

        # ---- permute: one row per (token, slot), sorted by global expert id (stable)
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        tok_of_row = order // k
        rows = normed.index_select(0, tok_of_row)
        counts = torch.zeros(cfg.num_experts, dtype=torch.long, device=x.device).scatter_add_(0, flat_e, torch.ones_like(flat_e))

        if self.ep > 1:
            group = mpu.get_expert_model_parallel_group()
            send_counts = counts.view(self.ep, self.num_local)
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts.view(-1), send_counts.reshape(-1).contiguous(), group=group)
            # the one host synchronisation of the layer: NCCL's all-to-all wants its split sizes on the host
            send_h, recv_h = torch.stack([send_counts, recv_counts]).tolist()
            in_splits, out_splits = [sum(r) for r in send_h], [sum(r) for r in recv_h]
            recv = _AllToAll.apply(rows, out_splits, in_splits, group)
            # received rows are ordered (source rank, local expert); regroup by local expert
            total = sum(out_splits)
            src_e = torch.repeat_interleave(torch.arange(self.num_local, device=x.device).repeat(self.ep), recv_counts.reshape(-1),
                                            output_size=total)  # fmt: skip
            local_order = torch.argsort(src_e, stable=True)
            grouped = recv.index_select(0, local_order)
            local_counts = [sum(recv_h[r][e] for r in range(self.ep)) for e in range(self.num_local)]
            y = self.experts(grouped, local_counts)
            back = torch.empty_like(y)
            back = back.index_copy(0, local_order, y)
            out_rows = _AllToAll.apply(back, in_splits, out_splits, group)
        else:
            out_rows = self.experts(rows, counts.tolist())

        # ---- combine: weight by router prob and sum the k copies of each token (fixed order)
        w = probs.reshape(-1).index_select(0, order).to(out_rows.dtype)
        weighted = out_rows * w[:, None]
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=order.device)
        out = weighted.index_select(0, inv).view(T, k, H).float().sum(1).to(x.dtype)
        if self.shared_experts is not None:
            shared = self.shared_experts.ffn(normed)
            if cfg.moe_shared_expert_gate:
                shared = shared * torch.sigmoid(normed.float() @ self.shared_experts.gate_weight.float().t()).to(shared.dtype)
            out = out + shared
        return out, residual
