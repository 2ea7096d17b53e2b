"""Decoder-only transformer for the training backend (dense and MoE, TP/SP/PP/EP aware).

Replaces the Megatron-core ``GPTModel`` + layer specs the reference builds in
slime/backends/megatron_utils/model_provider.py:92-239. Input is a packed
("thd") token stream with ``cu_seqlens``; there is no padding to a max length.

Parameter names follow the Megatron convention so checkpoints and weight sync
share one naming scheme:
  embedding.word_embeddings.weight
  decoder.layers.{i}.self_attention.linear_qkv.{weight,bias,layer_norm_weight}
  decoder.layers.{i}.self_attention.{q_layernorm,k_layernorm}.weight
  decoder.layers.{i}.self_attention.linear_proj.weight
  decoder.layers.{i}.mlp.linear_fc1.{weight,layer_norm_weight}   ([gate; up] rows)
  decoder.layers.{i}.mlp.linear_fc2.weight
  decoder.layers.{i}.mlp.router.weight / mlp.experts.linear_fc{1,2}.weight{e}
  decoder.final_layernorm.weight, output_layer.weight
In memory the fused qkv rows are ordered [q heads | k heads | v heads] of the
local TP shard (the on-disk Megatron layout interleaves per KV group; the
checkpoint and HF converters translate).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.utils.checkpoint

from slime_b200 import ops
from slime_b200.models.config import ModelConfig
from slime_b200.parallel import state as mpu
from slime_b200.parallel import tensor_parallel as tp


def _param(shape, dtype, device, std=None, ones=False, generator=None):
    t = torch.empty(*shape, dtype=torch.float32, device=device)
    if ones:
        t.fill_(1.0)
    elif std == 0.0:
        t.zero_()
    else:
        t.normal_(0.0, std, generator=generator)
    return nn.Parameter(t.to(dtype))


class PackedSeqParams:
    """Packed-sequence metadata: cumulative lengths (int32, device) and the longest sequence."""

    def __init__(self, cu_seqlens, max_seqlen, position_ids=None):
        self.cu_seqlens_q = self.cu_seqlens_kv = self.cu_seqlens = cu_seqlens
        self.max_seqlen_q = self.max_seqlen_kv = self.max_seqlen = int(max_seqlen)
        self.position_ids = position_ids
        self.mrope_positions = None  # [3, T] temporal / height / width streams when the batch carries images
        self.qkv_format = "thd"


def _fused_sp_linears(cfg: ModelConfig, x, rows_local: int):
    """The fused all-gather->GEMM / GEMM->reduce-scatter pair of the tensor-parallel group when it exists and this
    micro-batch fits its buffers (the same answer on every rank of the group: it depends on shapes only)."""
    if not x.is_cuda:
        return None
    from slime_b200.parallel import fused_tp

    fl = fused_tp.sequence_parallel_linears(mpu.get_tensor_model_parallel_group(), cfg.hidden_size, x.device)
    return fl if fl is not None and fl.fits(rows_local, cfg.hidden_size) else None


class SelfAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_number: int, dtype, device, sequence_parallel: bool):
        super().__init__()
        self.cfg, self.sp = cfg, sequence_parallel
        tps = mpu.get_tensor_model_parallel_world_size()
        assert cfg.num_attention_heads % tps == 0 and cfg.num_query_groups % tps == 0, "heads must divide by tp"
        self.hq, self.hkv, self.d = cfg.num_attention_heads // tps, cfg.num_query_groups // tps, cfg.head_dim
        h = cfg.hidden_size
        gen = tp.get_rng_tracker().states.get("tp")
        out_std = cfg.init_method_std / math.sqrt(2.0 * cfg.num_layers)
        qkv_rows = (self.hq + 2 * self.hkv) * self.d
        self.linear_qkv = nn.Module()
        self.linear_qkv.weight = tp.set_tp_attrs(_param((qkv_rows, h), dtype, device, cfg.init_method_std, generator=gen), True, 0, 1, "column")
        self.linear_qkv.layer_norm_weight = tp.set_tp_attrs(_param((h,), dtype, device, ones=True), False)
        self.linear_qkv.layer_norm_weight.sequence_parallel = sequence_parallel
        if cfg.add_qkv_bias:
            self.linear_qkv.bias = tp.set_tp_attrs(_param((qkv_rows,), dtype, device, 0.0), True, 0, 1, "column")
        else:
            self.linear_qkv.bias = None
        if cfg.qk_layernorm:
            self.q_layernorm = nn.Module()
            self.k_layernorm = nn.Module()
            self.q_layernorm.weight = tp.set_tp_attrs(_param((self.d,), dtype, device, ones=True), False)
            self.k_layernorm.weight = tp.set_tp_attrs(_param((self.d,), dtype, device, ones=True), False)
            # replicated across TP but fed TP-sharded heads: grads must be summed over TP
            self.q_layernorm.weight.needs_tp_grad_reduce = True
            self.k_layernorm.weight.needs_tp_grad_reduce = True
        else:
            self.q_layernorm = self.k_layernorm = None
        self.linear_proj = nn.Module()
        self.linear_proj.weight = tp.set_tp_attrs(_param((h, self.hq * self.d), dtype, device, out_std, generator=gen), True, 1, 1, "row")

    def forward(self, x, residual, rope_table, packed: PackedSeqParams):
        cfg = self.cfg
        normed, residual = ops.rmsnorm(x, self.linear_qkv.layer_norm_weight, cfg.norm_epsilon, residual)
        fused = _fused_sp_linears(cfg, normed, normed.shape[0]) if self.sp else None
        if fused is not None:
            qkv = fused.column(normed, self.linear_qkv.weight, self.linear_qkv.bias)
        else:
            inp = tp.gather_from_sequence_parallel_region(normed) if self.sp else tp.copy_to_tensor_model_parallel_region(normed)
            qkv = ops.linear(inp, self.linear_qkv.weight, self.linear_qkv.bias)
        cp = mpu.get_context_parallel_world_size()
        ctx = ops.rope_attention(
            qkv, packed.position_ids, rope_table, packed.cu_seqlens, packed.max_seqlen, self.hq, self.hkv, self.d,
            self.q_layernorm.weight if self.q_layernorm is not None else None,
            self.k_layernorm.weight if self.k_layernorm is not None else None, cfg.norm_epsilon,
            cp_local_cu_seqlens=getattr(packed, "local_cu_seqlens", None) if cp > 1 else None,
            cp_group=mpu.get_context_parallel_group() if cp > 1 else None,
        )  # fmt: skip
        if fused is not None:
            return fused.row(ctx, self.linear_proj.weight), residual
        out = ops.linear(ctx, self.linear_proj.weight)
        out = tp.reduce_scatter_to_sequence_parallel_region(out) if self.sp else tp.reduce_from_tensor_model_parallel_region(out)
        return out, residual


class MLP(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype, device, sequence_parallel: bool, ffn: int | None = None, with_norm=True):
        super().__init__()
        self.cfg, self.sp = cfg, sequence_parallel
        tps = mpu.get_tensor_model_parallel_world_size()
        ffn = ffn or cfg.ffn_hidden_size
        assert ffn % tps == 0
        self.f = ffn // tps
        h = cfg.hidden_size
        gen = tp.get_rng_tracker().states.get("tp")
        out_std = cfg.init_method_std / math.sqrt(2.0 * cfg.num_layers)
        self.linear_fc1 = nn.Module()
        # rows: [gate (f) ; up (f)] of the local shard; partition_stride 2 = "GLU halves sharded separately"
        self.linear_fc1.weight = tp.set_tp_attrs(_param((2 * self.f, h), dtype, device, cfg.init_method_std, generator=gen), True, 0, 2, "column")
        if with_norm:
            self.linear_fc1.layer_norm_weight = tp.set_tp_attrs(_param((h,), dtype, device, ones=True), False)
            self.linear_fc1.layer_norm_weight.sequence_parallel = sequence_parallel
        self.linear_fc2 = nn.Module()
        self.linear_fc2.weight = tp.set_tp_attrs(_param((h, self.f), dtype, device, out_std, generator=gen), True, 1, 1, "row")

    def forward(self, x, residual):
        normed, residual = ops.rmsnorm(x, self.linear_fc1.layer_norm_weight, self.cfg.norm_epsilon, residual)
        return self.ffn(normed), residual

    def ffn(self, normed):
        fused = _fused_sp_linears(self.cfg, normed, normed.shape[0]) if self.sp else None
        if fused is not None:
            return fused.row(ops.swiglu(fused.column(normed, self.linear_fc1.weight)), self.linear_fc2.weight)
        inp = tp.gather_from_sequence_parallel_region(normed) if self.sp else tp.copy_to_tensor_model_parallel_region(normed)
        act = ops.swiglu(ops.linear(inp, self.linear_fc1.weight))
        out = ops.linear(act, self.linear_fc2.weight)
        return tp.reduce_scatter_to_sequence_parallel_region(out) if self.sp else tp.reduce_from_tensor_model_parallel_region(out)


class TransformerLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_number: int, dtype, device, sequence_parallel: bool):
        super().__init__()
        self.layer_number = layer_number  # global, 0-based
        from slime_b200.models import mixers as _mixers

        if cfg.mixer(layer_number) == "attention" and _mixers._CUSTOM_BUILDER is None:
            self.self_attention = SelfAttention(cfg, layer_number, dtype, device, sequence_parallel)
        else:  # attention variants, linear attention, latent attention: models/mixers.py
            from slime_b200.models.mixers import build_mixer

            self.self_attention = build_mixer(cfg, layer_number, dtype, device, sequence_parallel)
        if cfg.is_moe_layer(layer_number):
            from slime_b200.models.moe import MoELayer

            self.mlp = MoELayer(cfg, layer_number, dtype, device, sequence_parallel)
        else:
            self.mlp = MLP(cfg, dtype, device, sequence_parallel)
        self.post_self_attn_layernorm = self.post_mlp_layernorm = None
        if cfg.post_self_attn_layernorm:
            self.post_self_attn_layernorm = nn.Module()
            self.post_self_attn_layernorm.weight = tp.set_tp_attrs(_param((cfg.hidden_size,), dtype, device, ones=True), False)
        if cfg.post_mlp_layernorm:
            self.post_mlp_layernorm = nn.Module()
            self.post_mlp_layernorm.weight = tp.set_tp_attrs(_param((cfg.hidden_size,), dtype, device, ones=True), False)
        self.eps = cfg.norm_epsilon

    def forward(self, x, residual, rope_table, packed):
        a, residual = self.self_attention(x, residual, rope_table, packed)
        if self.post_self_attn_layernorm is not None:
            a, _ = ops.rmsnorm(a, self.post_self_attn_layernorm.weight, self.eps)
        m, residual = self.mlp(a, residual)
        if self.post_mlp_layernorm is not None:
            m, _ = ops.rmsnorm(m, self.post_mlp_layernorm.weight, self.eps)
        return m, residual


class MTPLayer(nn.Module):
    """One multi-token-prediction depth (DeepSeek-V3 style draft head): the trunk's hidden state of position i and the
    embedding of token i+1 are normalised, concatenated, projected back to the model width and passed through one
    transformer layer; the shared output head then predicts token i+2. Parameters: ``enorm``, ``hnorm``, ``eh_proj``
    [H, 2H] (columns: embedding half, hidden half), ``transformer_layer.*``, ``final_layernorm``. Same role as the MTP
    block the reference enables with ``--mtp-num-layers`` / ``--enable-mtp-training``
    (slime/backends/megatron_utils/model_provider.py:200-232, docker/patch/latest/megatron.patch:556-640)."""

    def __init__(self, cfg: ModelConfig, layer_number: int, dtype, device, sequence_parallel: bool):
        super().__init__()
        h = cfg.hidden_size
        self.cfg, self.sp = cfg, sequence_parallel
        for n in ("enorm", "hnorm", "final_layernorm"):
            m = nn.Module()
            m.weight = tp.set_tp_attrs(_param((h,), dtype, device, ones=True), False)
            m.weight.sequence_parallel = sequence_parallel
            setattr(self, n, m)
        self.eh_proj = nn.Module()
        gen = tp.get_rng_tracker().states.get("default")
        self.eh_proj.weight = tp.set_tp_attrs(_param((h, 2 * h), dtype, device, cfg.init_method_std, generator=gen), False)
        self.eh_proj.weight.sequence_parallel = sequence_parallel  # fed this rank's rows only
        self.transformer_layer = TransformerLayer(cfg, layer_number, dtype, device, sequence_parallel)

    def forward(self, hidden, next_embedding, rope_table, packed):
        eps = self.cfg.norm_epsilon
        e, _ = ops.rmsnorm(next_embedding, self.enorm.weight, eps)
        hn, _ = ops.rmsnorm(hidden, self.hnorm.weight, eps)
        x = ops.linear(torch.cat([e, hn], dim=-1), self.eh_proj.weight)
        x, residual = self.transformer_layer(x, None, rope_table, packed)
        pre = x if residual is None else x + residual
        out, _ = ops.rmsnorm(pre, self.final_layernorm.weight, eps)
        return out, pre


class LinearForLastLayer(nn.Module):
    """Critic value head ``hidden -> 1`` (replicated across TP)."""

    def __init__(self, hidden, dtype, device):
        super().__init__()
        self.weight = tp.set_tp_attrs(_param((1, hidden), dtype, device, 0.02), False)
        self.bias = tp.set_tp_attrs(_param((1,), dtype, device, 0.0), False)

    def forward(self, x):
        return (x.float() @ self.weight.float().t() + self.bias.float()), None


def pipeline_layer_range(cfg: ModelConfig, pp_size: int, pp_rank: int, first: int | None = None, last: int | None = None,
                         vpp_size: int | None = None, vpp_rank: int = 0) -> range:
    """Global layer indices owned by a (virtual) pipeline stage. Uneven first/last stages supported."""
    L = cfg.num_layers
    if pp_size == 1:
        return range(0, L)
    counts = [0] * pp_size
    rest, stages = L, list(range(pp_size))
    if first is not None:
        counts[0] = first
        rest -= first
        stages.remove(0)
    if last is not None:
        counts[-1] = last
        rest -= last
        stages.remove(pp_size - 1)
    assert rest % len(stages) == 0, f"{rest} layers do not split over {len(stages)} middle stages"
    for s in stages:
        counts[s] = rest // len(stages)
    if vpp_size and vpp_size > 1:
        assert first is None and last is None and all(c % vpp_size == 0 for c in counts)
        per = counts[0] // vpp_size
        start = vpp_rank * (pp_size * per) + pp_rank * per
        return range(start, start + per)
    start = sum(counts[:pp_rank])
    return range(start, start + counts[pp_rank])


class GPTModel(nn.Module):
    def __init__(self, cfg: ModelConfig, *, dtype=torch.bfloat16, device="cpu", sequence_parallel=False,
                 pre_process=True, post_process=True, layer_range: range | None = None, value_head=False,
                 recompute_granularity: str | None = None, seed: int | None = None):  # fmt: skip
        super().__init__()
        self.cfg, self.dtype = cfg, dtype
        self.pre_process, self.post_process = pre_process, post_process
        self.sequence_parallel = sequence_parallel and mpu.get_tensor_model_parallel_world_size() > 1
        self.recompute = recompute_granularity == "full"
        if seed is not None:
            tp.model_parallel_seed(seed, device)
        tps, tpr = mpu.get_tensor_model_parallel_world_size(), mpu.get_tensor_model_parallel_rank()
        V = cfg.padded_vocab_size
        assert V % tps == 0, f"padded vocab {V} must divide by tp {tps}"
        self.vocab_per_rank = V // tps
        self.vocab_start = tpr * self.vocab_per_rank
        gen = tp.get_rng_tracker().states.get("tp")
        layer_range = layer_range if layer_range is not None else range(cfg.num_layers)
        self.layer_offset = layer_range.start

        if pre_process:
            self.embedding = nn.Module()
            self.embedding.word_embeddings = nn.Module()
            self.embedding.word_embeddings.weight = tp.set_tp_attrs(
                _param((self.vocab_per_rank, cfg.hidden_size), dtype, device, cfg.init_method_std, generator=gen), True, 0, 1
            )
        self.decoder = nn.Module()
        self.decoder.layers = nn.ModuleList(
            [TransformerLayer(cfg, i, dtype, device, self.sequence_parallel) for i in layer_range]
        )
        if post_process:
            self.decoder.final_layernorm = nn.Module()
            self.decoder.final_layernorm.weight = tp.set_tp_attrs(_param((cfg.hidden_size,), dtype, device, ones=True), False)
            self.decoder.final_layernorm.weight.sequence_parallel = self.sequence_parallel
            if value_head:
                self.output_layer = LinearForLastLayer(cfg.hidden_size, dtype, device)
            elif not cfg.tie_word_embeddings or not pre_process:
                self.output_layer = nn.Module()
                self.output_layer.weight = tp.set_tp_attrs(
                    _param((self.vocab_per_rank, cfg.hidden_size), dtype, device, cfg.init_method_std, generator=gen), True, 0, 1
                )
                # tied embeddings split across pipeline stages: the copies are kept equal by an
                # all-reduce of their grads over the embedding group
                self.output_layer.weight.shared_embedding = cfg.tie_word_embeddings
            else:
                self.output_layer = None
        self.value_head = value_head
        self.mtp = None
        if cfg.mtp_num_layers and post_process and not value_head:
            assert pre_process, "multi-token prediction shares the embedding table: it needs the first stage's weights (pp = 1)"
            self.mtp = nn.Module()
            self.mtp.layers = nn.ModuleList([MTPLayer(cfg, cfg.num_layers + k, dtype, device, self.sequence_parallel)
                                             for k in range(cfg.mtp_num_layers)])  # fmt: skip
        self.vision = None
        if cfg.vision is not None and pre_process:
            from slime_b200.models.vision import VisionConfig, VisionTower

            self.vision = VisionTower(VisionConfig.from_dict(cfg.vision), dtype, device)
        self.mtp_training = False  # set by the trainer (--enable-mtp-training): keep what the draft loss needs
        self._mtp_inputs = None
        self._rope = None
        self.input_tensor = None  # set by the pipeline schedule on non-first stages

    # ------------------------------------------------------------------ helpers
    def rope_table(self, device, need: int):
        if self._rope is None or self._rope.shape[0] < need or self._rope.device != torch.device(device):
            n = max(need, 4096)
            self._rope = ops.rope_table(self.cfg, n, self.cfg.head_dim, device)
        return self._rope

    def output_weight(self):
        if self.value_head:
            return None
        if self.output_layer is not None:
            return self.output_layer.weight
        return self.embedding.word_embeddings.weight

    def set_input_tensor(self, t):
        self.input_tensor = t

    # ------------------------------------------------------------------ forward
    def forward_hidden(self, input_ids, position_ids, packed: PackedSeqParams, vision_rows=None):
        """Runs this stage's layers; returns the final-normed hidden states on the last stage,
        else the ``(x, residual)`` pair stacked as ``[2, T, H]`` for the next stage. ``vision_rows``: (row indices,
        vectors) that replace the embeddings of the image / video placeholder tokens."""
        cfg = self.cfg
        if self.pre_process:
            x = ops.embedding(input_ids, self.embedding.word_embeddings.weight, self.vocab_start)
            if mpu.get_tensor_model_parallel_world_size() > 1:
                x = tp.reduce_from_tensor_model_parallel_region(x)
            if vision_rows is not None:
                x = x.index_put((vision_rows[0],), vision_rows[1].to(x.dtype))
                if len(vision_rows) > 2 and vision_rows[2] and (self.sequence_parallel or mpu.get_pipeline_model_parallel_world_size() > 1):
                    raise NotImplementedError("deepstack vision features with sequence or pipeline parallelism")
            if self.sequence_parallel:
                x = tp.scatter_to_sequence_parallel_region(x)
            residual = None
        else:
            x, residual = self.input_tensor[0], self.input_tensor[1]
        packed.position_ids = position_ids
        table = self.rope_table(x.device, int(packed.max_seqlen) + 1)
        deepstack = vision_rows[2] if vision_rows is not None and len(vision_rows) > 2 else []
        for li, layer in enumerate(self.decoder.layers):
            if self.recompute and torch.is_grad_enabled():
                x, residual = torch.utils.checkpoint.checkpoint(layer, x, residual, table, packed, use_reentrant=False)
            else:
                x, residual = layer(x, residual, table, packed)
            if li < len(deepstack):  # the stream is x + residual: adding to x adds to the stream
                x = x.index_add(0, vision_rows[0], deepstack[li].to(x.dtype))
        if not self.post_process:
            if residual is None:
                residual = torch.zeros_like(x)
            return torch.stack([x, residual])
        h, pre = ops.rmsnorm(x, self.decoder.final_layernorm.weight, cfg.norm_epsilon, residual)
        if self.mtp is not None and self.mtp_training and torch.is_grad_enabled():
            self._mtp_inputs = (pre if residual is not None else x, input_ids, packed, table)
        if self.sequence_parallel:
            h = tp.gather_from_sequence_parallel_region_no_reduce(h)
        return h

    def mtp_loss(self, full_loss_mask: torch.Tensor) -> torch.Tensor:
        """Draft-head loss of the micro-batch whose trunk forward just ran: mean over valid positions of the cross
        entropy of depth k predicting token i + k + 2 from position i, averaged over depths. ``full_loss_mask`` [T] is 1
        where position i predicts a trained token i + 1; a depth-k target is trained when it lies in the same sequence
        and its own predicting position is trained. Depth k + 1 consumes depth k's hidden state. (The reference's Megatron
        patch detaches the same three inputs: docker/patch/latest/megatron.patch:556-640.)"""
        from slime_b200.utils.ppo_utils import calculate_log_probs_and_entropy

        assert self._mtp_inputs is not None, "run the trunk forward with mtp_training set first"
        hidden, ids, packed, table = self._mtp_inputs
        self._mtp_inputs = None
        # the draft head is trained without touching the policy: it sees the trunk's hidden states, the embedding table
        # and the output head as constants, so only its own parameters receive gradients
        hidden = hidden.detach()
        ids = ids.reshape(-1)
        T = ids.numel()
        seq = torch.searchsorted(packed.cu_seqlens.long(), torch.arange(T, device=ids.device), right=True)
        mask = full_loss_mask.reshape(-1).float()
        w = self.output_weight().detach()
        total = hidden.new_zeros((), dtype=torch.float32)
        for k, layer in enumerate(self.mtp.layers):
            shift = k + 1
            nxt = torch.cat([ids[shift:], ids.new_zeros(shift)])  # token i + k + 1, the draft head's extra input
            emb = ops.embedding(nxt, self.embedding.word_embeddings.weight.detach(), self.vocab_start)
            if mpu.get_tensor_model_parallel_world_size() > 1:
                emb = tp.reduce_from_tensor_model_parallel_region(emb)
            if self.sequence_parallel:
                emb = tp.scatter_to_sequence_parallel_region(emb)
            out, hidden = layer(hidden, emb, table, packed)
            if self.sequence_parallel:
                out = tp.gather_from_sequence_parallel_region_no_reduce(out)
            logits = _lm_head(tp.copy_to_tensor_model_parallel_region(out), w)
            tgt = torch.cat([ids[shift + 1 :], ids.new_zeros(shift + 1)])  # token i + k + 2
            same = torch.cat([seq[shift + 1 :] == seq[: T - shift - 1], seq.new_zeros(shift + 1, dtype=torch.bool)])
            valid = torch.cat([mask[shift:], mask.new_zeros(shift)]) * same.float()
            lp, _ = calculate_log_probs_and_entropy(logits, tgt, mpu.get_tensor_model_parallel_group(), with_entropy=False)
            total = total - (lp.reshape(-1) * valid).sum() / valid.sum().clamp_min(1.0)
        return total / len(self.mtp.layers)

    def _vision_inputs(self, ids, packed, pixel_values, image_grid_thw, pixel_values_videos, video_grid_thw):
        """Encoder outputs for the placeholder rows and the three position streams of the packed stream (the reference
        does the same around a Transformers vision class: slime_plugins/models/qwen3_5_vl.py:150-200, :230-262)."""
        from slime_b200.models.vision import mrope_position_ids

        cfg = self.cfg
        if mpu.get_context_parallel_world_size() > 1:
            raise NotImplementedError("vision inputs with context parallelism: the placeholder rows of a rank's slices are not mapped yet")
        rows, vecs, deep = [], [], []
        for values, grids, tok in ((pixel_values, image_grid_thw, cfg.image_token_id), (pixel_values_videos, video_grid_thw, cfg.video_token_id)):
            if values is None:
                continue
            assert grids is not None and tok is not None and self.vision is not None, "pixel values need their grids, a placeholder id and an encoder"
            where = (ids == tok).nonzero(as_tuple=False).flatten()
            out, extras = self.vision(values.to(ids.device), grids, with_deepstack=True)
            if where.numel() != out.shape[0]:
                raise ValueError(f"{where.numel()} placeholder tokens for {out.shape[0]} encoder vectors")
            rows.append(where)
            vecs.append(out)
            deep.append(extras)
        if cfg.mrope_section:
            merge = (cfg.vision or {}).get("spatial_merge_size", 2)
            packed.mrope_positions, _ = mrope_position_ids(ids, packed.cu_seqlens, image_grid_thw, video_grid_thw, image_token_id=cfg.image_token_id,
                                                           video_token_id=cfg.video_token_id, spatial_merge_size=merge)  # fmt: skip
        if not rows:
            return None
        # per early layer, the extra vectors of all placeholder rows (images then videos, like the rows themselves)
        extras = [torch.cat([d[k] for d in deep]) for k in range(len(deep[0]))]
        return torch.cat(rows), torch.cat(vecs), extras

    def forward(self, input_ids, position_ids=None, attention_mask=None, labels=None, packed_seq_params=None,
                loss_mask=None, return_hidden=False, pixel_values=None, image_grid_thw=None, pixel_values_videos=None,
                video_grid_thw=None, **kw):  # fmt: skip
        """``input_ids``: [1, T] or [T]. Returns logits ``[1, T, V/tp]`` (fp32) on the last stage,
        values ``[1, T, 1]`` for a critic, or hidden states when ``return_hidden``. ``pixel_values`` / ``image_grid_thw``
        (and the video pair): image processor outputs for the placeholder tokens of the stream, in order."""
        ids = input_ids.reshape(-1)
        packed = packed_seq_params
        if packed is None:
            cu = torch.tensor([0, ids.numel()], dtype=torch.int32, device=ids.device)
            packed = PackedSeqParams(cu, ids.numel())
        if position_ids is None:
            position_ids = positions_from_cu_seqlens(packed.cu_seqlens, ids.numel())
        vision_rows = None
        packed.mrope_positions = None
        if pixel_values is not None or pixel_values_videos is not None:
            vision_rows = self._vision_inputs(ids, packed, pixel_values, image_grid_thw, pixel_values_videos, video_grid_thw)
            if not self.pre_process:
                vision_rows = None
        h = self.forward_hidden(ids, position_ids.reshape(-1).to(torch.int32), packed, vision_rows)
        if not self.post_process or return_hidden:
            return h
        if self.value_head:
            v, _ = self.output_layer(h)
            return v.unsqueeze(0)
        w = self.output_weight()
        inp = tp.copy_to_tensor_model_parallel_region(h)
        logits = ops.gemm(inp, w, out_dtype=torch.float32) if not torch.is_grad_enabled() else _lm_head(inp, w)
        return logits.unsqueeze(0)


class _LMHead(torch.autograd.Function):
    """fp32 logits = h W^T with bf16 operands (fp32 accumulate)."""

    @staticmethod
    def forward(ctx, h, w):
        ctx.save_for_backward(h, w)
        return ops.gemm(h, w, out_dtype=torch.float32)

    @staticmethod
    def backward(ctx, dlogits):
        h, w = ctx.saved_tensors
        d16 = dlogits.to(h.dtype)
        dh = ops.gemm(d16, w, b_mn=True)
        main_grad = getattr(w, "main_grad", None)
        if main_grad is not None:
            ops.gemm(d16, h, a_mn=True, b_mn=True, out=main_grad, accumulate=True)
            w.grad_added_to_main_grad = True
            return dh, None
        return dh, ops.gemm(d16, h, a_mn=True, b_mn=True, out_dtype=w.dtype)


def _lm_head(h, w):
    return _LMHead.apply(h, w)


def positions_from_cu_seqlens(cu_seqlens, total: int):
    """Position of every packed token inside its own sequence (tokens past the last sequence: 0...)."""
    cu = cu_seqlens.long()
    idx = torch.arange(total, device=cu.device)
    seq = torch.searchsorted(cu, idx, right=True) - 1
    seq = seq.clamp(0, cu.numel() - 2) if cu.numel() >= 2 else seq.clamp_min(0)
    return (idx - cu[seq]).to(torch.int32)


def named_parameters_with_layer_offset(model: GPTModel):
    """Yield ``(global_name, param)``: local layer indices are shifted by the stage's first layer."""
    for name, p in model.named_parameters():
        parts = name.split(".")
        if len(parts) > 2 and parts[0] == "decoder" and parts[1] == "layers":
            parts[2] = str(int(parts[2]) + model.layer_offset)
        yield ".".join(parts), p
