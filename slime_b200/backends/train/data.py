"""Micro-batch construction: varlen ("thd") packing with CP slicing and TP padding.

Parity: slime/backends/megatron_utils/data.py:14-149 (get_batch), :152-196
(DataIterator). Samples of a micro-batch are concatenated without per-sample
padding; the stream is padded once to a multiple of ``tp * data_pad_size_multiplier``
and the pad is described to attention as one more (ignored) sequence.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from slime_b200.backends.train.cp_utils import slice_with_cp
from slime_b200.models.gpt import PackedSeqParams
from slime_b200.parallel import state as mpu


class DataIterator:
    """Walks an explicit list of micro-batches (each a list of local sample indices)."""

    def __init__(self, rollout_data: dict, micro_batch_indices: list[list[int]]):
        self.rollout_data = rollout_data
        self.micro_batch_indices = micro_batch_indices
        self.offset = 0

    def get_next(self, keys):
        assert self.offset < len(self.micro_batch_indices), "data iterator exhausted"
        idx = self.micro_batch_indices[self.offset]
        self.offset += 1
        batch = {}
        for k in keys:
            v = self.rollout_data.get(k)
            batch[k] = None if v is None else [v[i] for i in idx]
        return batch

    def reset(self):
        self.offset = 0
        return self

    def __len__(self):
        return len(self.micro_batch_indices)


def get_data_iterator(args, model_chunks, rollout_data):
    """One iterator per virtual-pipeline chunk (all walk the same micro-batch list)."""
    n = len(model_chunks) if isinstance(model_chunks, (list, tuple)) else 1
    return [DataIterator(rollout_data, rollout_data["micro_batch_indices"]) for _ in range(n)]


def _get_batch_allgather_cp(batch, tokens_list, pad_multiplier, pad_token_id, device):
    """All-gather context parallelism: the samples are concatenated first, the stream is padded so that it divides into
    equal pieces that are multiples of ``tp * pad_multiplier``, and CP rank r takes the r-th contiguous piece. The
    cumulative lengths describe the whole stream; positions are the tokens' true in-sequence positions
    (slime/backends/megatron_utils/data.py:55-73,117-128 in the reference)."""
    cp, r = mpu.get_context_parallel_world_size(), mpu.get_context_parallel_rank()
    tp = mpu.get_tensor_model_parallel_world_size()
    cu = [0]
    for t in tokens_list:
        cu.append(cu[-1] + t.numel())
    tokens = torch.cat(tokens_list)
    positions = torch.cat([torch.arange(t.numel(), device=device, dtype=torch.int32) for t in tokens_list])
    mult = cp * tp * pad_multiplier
    pad = (-tokens.numel()) % mult
    if pad:
        tokens = F.pad(tokens, (0, pad), value=pad_token_id)
        positions = torch.cat([positions, torch.arange(pad, device=device, dtype=torch.int32)])
        cu.append(cu[-1] + pad)
    local = tokens.numel() // cp
    cu_t = torch.tensor(cu, dtype=torch.int32, device=device)
    max_len = max(b - a for a, b in zip(cu[:-1], cu[1:]))
    piece = slice(r * local, (r + 1) * local)
    batch["packed_seq_params"] = PackedSeqParams(cu_t, max_len, positions[piece])
    batch["packed_seq_params"].local_cu_seqlens = cu_t
    batch["tokens"] = tokens[piece].unsqueeze(0)
    batch["position_ids"] = positions[piece].unsqueeze(0)
    if batch.get("loss_masks") is not None:
        full = [F.pad(m.to(torch.float32), (tl - rl - 1, 1)) for m, tl, rl in zip(batch["loss_masks"], batch["total_lengths"], batch["response_lengths"])]
        fm = F.pad(torch.cat(full), (0, pad))
        batch["full_loss_masks"] = fm[piece].unsqueeze(0)
    return batch


def get_batch(data_iterator: DataIterator, keys, pad_multiplier: int = 128, pad_token_id: int = 0, device=None,
              allgather_cp: bool = False):
    """Build one packed micro-batch.

    Returns a dict with ``tokens`` [1, T_pad], ``position_ids`` [1, T_pad], ``packed_seq_params``,
    ``unconcat_tokens`` (per-sample full token tensors), ``full_loss_masks`` aligned to the packed
    stream, plus every requested key as a per-sample list.
    """
    assert "tokens" in keys
    batch = data_iterator.get_next(keys)
    tokens_list = batch["tokens"]
    device = device or tokens_list[0].device
    cp = mpu.get_context_parallel_world_size()
    tp = mpu.get_tensor_model_parallel_world_size()
    batch["unconcat_tokens"] = tokens_list
    if allgather_cp and cp > 1:
        if batch.get("multimodal_train_inputs") and any(batch["multimodal_train_inputs"]):
            raise NotImplementedError("vision inputs with context parallelism")
        return _get_batch_allgather_cp(batch, tokens_list, pad_multiplier, pad_token_id, device)

    pieces, pos_pieces, cu = [], [], [0]
    for t in tokens_list:
        local = slice_with_cp(t, pad_token_id)
        pieces.append(local)
        if cp == 1:
            pos_pieces.append(torch.arange(t.numel(), device=device, dtype=torch.int32))
        else:
            L = t.numel()
            cs = -(-L // (2 * cp))
            r = mpu.get_context_parallel_rank()
            pos_pieces.append(
                torch.cat([torch.arange(r * cs, (r + 1) * cs), torch.arange((2 * cp - r - 1) * cs, (2 * cp - r) * cs)])
                .to(device=device, dtype=torch.int32)
            )
        cu.append(cu[-1] + local.numel())
    tokens = torch.cat(pieces)
    positions = torch.cat(pos_pieces)
    mult = tp * pad_multiplier
    pad = (-tokens.numel()) % mult
    if pad:
        tokens = F.pad(tokens, (0, pad), value=pad_token_id)
        positions = torch.cat([positions, torch.arange(pad, device=device, dtype=torch.int32)])
        cu.append(cu[-1] + pad)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=device)
    max_len = max(b - a for a, b in zip(cu[:-1], cu[1:]))
    # attention sees global lengths: with zig-zag CP each local piece stands for cp x as many tokens
    batch["packed_seq_params"] = PackedSeqParams(cu_t * cp if cp > 1 else cu_t, max_len * cp, positions)
    batch["packed_seq_params"].local_cu_seqlens = cu_t
    batch["tokens"] = tokens.unsqueeze(0)
    batch["position_ids"] = positions.unsqueeze(0)

    mm = [d for d in (batch.get("multimodal_train_inputs") or []) if d]
    if mm:  # processor outputs of the samples that carry images, concatenated in stream order (model kwargs)
        batch["multimodal"] = {k: torch.cat([torch.as_tensor(d[k]) for d in mm if d.get(k) is not None]).to(device)
                               for k in sorted({k for d in mm for k in d}) if any(d.get(k) is not None for d in mm)}  # fmt: skip
    if batch.get("loss_masks") is not None:
        full = []
        for m, tl, rl in zip(batch["loss_masks"], batch["total_lengths"], batch["response_lengths"]):
            fm = F.pad(m.to(torch.float32), (tl - rl - 1, 1))  # aligned to the predicting position
            full.append(slice_with_cp(fm, 0.0))
        fm = torch.cat(full)
        if pad:
            fm = F.pad(fm, (0, pad))
        batch["full_loss_masks"] = fm.unsqueeze(0)
    return batch


def tensors_to_device(rollout_data: dict, device) -> dict:
    """Move the list-of-tensor fields of a rollout payload to ``device`` (non-blocking from pinned memory)."""
    out = {}
    for k, v in rollout_data.items():
        if isinstance(v, list) and v and torch.is_tensor(v[0]):
            out[k] = [t.to(device, non_blocking=True) for t in v]
        elif torch.is_tensor(v):
            out[k] = v.to(device, non_blocking=True)
        else:
            out[k] = v
    return out


def tensors_to_cpu(rollout_data: dict) -> dict:
    return tensors_to_device(rollout_data, "cpu")
