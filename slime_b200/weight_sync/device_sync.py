"""Device-side weight movement for the trainer -> engine sync.

``copy_tensors`` moves any number of (source, destination) tensor pairs of equal byte size in ONE kernel launch
(``sb_multi_copy``: a table of pointers and sizes, CTAs spread over the bytes), instead of one ``copy_`` launch per
parameter: a 36-layer dense model syncs ~400 tensors per step. Destinations may be peer-mapped memory of another GPU
on the same NVLink domain (plain stores), which is how shards reach an engine that lives on other GPUs.
CPU tensors fall back to ``copy_``.
"""

from __future__ import annotations

import torch


def copy_tensors(pairs) -> int:
    """Copy ``src -> dst`` for every pair (same dtype and number of elements, both contiguous). Returns bytes moved."""
    pairs = [(s, d) for s, d in pairs if s.numel() > 0]
    if not pairs:
        return 0
    total = 0
    if not pairs[0][0].is_cuda:
        for s, d in pairs:
            d.copy_(s.view_as(d))
            total += s.numel() * s.element_size()
        return total
    from slime_b200.ops import _lib

    n = len(pairs)
    table = torch.empty(3, n, dtype=torch.int64)
    for i, (s, d) in enumerate(pairs):
        assert s.is_contiguous() and d.is_contiguous() and s.dtype == d.dtype and s.numel() == d.numel(), "copy pairs must match"
        nbytes = s.numel() * s.element_size()
        table[0, i], table[1, i], table[2, i] = s.data_ptr(), d.data_ptr(), nbytes
        total += nbytes
    dev = pairs[0][0].device
    tdev = table.pin_memory().to(dev, non_blocking=True)
    fn = _lib.bind("sb_multi_copy", [_lib.c_void_p, _lib.c_void_p, _lib.c_void_p, _lib.c_int, _lib.c_long, _lib.c_int, _lib.c_void_p])
    _lib.check(fn(tdev[0].data_ptr(), tdev[1].data_ptr(), tdev[2].data_ptr(), n, total, _lib.sm_count(dev), _lib.stream()),
               "sb_multi_copy")
    # the table must outlive the launch: the caching allocator keeps the block bound to this stream until it is reused
    # by later work on the same stream, which is ordered after the kernel
    return total


def copy_tensors_2d(entries, device) -> int:
    """``entries``: (src_ptr, dst_ptr, rows, row_bytes, src_pitch, dst_pitch) integers (addresses may be peer-mapped
    memory of another GPU). One launch of ``sb_multi_copy_2d``. Returns the bytes moved."""
    from slime_b200.ops import _lib

    if not entries:
        return 0
    table = torch.tensor(entries, dtype=torch.int64)
    total = int((table[:, 2] * table[:, 3]).sum())
    tdev = table.pin_memory().to(device, non_blocking=True)
    fn = _lib.bind("sb_multi_copy_2d", [_lib.c_void_p, _lib.c_int, _lib.c_long, _lib.c_int, _lib.c_void_p])
    for s in range(0, len(entries), 4096):
        n = min(4096, len(entries) - s)
        _lib.check(fn(tdev[s].data_ptr(), n, total, _lib.sm_count(device), _lib.stream()), "sb_multi_copy_2d")
    return total


class GatherToEngine:
    """Weight sync from a tensor-parallel trainer into a rollout engine with a different sharding, on the device:
    gather of the TP shards, Megatron -> engine re-layout and the store into the engine's weight buffers are one
    kernel launch per sync (``sb_multi_copy_2d``), with no host work per parameter or per bucket.

    Every trainer rank copies its parameter shard (the flat bf16 buffer) into a symmetric staging buffer; after a
    bounded barrier each rank that hosts an engine reads, for every engine tensor, the row or column ranges it needs
    straight from the owning ranks' staging buffers (plain loads over NVLink for the peers') and writes them where the
    engine's layout wants them: fused QKV as [q heads | k heads | v heads] of the engine's own heads, gate / up halves,
    column ranges of the row-parallel matrices, row ranges of the vocabulary. The plan is a table of strided 2-D copies
    built once from the parameters' ``partition_dim`` / ``partition_stride`` attributes.

    Supported: dense models, trainer pipeline size 1, engine tensor-parallel size 1 (every GPU holds a whole engine) or
    equal to the trainer's (then ``UpdateWeightFromTensor._copy_fused`` is the cheaper path). Replaces the all-gather ->
    rename -> split -> load loop of the reference (slime/backends/megatron_utils/update_weight/update_weight_from_tensor.py:277-332).
    """

    def __init__(self, model, engine_weights, group):
        import torch.distributed as dist

        from slime_b200.parallel.fused_dp import SymmetricStorage
        from slime_b200.parallel.fused_tp import _SymmBarrier

        self.model, self.w, self.group = model, engine_weights, group
        self.device = model.device
        buf = model.dense_buffer
        self.buf = buf
        self.stage = SymmetricStorage(buf.numel, buf.param_data.dtype, self.device, group)
        self.world, self.rank = self.stage.world, self.stage.rank
        assert engine_weights.tp == 1, "GatherToEngine builds whole (TP1) engine tensors"
        self._barrier = _SymmBarrier(self.stage, 64, self.device)
        self._align = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.entries = self._plan()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)

    def _plan(self):
        cfg, w, n = self.model.cfg, self.w, self.world
        d, es = cfg.head_dim, self.buf.param_data.element_size()
        hq_l, hkv_l = cfg.num_attention_heads // n, cfg.num_query_groups // n
        Hq, Hkv = cfg.num_attention_heads, cfg.num_query_groups
        out = []

        def add(r, src_off_elems, dst_t, dst_off_elems, rows, row_elems, src_pitch_elems, dst_pitch_elems):
            out.append((self.stage.ptrs[r] + src_off_elems * es, dst_t.data_ptr() + dst_off_elems * es, rows, row_elems * es,
                        src_pitch_elems * es, dst_pitch_elems * es))  # fmt: skip

        def block(r, src_off, dst_t, dst_row0, rows, cols):  # a block of whole rows (the kernel splits it by rows)
            if (cols * es) % 16 == 0:
                add(r, src_off, dst_t, dst_row0 * cols, rows, cols, cols, cols)
            else:  # vectors: one short row
                add(r, src_off, dst_t, dst_row0 * cols, 1, rows * cols, rows * cols, rows * cols)

        for (name, p), (off, _e) in zip(zip(self.buf.names, self.buf.params), self.buf.offsets):
            sharded = getattr(p, "tensor_model_parallel", False)
            if name == "embedding.word_embeddings.weight" or name == "output_layer.weight":
                dst = w.embed if name.startswith("embedding") else w.lm_head
                if name == "output_layer.weight" and cfg.tie_word_embeddings:
                    continue
                rows, cols = p.shape
                for r in range(n):  # rows past the real vocabulary are padding of the trainer's sharding: not synced
                    valid = max(0, min(rows, cfg.vocab_size - r * rows))
                    if valid:
                        block(r, off, dst, r * rows, valid, cols)
                continue
            if name == "decoder.final_layernorm.weight":
                block(self.rank, off, w.final_norm, 0, 1, p.numel())
                continue
            _, _, i, sub = name.split(".", 3)
            L = w.layers[int(i)]
            H = cfg.hidden_size
            if sub == "self_attention.linear_qkv.weight":
                for r in range(n):
                    block(r, off, L["qkv"], r * hq_l * d, hq_l * d, H)
                    block(r, off + hq_l * d * H, L["qkv"], Hq * d + r * hkv_l * d, hkv_l * d, H)
                    block(r, off + (hq_l + hkv_l) * d * H, L["qkv"], (Hq + Hkv) * d + r * hkv_l * d, hkv_l * d, H)
            elif sub == "self_attention.linear_qkv.bias":
                for r in range(n):
                    block(r, off, L["qkv_bias"], r * hq_l * d, hq_l * d, 1)
                    block(r, off + hq_l * d, L["qkv_bias"], Hq * d + r * hkv_l * d, hkv_l * d, 1)
                    block(r, off + (hq_l + hkv_l) * d, L["qkv_bias"], (Hq + Hkv) * d + r * hkv_l * d, hkv_l * d, 1)
            elif sub == "mlp.linear_fc1.weight":
                f_l, F = p.shape[0] // 2, p.shape[0] // 2 * n
                for r in range(n):
                    block(r, off, L["gate_up"], r * f_l, f_l, H)
                    block(r, off + f_l * H, L["gate_up"], F + r * f_l, f_l, H)
            elif sub in ("self_attention.linear_proj.weight", "mlp.linear_fc2.weight"):
                dst = L["o"] if sub.startswith("self") else L["down"]
                rows, cols_l = p.shape
                for r in range(n):
                    add(r, off, dst, r * cols_l, rows, cols_l, cols_l, cols_l * n)
            else:
                key = {"self_attention.linear_qkv.layer_norm_weight": "ln1", "self_attention.q_layernorm.weight": "q_norm",
                       "self_attention.k_layernorm.weight": "k_norm", "mlp.linear_fc1.layer_norm_weight": "ln2"}.get(sub)  # fmt: skip
                assert key is not None and not sharded, f"no device-sync rule for {name}"
                block(self.rank, off, L[key], 0, 1, p.numel())
        return out

    @torch.no_grad()
    def sync(self) -> int:
        """Stage, meet, gather + re-layout + store, meet. Returns the bytes written into the engine's buffers."""
        import torch.distributed as dist

        self.stage.tensor.copy_(self.buf.param_data)
        dist.all_reduce(self._align, group=self.group)  # absorbs the skew between ranks; the bounded barrier only sees jitter
        self._barrier()
        moved = copy_tensors_2d(self.entries, self.device)
        self._barrier()  # nobody restages while a peer still reads
        return moved
