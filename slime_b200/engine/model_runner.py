"""Rollout-engine model execution: weight buffers, prefill (extend) and decode forward passes.

Weights live in fused per-layer buffers ([q|k|v] rows, [gate;up] rows) sharded for the engine's
own TP degree; ``load_weights`` accepts Hugging Face tensor names (``q_proj``, ``gate_proj``, ...)
and stacks them into the fused buffers, so the trainer->engine sync contract is "HF names on the
wire" exactly as with the reference's engines. The same sm_100a kernels as the trainer are used
(RMSNorm with fused residual, RoPE(+QK-norm), SwiGLU, tcgen05 GEMM), so train and rollout
log-probs agree by construction. Decode runs under CUDA graphs per batch-size bucket.
"""

from __future__ import annotations

import math
import re

import torch

from slime_b200 import ops
from slime_b200.engine.kv_cache import PagedKVCache
from slime_b200.models.config import ModelConfig

_LAYER_RE = re.compile(r"^model\.layers\.(\d+)\.(.+)$")


class EngineWeights:
    """Fused, TP-sharded weight buffers addressed by Hugging Face names."""

    def __init__(self, cfg: ModelConfig, dtype, device, tp_size=1, tp_rank=0):
        self.cfg, self.dtype, self.device, self.tp, self.rank = cfg, dtype, device, tp_size, tp_rank
        h, d = cfg.hidden_size, cfg.head_dim
        self.hq, self.hkv = cfg.num_attention_heads // tp_size, max(cfg.num_query_groups // tp_size, 1)
        self.f = cfg.ffn_hidden_size // tp_size
        self.vocab_local = cfg.padded_vocab_size // tp_size
        e = lambda *s: torch.zeros(*s, dtype=dtype, device=device)  # noqa: E731
        self.embed = e(self.vocab_local, h)
        self.lm_head = self.embed if cfg.tie_word_embeddings else e(self.vocab_local, h)
        self.final_norm = e(h)
        self.layers = []
        for i in range(cfg.num_layers):
            L = {
                "ln1": e(h), "qkv": e((self.hq + 2 * self.hkv) * d, h), "o": e(h, self.hq * d), "ln2": e(h),
                "qkv_bias": e((self.hq + 2 * self.hkv) * d) if cfg.add_qkv_bias else None,
                "q_norm": e(d) if cfg.qk_layernorm else None, "k_norm": e(d) if cfg.qk_layernorm else None,
            }  # fmt: skip
            if cfg.is_moe_layer(i):
                el = cfg.num_experts  # TODO(ep): shard experts over the engine's EP group
                fe = cfg.moe_ffn_hidden_size
                L.update(router=e(cfg.num_experts, h), w13=e(el, 2 * fe, h), w2=e(el, h, fe))
            else:
                L.update(gate_up=e(2 * self.f, h), down=e(h, self.f))
            self.layers.append(L)
        self.version = "default"

    def num_bytes(self) -> int:
        seen, total = set(), 0
        for t in self.tensors():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    def tensors(self):
        yield self.embed
        yield self.lm_head
        yield self.final_norm
        for L in self.layers:
            for v in L.values():
                if v is not None:
                    yield v

    # -- loading -----------------------------------------------------------------------
    def _rows(self, t, n_local):
        """This TP rank's slice of a tensor sharded on dim 0."""
        return t[self.rank * n_local : (self.rank + 1) * n_local]

    def load_weight(self, name: str, t: torch.Tensor):
        cfg, d = self.cfg, self.cfg.head_dim
        t = t.to(self.device, self.dtype, non_blocking=True)
        if name == "model.embed_tokens.weight":
            self.embed[: min(self.vocab_local, t.shape[0] - self.rank * self.vocab_local)].copy_(
                t[self.rank * self.vocab_local : (self.rank + 1) * self.vocab_local]
            )
            return True
        if name == "lm_head.weight":
            if not cfg.tie_word_embeddings:
                self.lm_head[: min(self.vocab_local, t.shape[0] - self.rank * self.vocab_local)].copy_(
                    t[self.rank * self.vocab_local : (self.rank + 1) * self.vocab_local]
                )
            return True
        if name == "model.norm.weight":
            self.final_norm.copy_(t)
            return True
        m = _LAYER_RE.match(name)
        if m is None:
            return False
        L = self.layers[int(m.group(1))]
        sub = m.group(2)
        hq, hkv = self.hq, self.hkv
        q_rows, kv_rows = hq * d, hkv * d
        table = {
            "input_layernorm.weight": lambda: L["ln1"].copy_(t),
            "post_attention_layernorm.weight": lambda: L["ln2"].copy_(t),
            "self_attn.q_proj.weight": lambda: L["qkv"][:q_rows].copy_(self._rows(t, q_rows)),
            "self_attn.k_proj.weight": lambda: L["qkv"][q_rows : q_rows + kv_rows].copy_(self._rows(t, kv_rows)),
            "self_attn.v_proj.weight": lambda: L["qkv"][q_rows + kv_rows :].copy_(self._rows(t, kv_rows)),
            "self_attn.qkv_proj.weight": lambda: L["qkv"].copy_(t),  # already fused + sharded for this rank
            "self_attn.q_proj.bias": lambda: L["qkv_bias"][:q_rows].copy_(self._rows(t, q_rows)),
            "self_attn.k_proj.bias": lambda: L["qkv_bias"][q_rows : q_rows + kv_rows].copy_(self._rows(t, kv_rows)),
            "self_attn.v_proj.bias": lambda: L["qkv_bias"][q_rows + kv_rows :].copy_(self._rows(t, kv_rows)),
            "self_attn.qkv_proj.bias": lambda: L["qkv_bias"].copy_(t),
            "self_attn.o_proj.weight": lambda: L["o"].copy_(t[:, self.rank * q_rows : (self.rank + 1) * q_rows]),
            "self_attn.q_norm.weight": lambda: L["q_norm"].copy_(t),
            "self_attn.k_norm.weight": lambda: L["k_norm"].copy_(t),
            "mlp.gate_proj.weight": lambda: L["gate_up"][: self.f].copy_(self._rows(t, self.f)),
            "mlp.up_proj.weight": lambda: L["gate_up"][self.f :].copy_(self._rows(t, self.f)),
            "mlp.gate_up_proj.weight": lambda: L["gate_up"].copy_(t),
            "mlp.down_proj.weight": lambda: L["down"].copy_(t[:, self.rank * self.f : (self.rank + 1) * self.f]),
            "mlp.gate.weight": lambda: L["router"].copy_(t),
        }
        if sub in table:
            table[sub]()
            return True
        em = re.match(r"^mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$", sub)
        if em:
            e, kind = int(em.group(1)), em.group(2)
            fe = cfg.moe_ffn_hidden_size
            if kind == "gate_proj":
                L["w13"][e, :fe].copy_(t)
            elif kind == "up_proj":
                L["w13"][e, fe:].copy_(t)
            else:
                L["w2"][e].copy_(t)
            return True
        return False

    def load_weights(self, named_tensors, version: str | None = None):
        missing = [n for n, t in named_tensors if not self.load_weight(n, t)]
        if version is not None:
            self.version = version
        return missing

    def init_random(self, seed: int = 0, std: float = 0.02):
        g = torch.Generator(device=self.device).manual_seed(seed)
        for t in self.tensors():
            if t.dim() == 1:
                t.fill_(1.0)
            else:
                t.copy_(torch.empty(t.shape, dtype=torch.float32, device=self.device).normal_(0, std, generator=g))
        for L in self.layers:
            if L.get("qkv_bias") is not None:
                L["qkv_bias"].zero_()


class ModelRunner:
    def __init__(self, cfg: ModelConfig, weights: EngineWeights, kv: PagedKVCache, max_batch: int, max_context: int,
                 use_cuda_graph: bool = True, tp_group=None):  # fmt: skip
        self.cfg, self.w, self.kv = cfg, weights, kv
        self.device = weights.device
        self.max_batch, self.max_context = max_batch, max_context
        self.max_pages_per_req = -(-max_context // kv.page_size)
        self.use_cuda_graph = use_cuda_graph and self.device.type == "cuda"
        self.tp_group = tp_group
        self.rope = ops.rope_cos_sin(max_context + 1, cfg.head_dim, cfg.rotary_base, device=self.device,
                                     scaling_factor=cfg.rotary_scaling_factor)  # fmt: skip
        self.scale = 1.0 / math.sqrt(cfg.head_dim)
        self.graphs: dict[int, tuple] = {}
        self.replayed_launches = 0  # kernel-library launches executed through graph replays
        self.graph_buckets = [b for b in (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512) if b <= max_batch]
        if max_batch not in self.graph_buckets:
            self.graph_buckets.append(max_batch)
        self._static = None

    # ------------------------------------------------------------------ layer math
    def _tp_reduce(self, x):
        if self.tp_group is not None:
            import torch.distributed as dist

            dist.all_reduce(x, group=self.tp_group)
        return x

    def _mlp(self, L, x):
        if "gate_up" in L:
            act = ops.swiglu(ops.gemm(x, L["gate_up"]))
            return self._tp_reduce(ops.gemm(act, L["down"]))
        return self._moe(L, x)

    def _moe(self, L, x):
        cfg = self.cfg
        logits = ops.router_gemm(x, L["router"])
        k = cfg.moe_router_topk
        topv, idx = torch.topk(logits, k, dim=-1)
        probs = torch.softmax(topv, -1) if cfg.norm_topk_prob else torch.softmax(logits, -1).gather(-1, idx)
        self._last_routed = idx
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        rows = x.index_select(0, order // k)
        counts = torch.bincount(flat, minlength=cfg.num_experts).tolist()
        outs, s = [], 0
        for e, n in enumerate(counts):
            if n:
                act = ops.swiglu(ops.gemm(rows[s : s + n], L["w13"][e]))
                outs.append(ops.gemm(act, L["w2"][e]))
                s += n
        y = torch.cat(outs) * probs.reshape(-1).index_select(0, order).to(x.dtype)[:, None]
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=order.device)
        return y.index_select(0, inv).view(x.shape[0], k, -1).float().sum(1).to(x.dtype)

    def _qkv(self, L, normed, positions):
        cfg = self.cfg
        qkv = ops.gemm(normed, L["qkv"], bias=L["qkv_bias"])
        return ops.rope_qk(qkv, positions, self.rope, self.w.hq, self.w.hkv, cfg.head_dim, L["q_norm"], L["k_norm"],
                           cfg.norm_epsilon)  # fmt: skip

    # --------------------------------------------------------------------- prefill
    @torch.no_grad()
    def prefill(self, ids, positions, slots, cu_q, kv_gather_slots, cu_k, max_q, max_k, last_rows, fresh: bool):
        """Extend pass over packed new tokens.

        ids/positions/slots: [T] for the new tokens; ``cu_q`` their per-request boundaries.
        ``kv_gather_slots``/``cu_k``: cache slots of every context token (cached prefix + new) per
        request, used when some context is already cached (``fresh`` False). Returns logits
        ``[len(last_rows), V/tp]`` fp32 for the requested rows and, when ``last_rows`` is None, all rows.
        """
        cfg, w, d = self.cfg, self.w, self.cfg.head_dim
        x = ops.embedding(ids, w.embed, w.rank * w.vocab_local)
        x = self._tp_reduce(x) if w.tp > 1 else x
        res = None
        T = ids.numel()
        for li, L in enumerate(w.layers):
            normed, res = ops.rmsnorm(x, L["ln1"], cfg.norm_epsilon, res)
            qkv = self._qkv(L, normed, positions)
            q3 = qkv.view(T, w.hq + 2 * w.hkv, d)
            q, k, v = q3[:, : w.hq], q3[:, w.hq : w.hq + w.hkv], q3[:, w.hq + w.hkv :]
            ops.kv_write(k.reshape(T, -1), v.reshape(T, -1), slots, self.kv.k[li], self.kv.v[li])
            if fresh:
                ctx = ops.varlen_attention(q, k, v, cu_q, max_q, self.scale)
            else:
                k_all = self.kv.k[li].index_select(0, kv_gather_slots)
                v_all = self.kv.v[li].index_select(0, kv_gather_slots)
                ctx = _extend_attention(q, k_all, v_all, cu_q, cu_k, max_q, max_k, self.scale)
            x = self._tp_reduce(ops.gemm(ctx.reshape(T, -1), L["o"]))
            normed, res = ops.rmsnorm(x, L["ln2"], cfg.norm_epsilon, res)
            x = self._mlp(L, normed)
        h, _ = ops.rmsnorm(x, w.final_norm, cfg.norm_epsilon, res)
        if last_rows is not None:
            h = h.index_select(0, last_rows)
        return ops.gemm(h, w.lm_head, out_dtype=torch.float32)

    # ---------------------------------------------------------------------- decode
    def _decode_body(self, ids, positions, block_table, seq_lens):
        cfg, w, d = self.cfg, self.w, self.cfg.head_dim
        ps = self.kv.page_size
        B = ids.numel()
        pos64 = positions.long()
        slots = (block_table.gather(1, (pos64 // ps)[:, None]).squeeze(1).long() * ps + pos64 % ps).to(torch.int32)
        x = ops.embedding(ids, w.embed, w.rank * w.vocab_local)
        x = self._tp_reduce(x) if w.tp > 1 else x
        res = None
        for li, L in enumerate(w.layers):
            normed, res = ops.rmsnorm(x, L["ln1"], cfg.norm_epsilon, res)
            qkv = self._qkv(L, normed, positions)
            q3 = qkv.view(B, w.hq + 2 * w.hkv, d)
            k, v = q3[:, w.hq : w.hq + w.hkv], q3[:, w.hq + w.hkv :]
            ops.kv_write(k.reshape(B, -1), v.reshape(B, -1), slots, self.kv.k[li], self.kv.v[li])
            ctx = ops.paged_decode_attention(q3[:, : w.hq], self.kv.k[li], self.kv.v[li], block_table, seq_lens, ps, self.scale)
            x = self._tp_reduce(ops.gemm(ctx.reshape(B, -1), L["o"]))
            normed, res = ops.rmsnorm(x, L["ln2"], cfg.norm_epsilon, res)
            x = self._mlp(L, normed)
        h, _ = ops.rmsnorm(x, w.final_norm, cfg.norm_epsilon, res)
        return ops.gemm(h, w.lm_head, out_dtype=torch.float32)

    def _alloc_static(self):
        """Decode inputs live in ONE flat int32 device buffer mirrored by a pinned host buffer, so a
        step uploads everything (ids, positions, lengths, sampling parameters, block table) with a
        single copy. Sections are contiguous arrays of ``max_batch`` entries; float / int64 fields
        are bit views of the same memory."""
        B, W, dev = self.max_batch, self.max_pages_per_req, self.device
        fields = ["ids", "positions", "seq_lens", "top_k", "out_pos", "temperature", "top_p", "min_p"]
        total = (len(fields) + 2) * B + B * W
        self._flat_dev = torch.zeros(total, dtype=torch.int32, device=dev)
        self._flat_host = torch.zeros(total, dtype=torch.int32, pin_memory=(dev.type == "cuda"))

        def views(flat):
            out, off = {}, 0
            for f in fields:
                v = flat[off : off + B]
                out[f] = v.view(torch.float32) if f in ("temperature", "top_p", "min_p") else v
                off += B
            out["seeds"] = flat[off : off + 2 * B].view(torch.int64)
            off += 2 * B
            out["block_table"] = flat[off : off + B * W].view(B, W)
            return out

        self._static = views(self._flat_dev)
        self.host = {k: v.numpy() for k, v in views(self._flat_host).items()}
        self.host["temperature"][:] = 1.0
        self.host["top_p"][:] = 1.0
        self.host["seq_lens"][:] = 1

    def upload_static(self):
        self._flat_dev.copy_(self._flat_host, non_blocking=True)

    @torch.no_grad()
    def decode(self, n: int, filtered: bool, kept_cap: int = 0):
        """One decode step for the first ``n`` rows of the static buffers (filled by the scheduler).
        Returns ``(tokens, logprobs, kept_ids, kept_count)`` device tensors of length >= n."""
        st = self._static
        if not self.use_cuda_graph or self.cfg.num_experts is not None:
            return self._decode_eager(n, filtered, kept_cap)
        bucket = next(b for b in self.graph_buckets if b >= n)
        key = (bucket, filtered, kept_cap)
        if key not in self.graphs:
            self._capture(bucket, filtered, kept_cap)
        graph, outs, n_kernels = self.graphs[key]
        self.replayed_launches += n_kernels
        graph.replay()
        return outs

    def _decode_eager(self, n, filtered, kept_cap):
        st = self._static
        logits = self._decode_body(st["ids"][:n], st["positions"][:n], st["block_table"][:n], st["seq_lens"][:n])
        return self._sample(logits, n, filtered, kept_cap)

    def _sample(self, logits, n, filtered, kept_cap):
        st = self._static
        return ops.sample(
            logits, st["temperature"][:n], st["top_k"][:n] if filtered else None, st["top_p"][:n] if filtered else None,
            st["min_p"][:n] if filtered else None, st["seeds"][:n], st["out_pos"][:n], kept_cap,
        )  # fmt: skip

    def _capture(self, bucket, filtered, kept_cap):
        st = self._static
        # warm up outside capture (lazy kernel attribute setup, allocator pools)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._decode_eager(bucket, filtered, kept_cap)
        torch.cuda.current_stream().wait_stream(side)
        from slime_b200.ops import _lib

        g = torch.cuda.CUDAGraph()
        before = _lib.launch_count()
        with torch.cuda.graph(g):
            outs = self._decode_eager(bucket, filtered, kept_cap)
        self.graphs[(bucket, filtered, kept_cap)] = (g, outs, _lib.launch_count() - before)

    def drop_graphs(self):
        """Memory tag ``cuda_graph``: captured graphs pin their private pools."""
        self.graphs.clear()


def _extend_attention(q, k_all, v_all, cu_q, cu_k, max_q, max_k, scale):
    """Attention of new tokens over (cached + new) context, causal aligned to the sequence end."""
    if q.is_cuda:
        from flash_attn import flash_attn_varlen_func

        return flash_attn_varlen_func(q, k_all, v_all, cu_q.to(torch.int32), cu_k.to(torch.int32), max_q, max_k,
                                      softmax_scale=scale, causal=True)  # fmt: skip
    out = torch.empty_like(q)
    cq, ck = cu_q.tolist(), cu_k.tolist()
    Hq, Hkv = q.shape[1], k_all.shape[1]
    for i in range(len(cq) - 1):
        qs = q[cq[i] : cq[i + 1]].float().transpose(0, 1)
        ks = k_all[ck[i] : ck[i + 1]].float().transpose(0, 1).repeat_interleave(Hq // Hkv, 0)
        vs = v_all[ck[i] : ck[i + 1]].float().transpose(0, 1).repeat_interleave(Hq // Hkv, 0)
        Lq, Lk = qs.shape[1], ks.shape[1]
        att = (qs @ ks.transpose(-1, -2)) * scale
        mask = torch.ones(Lq, Lk, dtype=torch.bool, device=q.device).tril(diagonal=Lk - Lq)
        out[cq[i] : cq[i + 1]] = (att.masked_fill(~mask, float("-inf")).softmax(-1) @ vs).transpose(0, 1).to(q.dtype)
    return out
