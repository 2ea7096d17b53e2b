"""Rollout-engine model execution: weight buffers, prefill (extend) and decode forward passes.

Weights live in fused per-layer buffers ([q|k|v] rows, [gate;up] rows) sharded for the engine's
own TP degree; ``load_weights`` accepts Hugging Face tensor names (``q_proj``, ``gate_proj``, ...)
and stacks them into the fused buffers, so the trainer->engine sync contract is "HF names on the
wire" exactly as with the reference's engines. The same sm_100a kernels as the trainer are used
(RMSNorm with fused residual, RoPE(+QK-norm), SwiGLU, tcgen05 GEMM), so train and rollout
log-probs agree by construction. Decode runs under CUDA graphs per batch-size bucket.
"""

from __future__ import annotations

import logging
import math
import re

import torch

from slime_b200 import ops
from slime_b200.engine.kv_cache import PagedKVCache
from slime_b200.models.config import ModelConfig

logger = logging.getLogger(__name__)

_LAYER_RE = re.compile(r"^model\.layers\.(\d+)\.(.+)$")
_MIMO_DRAFT_RE = re.compile(r"^model\.mtp_layers\.(\d+)\.(.+)$")


class EngineWeights:
    """Fused, TP-sharded weight buffers addressed by Hugging Face names."""

    def __init__(self, cfg: ModelConfig, dtype, device, tp_size=1, tp_rank=0, ep_size=1, quantization: str | None = None,
                 draft_layers: int = 0):
        """``draft_layers``: how many multi-token-prediction depths (checkpoint layers ``num_layers + k``) to keep for
        speculative decoding; 0 ignores them.
        ``quantization="fp8"`` keeps the projection matrices whose shapes allow it as block-scaled e4m3
        (``engine/quant.py``); embeddings, the LM head, routers, norms and biases stay in ``dtype``.
        ``ep_size`` is 1 (every rank holds all experts and computes all routes) or ``tp_size`` (rank r holds experts
        ``r*E/ep ... (r+1)*E/ep - 1`` at full width; the ranks' expert outputs are summed like any row-parallel
        projection). Same split as ``--sglang-ep-size`` with the all-reduce MoE path (scripts/models/qwen3-30B-A3B.sh and
        tests/test_qwen3_30B_A3B.py:98-120 in the reference run rollout engines with ep 8)."""
        self.cfg, self.dtype, self.device, self.tp, self.rank = cfg, dtype, device, tp_size, tp_rank
        if ep_size not in (1, tp_size):
            raise ValueError(f"engine expert parallelism must be 1 or the engine's size ({tp_size}), got {ep_size}")
        self.ep = ep_size
        if cfg.num_experts is not None and cfg.num_experts % ep_size:
            raise ValueError(f"{cfg.num_experts} experts do not divide over {ep_size} ranks")
        self.experts_local = None if cfg.num_experts is None else cfg.num_experts // ep_size
        self.first_expert = 0 if cfg.num_experts is None or ep_size == 1 else tp_rank * self.experts_local
        h, d = cfg.hidden_size, cfg.head_dim
        self.hq, self.hkv = cfg.num_attention_heads // tp_size, max(cfg.num_query_groups // tp_size, 1)
        self.f = cfg.ffn_hidden_size // tp_size
        self.vocab_local = cfg.padded_vocab_size // tp_size
        e = lambda *s: torch.zeros(*s, dtype=dtype, device=device)  # noqa: E731
        if quantization not in (None, "fp8"):
            raise ValueError(f"unknown engine quantization {quantization!r} (None or 'fp8')")
        self.quantization = quantization

        def mat(*shape, parts=()):
            """A projection matrix: fp8 when asked for and every separately loaded row range starts on a scale block."""
            from slime_b200.engine import quant

            if quantization == "fp8" and quant.supported(shape[-2], shape[-1], parts):
                return quant.Fp8Weight(*shape, device=device)
            return e(*shape)

        self.vision = None  # image encoder, replicated on every rank of the engine
        if cfg.vision is not None:
            from slime_b200.models.vision import VisionConfig, VisionTower

            self.vision = VisionTower(VisionConfig.from_dict(cfg.vision), dtype, device).requires_grad_(False)
        self.embed = e(self.vocab_local, h)
        self.lm_head = self.embed if cfg.tie_word_embeddings else e(self.vocab_local, h)
        self.final_norm = e(h)
        self.layers = []
        self.draft = []  # draft heads: an ordinary layer plus the two input norms, the joining projection and a final norm
        self.num_draft_layers = draft_layers
        for i in range(cfg.num_layers + draft_layers):
            kind = cfg.mixer(i)
            if kind not in ("attention", "general_attention", "gated_delta_net", "mla", "dsa"):
                raise NotImplementedError(f"the rollout engine has no layer of kind {kind!r} (layer {i})")
            full_norm = cfg.qk_layernorm_full  # one weight per projection (sharded like it) instead of one per head
            if kind == "gated_delta_net":
                # linear-attention layer: replicated over tensor-parallel ranks (every rank computes all of it)
                kd, vd = cfg.linear_num_key_heads * cfg.linear_key_head_dim, cfg.linear_num_value_heads * cfg.linear_value_head_dim
                hv = cfg.linear_num_value_heads
                f32 = lambda *sh: torch.zeros(*sh, dtype=torch.float32, device=device)  # noqa: E731
                L = {"kind": "gdn", "ln1": e(h), "ln2": e(h), "post_attn_ln": None, "post_mlp_ln": None,
                     "gdn_conv": e(2 * kd + vd, cfg.linear_conv_kernel_dim), "gdn_dt_bias": f32(hv), "gdn_A_log": f32(hv),
                     "gdn_norm": e(cfg.linear_value_head_dim), "gdn_out": e(h, vd)}  # fmt: skip
                if "qwen3next" in (cfg.model_arch or "").lower().replace("_", ""):
                    L.update(gdn_qkvz=e(2 * kd + 2 * vd, h), gdn_ba=e(2 * hv, h))
                else:
                    L.update(gdn_qkv=e(2 * kd + vd, h), gdn_z=e(vd, h), gdn_b=e(hv, h), gdn_a=e(hv, h))
            elif kind in ("mla", "dsa"):
                # latent attention: the compressions are replicated, the per-head expansions are sharded by head
                hq_l, dn, dr, dv = cfg.num_attention_heads // tp_size, cfg.qk_head_dim, cfg.qk_pos_emb_head_dim, cfg.v_head_dim
                L = {"kind": "mla", "ln1": e(h), "ln2": e(h), "post_attn_ln": None, "post_mlp_ln": None,
                     "kv_a": e(cfg.kv_lora_rank + dr, h), "kv_a_ln": e(cfg.kv_lora_rank), "kv_b": e(hq_l * (dn + dv), cfg.kv_lora_rank),
                     "o": e(h, hq_l * dv)}  # fmt: skip
                if cfg.q_lora_rank:
                    L.update(q_a=e(cfg.q_lora_rank, h), q_a_ln=e(cfg.q_lora_rank), q_b=e(hq_l * (dn + dr), cfg.q_lora_rank))
                else:
                    L["q_proj"] = e(hq_l * (dn + dr), h)
                if kind == "dsa":
                    # lightning indexer (replicated): which cached tokens a query may attend; a layer for which
                    # max(layer - offset, 0) % freq != 0 (1-based) reuses the choice of the nearest earlier computing layer
                    one_based = i + 1
                    src = one_based
                    while (max(src - cfg.index_skip_topk_offset, 0) % cfg.index_topk_freq) != 0:
                        src -= 1
                    L["index_source"] = src - 1
                    if src == one_based:
                        hi, di = cfg.index_n_heads, cfg.index_head_dim
                        L.update(idx_wq_b=e(hi * di, cfg.q_lora_rank), idx_wk=e(di, h), idx_k_norm_w=e(di), idx_k_norm_b=e(di),
                                 idx_weights=e(hi, h))  # fmt: skip
            else:
                L = self._attention_buffers(e, mat, h, d, full_norm)
            L.setdefault("kind", "attention")
            if cfg.is_moe_layer(i):
                el = self.experts_local
                fe = cfg.moe_ffn_hidden_size
                L.update(router=e(cfg.num_experts, h), w13=mat(el, 2 * fe, h, parts=(fe,)), w2=mat(el, h, fe))
                if cfg.moe_router_enable_expert_bias:
                    L["router_bias"] = torch.zeros(cfg.num_experts, dtype=torch.float32, device=device)
                if cfg.moe_shared_expert_intermediate_size:
                    fs = cfg.moe_shared_expert_intermediate_size // tp_size
                    L.update(shared_gate_up=mat(2 * fs, h, parts=(fs,)), shared_down=mat(h, fs))
                    if cfg.moe_shared_expert_gate:
                        L["shared_gate"] = e(1, h)
            else:
                L.update(gate_up=mat(2 * self.f, h, parts=(self.f,)), down=mat(h, self.f))
            if i >= cfg.num_layers:
                if L["kind"] == "gdn" or kind == "dsa":
                    raise NotImplementedError(f"a draft head with a {kind} mixer is not supported by the rollout engine")
                L.update(enorm=e(h), hnorm=e(h), eh_proj=e(h, 2 * h), final_ln=e(h))
                self.draft.append(L)
            else:
                self.layers.append(L)
        self.version = "default"

    def _attention_buffers(self, e, mat, h, d, full_norm):
        cfg = self.cfg
        L = {
            "ln1": e(h), "qkv": mat((self.hq + 2 * self.hkv) * d, h, parts=(self.hq * d, (self.hq + self.hkv) * d)),
            "o": mat(h, self.hq * d), "ln2": e(h),
            "qkv_bias": e((self.hq + 2 * self.hkv) * d) if cfg.add_qkv_bias else None,
            "q_norm": e(self.hq * d if full_norm else d) if (cfg.qk_layernorm or full_norm) else None,
            "k_norm": e(self.hkv * d if full_norm else d) if (cfg.qk_layernorm or full_norm) else None,
            "post_attn_ln": e(h) if cfg.post_self_attn_layernorm else None,
            "post_mlp_ln": e(h) if cfg.post_mlp_layernorm else None,
        }  # fmt: skip
        if cfg.attention_output_gate:
            L["gate"] = e(self.hq * d, h)  # sigmoid gate of the attention output, one row per query channel
        if cfg.softmax_sinks:
            L["sinks"] = torch.zeros(self.hq, dtype=torch.float32, device=self.device)  # per-head logit in the denominator
        return L

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
        if self.vision is not None:
            yield from self.vision.parameters()
        for L in self.layers + self.draft:
            for v in L.values():
                if v is None or isinstance(v, (str, int)):  # absent buffers, the layer's kind tag, the indexer's source layer
                    continue
                if hasattr(v, "tensors"):  # a quantised matrix: its bytes and its scales
                    yield from v.tensors()
                else:
                    yield v

    # -- loading -----------------------------------------------------------------------
    def _rows(self, t, n_local):
        """This TP rank's slice of a tensor sharded on dim 0."""
        return t[self.rank * n_local : (self.rank + 1) * n_local]

    def load_weight(self, name: str, t: torch.Tensor):
        cfg, d = self.cfg, self.cfg.head_dim
        if name.startswith("model.visual."):  # the image encoder keeps the checkpoint's parameter names
            if self.vision is None:
                return True
            target = dict(self.vision.named_parameters()).get(name[len("model.visual.") :])
            if target is None:
                return False
            target.data.copy_(t.to(self.device, target.dtype))
            return True
        if name.startswith("model.language_model."):  # checkpoints with a vision tower nest the language model
            name = "model." + name[len("model.language_model.") :]
        if name.endswith((".mlp.experts.gate_up_proj", ".mlp.experts.down_proj")):  # a layer's experts in one stacked tensor
            from slime_b200.weight_sync.convert import split_stacked_experts

            return all([self.load_weight(n, w) for n, w in split_stacked_experts(cfg, name, t)])
        if ".block_sparse_moe." in name:  # MiniMax-M2 spelling of the expert tensors
            from slime_b200.weight_sync.convert import family_name_to_generic

            name = family_name_to_generic(name)
        raw = t
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
        from slime_b200.weight_sync import convert

        plus1 = 1.0 if convert._zero_centred(cfg) else 0.0  # Qwen3-Next / Qwen3.5 store their RMSNorm weights minus one
        if name == "model.norm.weight":
            self.final_norm.copy_(t + plus1)
            return True
        if name.startswith("mtp."):
            return True  # Qwen3-Next / Qwen3.5 draft block: their recurrent trunks are not speculated on, the block is not kept
        mimo = _MIMO_DRAFT_RE.match(name)
        if mimo is not None:
            # MiMo stores its draft head outside the layer list, the joining projection's halves as (hidden, embedding)
            depth, sub = int(mimo.group(1)), mimo.group(2)
            if depth >= len(self.draft):
                return True
            if sub == "input_proj.weight":
                h_half, e_half = t.chunk(2, dim=1)
                self.draft[depth]["eh_proj"].copy_(torch.cat([e_half, h_half], dim=1))
                return True
            own = {"token_layernorm.weight": "enorm.weight", "hidden_layernorm.weight": "hnorm.weight",
                   "final_layernorm.weight": "shared_head.norm.weight"}  # fmt: skip
            return self.load_weight(f"model.layers.{len(self.layers) + depth}.{own.get(sub, sub)}", raw)
        m = _LAYER_RE.match(name)
        if m is None:
            return False
        sub = m.group(2)
        if int(m.group(1)) >= len(self.layers):
            # a draft (multi-token-prediction) depth stored as an extra layer (DeepSeek-V3 layout): kept only when the
            # engine speculates; its copies of the embedding and the output head are the trunk's
            depth = int(m.group(1)) - len(self.layers)
            if depth >= len(self.draft) or sub in ("embed_tokens.weight", "shared_head.head.weight"):
                return True
            L = self.draft[depth]
            own = {"enorm.weight": "enorm", "hnorm.weight": "hnorm", "eh_proj.weight": "eh_proj", "shared_head.norm.weight": "final_ln"}
            if sub in own:
                L[own[sub]].copy_(t)
                return True
        else:
            L = self.layers[int(m.group(1))]
        hq, hkv = self.hq, self.hkv
        q_rows, kv_rows = hq * d, hkv * d
        if sub.startswith("linear_attn."):
            if L["kind"] != "gdn":
                return False
            inner = sub[len("linear_attn.") :]
            table = {"in_proj_qkvz.weight": "gdn_qkvz", "in_proj_ba.weight": "gdn_ba", "in_proj_qkv.weight": "gdn_qkv",
                     "in_proj_z.weight": "gdn_z", "in_proj_b.weight": "gdn_b", "in_proj_a.weight": "gdn_a", "conv1d.weight": "gdn_conv",
                     "dt_bias": "gdn_dt_bias", "A_log": "gdn_A_log", "norm.weight": "gdn_norm", "out_proj.weight": "gdn_out"}  # fmt: skip
            key = table.get(inner)
            if key is None or key not in L:
                return False
            src = raw.to(self.device, L[key].dtype)
            L[key].copy_(src.squeeze(1) if inner == "conv1d.weight" and src.dim() == 3 else src)
            return True
        if L["kind"] == "mla" and sub.startswith("self_attn."):
            inner = sub[len("self_attn.") :]
            hq_l, dn, dr, dv = cfg.num_attention_heads // self.tp, cfg.qk_head_dim, cfg.qk_pos_emb_head_dim, cfg.v_head_dim
            whole = {"q_a_proj.weight": "q_a", "q_a_layernorm.weight": "q_a_ln", "kv_a_proj_with_mqa.weight": "kv_a",
                     "kv_a_layernorm.weight": "kv_a_ln"}  # fmt: skip
            by_head = {"q_b_proj.weight": ("q_b", dn + dr), "q_proj.weight": ("q_proj", dn + dr), "kv_b_proj.weight": ("kv_b", dn + dv)}
            if inner in whole and whole[inner] in L:
                L[whole[inner]].copy_(t)
                return True
            if inner in by_head and by_head[inner][0] in L:
                key, per = by_head[inner]
                L[key].copy_(self._rows(t, hq_l * per))
                return True
            if inner == "o_proj.weight":
                L["o"].copy_(t[:, self.rank * hq_l * dv : (self.rank + 1) * hq_l * dv])
                return True
            indexer = {"indexer.wq_b.weight": "idx_wq_b", "indexer.wk.weight": "idx_wk", "indexer.k_norm.weight": "idx_k_norm_w",
                       "indexer.k_norm.bias": "idx_k_norm_b", "indexer.weights_proj.weight": "idx_weights"}  # fmt: skip
            if inner in indexer and indexer[inner] in L:
                L[indexer[inner]].copy_(t)
                return True
            return False
        if sub == "self_attn.q_proj.weight" and cfg.attention_output_gate and L["kind"] == "attention":
            # checkpoint rows are per head (query, gate): split them into the fused projection's q rows and the gate matrix
            x = t.view(cfg.num_attention_heads, 2 * d, -1)
            q_full, g_full = x[:, :d].reshape(-1, x.shape[-1]), x[:, d:].reshape(-1, x.shape[-1])
            L["qkv"][: hq * d].copy_(self._rows(q_full, hq * d))
            L["gate"].copy_(self._rows(g_full, hq * d))
            return True
        vectors = {
            "input_layernorm.weight": lambda: L["ln1"].copy_(t + plus1),
            "post_attention_layernorm.weight": lambda: L["ln2"].copy_(t + plus1),
            "self_attn.q_proj.bias": lambda: L["qkv_bias"][:q_rows].copy_(self._rows(t, q_rows)),
            "self_attn.k_proj.bias": lambda: L["qkv_bias"][q_rows : q_rows + kv_rows].copy_(self._rows(t, kv_rows)),
            "self_attn.v_proj.bias": lambda: L["qkv_bias"][q_rows + kv_rows :].copy_(self._rows(t, kv_rows)),
            "self_attn.qkv_proj.bias": lambda: L["qkv_bias"].copy_(t),
            "self_attn.q_norm.weight": lambda: L["q_norm"].copy_((self._rows(t, q_rows) if cfg.qk_layernorm_full else t) + plus1),
            "self_attn.k_norm.weight": lambda: L["k_norm"].copy_((self._rows(t, kv_rows) if cfg.qk_layernorm_full else t) + plus1),
            "mlp.gate.weight": lambda: L["router"].copy_(t),
            "post_self_attn_layernorm.weight": lambda: L["post_attn_ln"].copy_(t),
            "post_mlp_layernorm.weight": lambda: L["post_mlp_ln"].copy_(t),
            "mlp.gate.e_score_correction_bias": lambda: L["router_bias"].copy_(raw.to(self.device, torch.float32)),
            "mlp.shared_expert_gate.weight": lambda: L["shared_gate"].copy_(t),
            "self_attn.sinks": lambda: L["sinks"].copy_(self._rows(raw.to(self.device, torch.float32), hq)),
        }
        if sub in vectors and sub.split(".")[0] in ("post_self_attn_layernorm", "post_mlp_layernorm") and L.get(
                "post_attn_ln" if sub.startswith("post_self") else "post_mlp_ln") is None:
            return False
        if sub in vectors:
            vectors[sub]()
            return True
        # matrices: (buffer, first row in the buffer, rows there, how the incoming tensor is cut for this rank:
        # 0 = by rows, 1 = by columns, None = already this rank's)
        f = self.f
        matrices = {
            "self_attn.q_proj": ("qkv", 0, q_rows, 0), "self_attn.k_proj": ("qkv", q_rows, kv_rows, 0),
            "self_attn.v_proj": ("qkv", q_rows + kv_rows, kv_rows, 0), "self_attn.qkv_proj": ("qkv", 0, q_rows + 2 * kv_rows, None),
            "self_attn.o_proj": ("o", 0, cfg.hidden_size, 1), "mlp.gate_proj": ("gate_up", 0, f, 0),
            "mlp.up_proj": ("gate_up", f, f, 0), "mlp.gate_up_proj": ("gate_up", 0, 2 * f, None),
            "mlp.down_proj": ("down", 0, cfg.hidden_size, 1),
        }  # fmt: skip
        if cfg.moe_shared_expert_intermediate_size:
            fs = cfg.moe_shared_expert_intermediate_size // self.tp
            for prefix in ("mlp.shared_experts", "mlp.shared_expert"):
                matrices.update({f"{prefix}.gate_proj": ("shared_gate_up", 0, fs, 0), f"{prefix}.up_proj": ("shared_gate_up", fs, fs, 0),
                                 f"{prefix}.down_proj": ("shared_down", 0, cfg.hidden_size, 1)})  # fmt: skip
        stem, _, kind = sub.rpartition(".")
        buf = None
        if stem in matrices and kind in ("weight", "weight_scale_inv"):
            key, r0, rows, cut = matrices[stem]
            if key not in L:
                return False
            buf = L[key]
        else:
            em = re.match(r"^mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)$", stem)
            if em is None or kind not in ("weight", "weight_scale_inv") or "w13" not in L:
                return False
            e, which = int(em.group(1)) - self.first_expert, em.group(2)
            if not 0 <= e < self.experts_local:
                return True  # another rank's expert
            fe = cfg.moe_ffn_hidden_size
            buf = L["w13"][e] if which != "down_proj" else L["w2"][e]
            r0, rows, cut = (fe if which == "up_proj" else 0), (cfg.hidden_size if which == "down_proj" else fe), None
        self._put(buf, r0, rows, cut, t, raw, scale=kind == "weight_scale_inv")
        return True

    def _put(self, buf, r0: int, rows: int, cut, t, raw, scale: bool):
        """Write this rank's part of an incoming matrix (or of its block scales) into rows ``[r0, r0 + rows)`` of ``buf``."""
        from slime_b200.engine.quant import BLOCK, Fp8Weight

        fp8_in = raw.dtype == torch.float8_e4m3fn
        src = raw.to(self.device, non_blocking=True) if (scale or fp8_in) else t
        unit = BLOCK if scale else 1  # scale tensors count in blocks of 128 rows / columns
        if cut == 0:
            n = -(-rows // unit)
            src = src[self.rank * n : (self.rank + 1) * n]
        elif cut == 1:
            cols = buf.shape[-1] // unit
            src = src[:, self.rank * cols : (self.rank + 1) * cols]
        if isinstance(buf, Fp8Weight):
            if scale:
                buf.load_scale_rows(r0, src)
            else:
                buf.load_rows(r0, src)
            return
        if scale or fp8_in:
            raise ValueError("block-fp8 weights were sent to an engine that keeps this matrix in bf16; start it with "
                             "quantization='fp8' (and shapes that are multiples of 128) or send bf16 weights")
        buf[r0 : r0 + src.shape[0]].copy_(src)

    def load_weights(self, named_tensors, version: str | None = None):
        missing = [n for n, t in named_tensors if not self.load_weight(n, t)]
        if version is not None:
            self.version = version
        return missing

    def init_random(self, seed: int = 0, std: float = 0.02):
        from slime_b200.engine.quant import Fp8Weight

        g = torch.Generator(device=self.device).manual_seed(seed)
        quantised = [v for L in self.layers + self.draft for v in L.values() if isinstance(v, Fp8Weight)]
        for L in self.layers:  # the decay parameter of delta-net layers must start in its valid range
            if "gdn_A_log" in L:
                L["gdn_A_log"].copy_(torch.empty_like(L["gdn_A_log"]).uniform_(1e-3, 16.0, generator=g).log())
        skip = {t.data_ptr() for v in quantised for t in v.tensors()}
        for t in self.tensors():
            if t.data_ptr() in skip:
                continue
            if t.dim() == 1:
                t.fill_(1.0)
            else:
                t.copy_(torch.empty(t.shape, dtype=torch.float32, device=self.device).normal_(0, std, generator=g))
        for v in quantised:
            v.fill_random_(std, g)
        for L in self.layers + self.draft:
            if L.get("qkv_bias") is not None:
                L["qkv_bias"].zero_()


def _linear(x, w, bias=None, out_dtype=None, out=None):
    """``x @ w^T`` for a bf16 matrix (tcgen05 bf16 GEMM) or a block-fp8 one (activation quantised here, fp8 GEMM)."""
    if isinstance(w, torch.Tensor):
        return ops.gemm(x, w, bias=bias, out_dtype=out_dtype, out=out)
    from slime_b200.engine import quant

    return quant.linear(x, w, bias=bias, out_dtype=out_dtype, out=out)


def _grouped_linear(x, w, lay):
    from slime_b200.ops import grouped

    if isinstance(w, torch.Tensor):
        return grouped.grouped_gemm(x, w, lay)
    return grouped.grouped_gemm_fp8(x, w.q, w.scale, lay, out_dtype=x.dtype)


class ModelRunner:
    def __init__(self, cfg: ModelConfig, weights: EngineWeights, kv: PagedKVCache, max_batch: int, max_context: int,
                 use_cuda_graph: bool = True, tp_group=None):  # fmt: skip
        self.cfg, self.w, self.kv = cfg, weights, kv
        self.device = weights.device
        self.max_batch, self.max_context = max_batch, max_context
        self.max_pages_per_req = -(-max_context // kv.page_size)
        # head dims other than 64 / 128 fall back to attention written with plain ops, which reads lengths on the host
        self.use_cuda_graph = (use_cuda_graph and self.device.type == "cuda" and cfg.head_dim in (64, 128)
                               and not cfg.multi_latent_attention and not cfg.softmax_sinks)  # fmt: skip
        self.tp_group = tp_group
        # Row-parallel projections (attention output, MLP down) leave their result in fp32 when no cross-rank sum
        # follows: the fused add+RMSNorm reads it unrounded, and a skinny decode GEMM with a long K can then be cut
        # into K slices that the epilogue sums with TMA reduce-add.
        self._proj_dtype = torch.float32 if (self.device.type == "cuda" and weights.tp == 1 and not ops.library_mode()) else None
        # Tensor-parallel decode: all-reduce + residual add + RMSNorm as one peer-memory kernel when the ranks share an
        # NVLink domain; otherwise NCCL all-reduce followed by the fused add+norm.
        self._fused_tp = None
        if tp_group is not None and weights.tp > 1 and self.device.type == "cuda":
            from slime_b200.parallel import fused_tp

            if fused_tp.usable(weights.tp, self.device, cfg.hidden_size):
                try:
                    self._fused_tp = fused_tp.FusedAllReduceNorm(tp_group, max_batch, cfg.hidden_size, self.device)
                except Exception as e:  # noqa: BLE001
                    logger.warning("fused tensor-parallel all-reduce unavailable (%r): using NCCL", e)
        # KV slabs exist for the attention layers only; gated delta-net layers keep a recurrent state per decode slot
        self.kv_of, n_attn = [], 0
        for L in weights.layers + weights.draft:  # a draft head's layer number is num_layers + depth
            self.kv_of.append(n_attn if L["kind"] in ("attention", "mla") else None)
            n_attn += L["kind"] in ("attention", "mla")
        self.has_mla = any(L["kind"] == "mla" for L in weights.layers)
        self._dsa_masks: dict[int, torch.Tensor] = {}  # key choices of the indexer layers of the pass in flight
        self.has_gdn = any(L["kind"] == "gdn" for L in weights.layers)
        self.gdn_S, self.gdn_conv, self.last_gdn_states = {}, {}, None
        if self.has_gdn:
            hv, dk, dv = cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
            C, K = 2 * cfg.linear_num_key_heads * dk + hv * dv, cfg.linear_conv_kernel_dim
            for li, L in enumerate(weights.layers):
                if L["kind"] == "gdn":
                    self.gdn_S[li] = torch.zeros(max_batch, hv, dk, dv, dtype=torch.float32, device=self.device)
                    self.gdn_conv[li] = torch.zeros(max_batch, K - 1, C, dtype=weights.dtype, device=self.device)
        self._composed_attention = cfg.rotary_percent < 1.0 or cfg.rotary_interleaved or cfg.qk_layernorm_full or bool(cfg.mrope_section)
        # vision inputs: decode positions are the token index plus a per-request offset (an image advances the position
        # by its larger grid side only), prefill positions are three streams
        self.rope_delta = torch.zeros(max_batch, dtype=torch.int32, device=self.device) if cfg.mrope_section else None
        self._mrope_axes = None
        rot = int(cfg.head_dim * cfg.rotary_percent) // 2 * 2
        self.rope = ops.rope_table(cfg, max_context + 1, rot, self.device)
        self.scale = 1.0 / math.sqrt(cfg.head_dim)
        if cfg.multi_latent_attention:
            from slime_b200.models import mixers

            self.rope = mixers.mla_rope_table(cfg, max_context + 1, self.device)
            self.scale = mixers.mla_softmax_scale(cfg)
        self.graphs: dict[int, tuple] = {}
        self.replayed_launches = 0  # kernel-library launches executed through graph replays
        self.graph_buckets = [b for b in (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512) if b <= max_batch]
        if max_batch not in self.graph_buckets:
            self.graph_buckets.append(max_batch)
        self._static = None
        # expert choices of the tokens of the current forward pass, one [T, k] tensor per MoE layer (routing replay)
        self.record_routed = False
        self._moe_layer_idx = torch.tensor([i for i in range(cfg.num_layers) if cfg.is_moe_layer(i)], dtype=torch.long,
                                           device=self.device)  # fmt: skip
        self._routed: list[torch.Tensor] = []
        self.last_routed = None
        self.last_hidden = None  # residual stream before the final norm of the last prefill pass, all rows (draft heads read it)

    def take_routed(self):
        """``[T, layers, k]`` int32 expert ids of the pass just run, one column per layer of the model (zeros for dense
        layers: the consumer indexes by layer number); None when not recording."""
        if not self._routed:
            return None
        picked = torch.stack(self._routed, 1)
        self._routed = []
        if self._moe_layer_idx.numel() == self.cfg.num_layers:
            return picked
        out = picked.new_zeros(picked.shape[0], self.cfg.num_layers, picked.shape[2])
        return out.index_copy_(1, self._moe_layer_idx, picked)  # the index lives on the device: capturable

    # ------------------------------------------------------------------ layer math
    def _tp_reduce(self, x):
        if self.tp_group is not None:
            import torch.distributed as dist

            dist.all_reduce(x, group=self.tp_group)
        return x

    def _gather_logits(self, logits):
        """Vocab-parallel LM head: [T, V/tp] per rank -> [T, V] on every rank (rank r owns columns r*V/tp ...)."""
        V = self.cfg.vocab_size  # columns past it are padding of the vocabulary sharding: never sampled, never scored
        if self.tp_group is None or self.w.tp == 1:
            return logits if logits.shape[1] == V else logits[:, :V]
        import torch.distributed as dist

        T, vl = logits.shape
        parts = torch.empty(self.w.tp * T, vl, dtype=logits.dtype, device=logits.device)  # rank-major concatenation
        dist.all_gather_into_tensor(parts, logits.contiguous(), group=self.tp_group)
        full = parts.view(self.w.tp, T, vl).permute(1, 0, 2).reshape(T, -1)
        return full if full.shape[1] == V else full[:, :V]

    def _row_parallel_norm(self, inp, weight, ln, res, T: int, post=None):
        """``rmsnorm(sum over TP ranks of inp @ weight^T + res)`` -> (normed, new residual); ``post``: a sandwich norm
        applied to the projected sum before it joins the residual stream."""
        if post is not None:
            x = self._post_norm(self._tp_reduce(_linear(inp, weight)), post)
            return ops.rmsnorm(x, ln, self.cfg.norm_epsilon, res)
        if self._fused_tp is not None and T <= self._fused_tp.max_tokens:
            _linear(inp, weight, out=self._fused_tp.partial(T))
            return self._fused_tp(T, res, ln, self.cfg.norm_epsilon)
        x = self._tp_reduce(_linear(inp, weight, out_dtype=self._proj_dtype))
        return ops.rmsnorm(x, ln, self.cfg.norm_epsilon, res)

    def _mlp(self, L, x):
        if "gate_up" in L:
            act = ops.swiglu(_linear(x, L["gate_up"]))
            return self._tp_reduce(_linear(act, L["down"], out_dtype=self._proj_dtype))
        return self._moe(L, x)

    def _route(self, L, logits):
        """Expert choice and weights of every token, as the trainer's router computes them."""
        cfg = self.cfg
        from slime_b200.ops import grouped

        if cfg.moe_router_num_groups and cfg.moe_router_group_topk and cfg.moe_router_num_groups > 1:
            # group-limited routing (sigmoid scores): no kernel for it; a handful of small device ops, capturable
            from slime_b200.models.moe import group_limited

            scores = torch.sigmoid(logits.float())
            sel = scores + L["router_bias"] if L.get("router_bias") is not None else scores
            idx = torch.topk(group_limited(sel, cfg.moe_router_num_groups, cfg.moe_router_group_topk), cfg.moe_router_topk, dim=-1).indices
            probs = scores.gather(-1, idx)
            if cfg.norm_topk_prob:
                probs = probs / (probs.sum(-1, keepdim=True) + 1e-20)
            return probs * (cfg.moe_router_topk_scaling_factor or 1.0), idx
        return grouped.route_topk(logits, cfg.moe_router_topk, score=cfg.moe_router_score_function,
                                  pre_softmax=cfg.moe_router_pre_softmax, renorm=cfg.norm_topk_prob,
                                  bias=L.get("router_bias"), scale=cfg.moe_router_topk_scaling_factor)  # fmt: skip

    def _moe(self, L, x):
        from slime_b200.ops import grouped

        probs, idx = self._route(L, ops.router_gemm(x, L["router"]))
        if self.record_routed:
            self._routed.append(idx.to(torch.int32))
        # expert-sorted, tile-padded layout built on the device (no host sync: the step stays graph-capturable), then
        # one grouped GEMM per projection over all experts

        lay = grouped.DeviceLayout(idx, L["w13"].shape[0], self.w.first_expert)
        y = lay.combine(_grouped_linear(ops.swiglu(_grouped_linear(lay.pad(x), L["w13"], lay)), L["w2"], lay), probs, x.shape[0])
        shared = None
        if "shared_gate_up" in L:  # always-on expert, tensor-parallel like a dense MLP
            shared = _linear(ops.swiglu(_linear(x, L["shared_gate_up"])), L["shared_down"])
            if L.get("shared_gate") is not None:
                shared = shared * torch.sigmoid(x.float() @ L["shared_gate"].float().t()).to(shared.dtype)
        if self.w.ep > 1:  # expert outputs and the shared expert's partial sums travel in one reduction
            return self._tp_reduce(y if shared is None else y + shared)
        if shared is not None:
            y = y + (self._tp_reduce(shared) if self.w.tp > 1 else shared)
        return y

    def _qkv(self, L, normed, positions, slots, li):
        """Packed q / k / v of the new tokens, rotated (and per-head normalised) in place, k and v also written to
        their cache slots of layer ``li``: one GEMM and one fused launch."""
        cfg = self.cfg
        qkv = _linear(normed, L["qkv"], bias=L["qkv_bias"])
        if not self._composed_attention:
            return ops.rope_kv_write(qkv, positions, self.rope, slots, self.kv.k[self.kv_of[li]], self.kv.v[self.kv_of[li]], self.w.hq, self.w.hkv,
                                     cfg.head_dim, L["q_norm"], L["k_norm"], cfg.norm_epsilon)  # fmt: skip
        # attention variants the fused kernel does not cover (partial / interleaved rotary, RMSNorm over all heads):
        # the same steps as separate ops, then the ordinary cache write
        from slime_b200.models import mixers

        T, d, hq, hkv = qkv.shape[0], cfg.head_dim, self.w.hq, self.w.hkv
        q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
        if L["q_norm"] is not None:
            if cfg.qk_layernorm_full:
                q, k = self._full_norm(q, L["q_norm"]), self._full_norm(k, L["k_norm"])
            else:
                q = mixers._rms(q.view(T, hq, d), L["q_norm"], cfg.norm_epsilon).view(T, -1)
                k = mixers._rms(k.view(T, hkv, d), L["k_norm"], cfg.norm_epsilon).view(T, -1)
        if self.rope.shape[1] > 0:
            cos, sin = mixers.rotary_cos_sin(self.rope, positions, self._band_axes() if positions.dim() == 2 else None)
            q = mixers.apply_rotary(q.view(T, hq, d), cos, sin, cfg.rotary_interleaved).view(T, -1)
            k = mixers.apply_rotary(k.view(T, hkv, d), cos, sin, cfg.rotary_interleaved).view(T, -1)
        k, v = k.contiguous(), v.contiguous()
        ops.kv_write(k, v, slots, self.kv.k[self.kv_of[li]], self.kv.v[self.kv_of[li]])
        return torch.cat([q, k, v], dim=-1)

    def _band_axes(self):
        if self._mrope_axes is None:
            from slime_b200.models.vision import mrope_band_axes

            self._mrope_axes = mrope_band_axes(self.cfg.mrope_section, self.rope.shape[1] // 2, self.cfg.mrope_interleaved, self.device)
        return self._mrope_axes

    @torch.no_grad()
    def encode_images(self, pixel_values, grid_thw):
        """Image encoder outputs [placeholder tokens, H] for one request's images, and the list of same-shaped vectors
        that join the stream after the first layers (empty unless the encoder has deepstack outputs)."""
        out, extras = self.w.vision(pixel_values.to(self.device), grid_thw.to(self.device), with_deepstack=True)
        return out.to(self.w.dtype), [e.to(self.w.dtype) for e in extras]

    def _full_norm(self, t, w):
        """RMSNorm over all heads of the model: the sum of squares crosses the tensor-parallel ranks."""
        f = t.float()
        ss = f.pow(2).sum(-1, keepdim=True)
        n = f.shape[-1] * self.w.tp
        if self.w.tp > 1:
            ss = self._tp_reduce(ss)
        return (f * torch.rsqrt(ss / n + self.cfg.norm_epsilon) * w.float()).to(t.dtype)

    # ------------------------------------------------------------ latent attention layers
    def _mla_project(self, L, x, positions, slots, li):
        """Queries [T, hq, dn + dr] (rotary part rotated) of the new tokens; their latent vectors (normalised compressed
        key/value + rotated shared key) are written to the cache slab of layer ``li`` and returned [T, kv_lora + dr]."""
        from slime_b200.models import mixers

        cfg, T = self.cfg, x.shape[0]
        dn, dr = cfg.qk_head_dim, cfg.qk_pos_emb_head_dim
        hq = cfg.num_attention_heads // self.w.tp
        if "q_a" in L:
            q = ops.gemm(mixers._rms(ops.gemm(x, L["q_a"]), L["q_a_ln"], cfg.norm_epsilon), L["q_b"])
        else:
            q = ops.gemm(x, L["q_proj"])
        q = q.view(T, hq, dn + dr)
        c_kv, k_pe = ops.gemm(x, L["kv_a"]).split([cfg.kv_lora_rank, dr], dim=-1)
        cos, sin = mixers.rotary_cos_sin(self.rope, positions)
        q = torch.cat([q[..., :dn], mixers.apply_rotary(q[..., dn:], cos, sin, cfg.rotary_interleaved)], dim=-1)
        k_pe = mixers.apply_rotary(k_pe.reshape(T, 1, dr), cos, sin, cfg.rotary_interleaved).reshape(T, dr)
        parts = [mixers._rms(c_kv, L["kv_a_ln"], cfg.norm_epsilon), k_pe]
        index_q = None
        if cfg.index_topk:  # every layer caches an indexer key slot (unused on layers that reuse another layer's choice)
            hi, di = cfg.index_n_heads, cfg.index_head_dim
            if "idx_wk" in L:
                q_latent = mixers._rms(ops.gemm(x, L["q_a"]), L["q_a_ln"], cfg.norm_epsilon)
                il = cfg.rotary_interleaved if cfg.index_rotary_interleaved is None else cfg.index_rotary_interleaved
                qi = mixers.apply_rotary(ops.gemm(q_latent, L["idx_wq_b"]).view(T, hi, di), cos, sin, il)
                ki = torch.nn.functional.layer_norm(ops.gemm(x, L["idx_wk"]).float(), (di,), L["idx_k_norm_w"].float(), L["idx_k_norm_b"].float())
                ki = mixers.apply_rotary(ki.view(T, 1, di), cos, sin, il).view(T, di)
                wi = ops.gemm(x, L["idx_weights"]).float() * (hi**-0.5) * (di**-0.5)
                index_q = (qi.float(), wi)
                parts.append(ki.to(x.dtype))
            else:
                parts.append(x.new_zeros(T, di))
        latent = torch.cat(parts, dim=-1).contiguous()
        cache = self.kv.k[self.kv_of[li]]
        ok = slots >= 0
        cache.view(cache.shape[0], -1)[slots[ok].long()] = latent[ok].to(cache.dtype)
        return q, latent, index_q

    def _dsa_restrict(self, L, li, index_q, lat, allowed):
        """Keep, per query row, the ``index_topk`` cached tokens the indexer scores highest (rows that see fewer keep all).
        The choice is remembered for the layers of this pass that reuse it."""
        cfg = self.cfg
        if not cfg.index_topk:
            return allowed
        if index_q is None:
            return self._dsa_masks[L["index_source"]]
        if allowed.shape[1] > cfg.index_topk:
            qi, wi = index_q
            ki = lat[..., cfg.kv_lora_rank + cfg.qk_pos_emb_head_dim :].float()
            logits = (torch.einsum("bhd,bld->bhl", qi, ki).relu_() * wi[:, :, None]).sum(1).masked_fill(~allowed, float("-inf"))
            pick = torch.zeros_like(allowed).scatter_(1, logits.topk(cfg.index_topk, dim=-1).indices, True)
            allowed = pick & allowed
        self._dsa_masks[li] = allowed
        return allowed

    def _mla_absorbed(self, L, q, latent, allowed):
        """Attention of queries ``q`` [B, hq, dn + dr] over per-row latent contexts ``latent`` [B, Lmax, kv_lora + dr] with
        ``allowed`` [B, Lmax]: the key expansion is folded into the query and the value expansion applied after the
        weighted sum, so the cached vector is never expanded per head. Returns [B, hq * dv]."""
        cfg = self.cfg
        dn, dv, r = cfg.qk_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        hq = q.shape[1]
        dr = cfg.qk_pos_emb_head_dim
        w = L["kv_b"].float().view(hq, dn + dv, r)
        q_lat = torch.einsum("bhd,hdr->bhr", q[..., :dn].float(), w[:, :dn])  # queries in latent coordinates
        lat = latent.float()
        scores = (torch.einsum("bhr,blr->bhl", q_lat, lat[..., :r]) + torch.einsum("bhd,bld->bhl", q[..., dn:].float(), lat[..., r : r + dr]))
        scores = (scores * self.scale).masked_fill(~allowed[:, None, :], float("-inf"))
        out_lat = torch.einsum("bhl,blr->bhr", scores.softmax(-1), lat[..., :r])
        return torch.einsum("bhr,hdr->bhd", out_lat, w[:, dn:]).reshape(q.shape[0], hq * dv).to(self.w.dtype)

    def _mla_prefill(self, L, li, x, positions, slots, cu_q, kv_gather_slots, cu_k, fresh):
        q, latent, index_q = self._mla_project(L, x, positions, slots, li)
        cache = self.kv.k[self.kv_of[li]]
        ctx_lat = latent if fresh else cache.view(cache.shape[0], -1).index_select(0, kv_gather_slots)
        cq, ck = cu_q.tolist(), (cu_q if fresh else cu_k).tolist()
        lmax = max(b - a for a, b in zip(ck[:-1], ck[1:]))
        T = x.shape[0]
        lat = ctx_lat.new_zeros(T, lmax, ctx_lat.shape[-1])
        allowed = torch.zeros(T, lmax, dtype=torch.bool, device=x.device)
        for (qa, qb), (ka, kb) in zip(zip(cq[:-1], cq[1:]), zip(ck[:-1], ck[1:])):
            n_q, n_k = qb - qa, kb - ka
            if n_q <= 0:
                continue
            lat[qa:qb, :n_k] = ctx_lat[ka:kb]
            allowed[qa:qb, :n_k] = torch.ones(n_q, n_k, dtype=torch.bool, device=x.device).tril(diagonal=n_k - n_q)
        return self._mla_absorbed(L, q, lat, self._dsa_restrict(L, li, index_q, lat, allowed))

    def _mla_decode(self, L, li, x, positions, slots, block_table, seq_lens, n):
        q, _, index_q = self._mla_project(L, x, positions, slots, li)
        cache = self.kv.k[self.kv_of[li]]
        ps = self.kv.page_size
        lmax = int(seq_lens.max())
        pos = torch.arange(lmax, device=x.device)
        idx = block_table[:, (pos // ps).clamp_max(block_table.shape[1] - 1)].long() * ps + pos % ps  # [n, lmax]
        lat = cache.view(cache.shape[0], -1)[idx.clamp_(0, cache.shape[0] - 1)]
        return self._mla_absorbed(L, q, lat, self._dsa_restrict(L, li, index_q, lat, pos[None, :] < seq_lens[:, None]))

    # ------------------------------------------------------------ gated delta-net layers
    def _gdn_project(self, L, x):
        """Input projections of a delta-net layer -> (pre-convolution q|k|v channels [T, C], z [T, Hv, Dv], b, a [T, Hv])."""
        cfg, T = self.cfg, x.shape[0]
        hk, hv, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
        if "gdn_qkvz" in L:  # rows grouped per key head: q, k, then that head's value and gate heads
            r = hv // hk
            qkvz = ops.gemm(x, L["gdn_qkvz"]).view(T, hk, 2 * dk + 2 * r * dv)
            q, k, v, z = qkvz.split([dk, dk, r * dv, r * dv], dim=-1)
            b, a = ops.gemm(x, L["gdn_ba"]).view(T, hk, 2 * r).split([r, r], dim=-1)
            mixed = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=-1)
            return mixed, z.reshape(T, hv, dv), b.reshape(T, hv), a.reshape(T, hv)
        return ops.gemm(x, L["gdn_qkv"]), ops.gemm(x, L["gdn_z"]).view(T, hv, dv), ops.gemm(x, L["gdn_b"]), ops.gemm(x, L["gdn_a"])

    def _gdn_finish(self, L, o, z):
        """Gated RMSNorm of the delta-rule output and the output projection."""
        from slime_b200.models import mixers

        T = o.shape[0]
        y = mixers._rms(o, L["gdn_norm"], self.cfg.norm_epsilon).float() * torch.nn.functional.silu(z.float())
        return ops.gemm(y.to(self.w.dtype).reshape(T, -1), L["gdn_out"])

    def _gdn_gates(self, L, b, a):
        beta = torch.sigmoid(b.float())
        g = -L["gdn_A_log"].float().exp() * torch.nn.functional.softplus(a.float() + L["gdn_dt_bias"].float())
        return g, beta

    def _gdn_heads(self, mixed):
        cfg, T = self.cfg, mixed.shape[0]
        hk, hv, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
        q, k, v = mixed.split([hk * dk, hk * dk, hv * dv], dim=-1)
        q, k, v = q.view(T, hk, dk), k.view(T, hk, dk), v.view(T, hv, dv)
        if hv // hk > 1:
            q, k = q.repeat_interleave(hv // hk, dim=1), k.repeat_interleave(hv // hk, dim=1)
        return q, k, v

    def _gdn_prefill(self, L, li, x, positions_in_call, cu_q, states_in, states_out):
        """Delta-net layer over the new tokens of every request; ``states_in[i][li]`` = (state, convolution history) the
        request arrived with (None at its first chunk); the states after the chunk go to ``states_out[i][li]``."""
        from slime_b200.models import mixers

        K = self.cfg.linear_conv_kernel_dim
        mixed_in, z, b, a = self._gdn_project(L, x)
        n_req = cu_q.numel() - 1
        S_in = [None if states_in is None or states_in[i] is None else states_in[i][li][0] for i in range(n_req)]
        h_in = [None if states_in is None or states_in[i] is None else states_in[i][li][1] for i in range(n_req)]
        mixed = mixers.causal_short_conv(mixed_in, L["gdn_conv"], positions_in_call, history=h_in if any(h is not None for h in h_in) else None,
                                         cu_seqlens=cu_q)  # fmt: skip
        q, k, v = self._gdn_heads(mixed)
        g, beta = self._gdn_gates(L, b, a)
        o, finals = mixers.gated_delta_rule_chunked(q, k, v, g, beta, cu_q, initial_states=S_in, return_final_states=True)
        bounds = cu_q.tolist()
        for i, (lo, hi) in enumerate(zip(bounds[:-1], bounds[1:])):
            prev = h_in[i] if h_in[i] is not None else mixed_in.new_zeros(K - 1, mixed_in.shape[1])
            hist = torch.cat([prev.to(mixed_in.dtype), mixed_in[lo:hi]])[-(K - 1):]
            states_out[i][li] = (finals[i], hist)
        return self._gdn_finish(L, o.to(self.w.dtype), z)

    def _gdn_decode(self, L, li, x, n):
        from slime_b200.models import mixers

        mixed_in, z, b, a = self._gdn_project(L, x)
        mixed = mixers.short_conv_step(mixed_in, L["gdn_conv"], self.gdn_conv[li][:n])
        q, k, v = self._gdn_heads(mixed)
        g, beta = self._gdn_gates(L, b, a)
        o = mixers.gated_delta_rule_step(q, k, v, g, beta, self.gdn_S[li][:n])
        return self._gdn_finish(L, o.to(self.w.dtype), z)

    def load_gdn_state(self, slot: int, states: dict | None):
        """Put a request's recurrent states (from its prefill) into decode slot ``slot``."""
        for li in self.gdn_S:
            S, hist = states[li]
            self.gdn_S[li][slot].copy_(S)
            self.gdn_conv[li][slot].copy_(hist)

    def _post_norm(self, x, w):
        """GLM-4 sandwich norm: the sub-layer's output is normalised before it joins the residual stream."""
        return x if w is None else ops.rmsnorm(x, w, self.cfg.norm_epsilon)[0]

    # --------------------------------------------------------------------- prefill
    @torch.no_grad()
    def prefill(self, ids, positions, slots, cu_q, kv_gather_slots, cu_k, max_q, max_k, last_rows, fresh: bool, gdn_states=None,
                embed_rows=None):
        """Extend pass over packed new tokens.

        ids/positions/slots: [T] for the new tokens; ``cu_q`` their per-request boundaries.
        ``kv_gather_slots``/``cu_k``: cache slots of every context token (cached prefix + new) per
        request, used when some context is already cached (``fresh`` False). Returns logits
        ``[len(last_rows), V/tp]`` fp32 for the requested rows and, when ``last_rows`` is None, all rows.
        Models with delta-net layers: ``gdn_states[i]`` is request i's recurrent state from its earlier chunks (or
        None); the states after this pass are left in ``last_gdn_states``.
        Vision inputs: ``positions`` may be ``[3, T]`` (temporal / height / width streams) and ``embed_rows`` = (rows,
        vectors) replaces the embeddings of image placeholder tokens by the encoder's outputs.
        """
        cfg, w, d = self.cfg, self.w, self.cfg.head_dim
        x = ops.embedding(ids, w.embed, w.rank * w.vocab_local)
        x = self._tp_reduce(x) if w.tp > 1 else x
        deepstack = []
        if embed_rows is not None:
            x = x.index_copy(0, embed_rows[0], embed_rows[1].to(x.dtype))
            deepstack = embed_rows[2] if len(embed_rows) > 2 else []
        res = None
        T = ids.numel()
        if self.has_gdn:
            from slime_b200.models.gpt import positions_from_cu_seqlens

            in_call = positions_from_cu_seqlens(cu_q, T)  # position inside this pass (a later chunk starts at 0 again)
            self.last_gdn_states = [dict() for _ in range(cu_q.numel() - 1)]
        for li, L in enumerate(w.layers):
            if 0 < li <= len(deepstack):  # vision vectors that join the stream after layer li - 1 (stream = x + res)
                x = x.index_add(0, embed_rows[0], deepstack[li - 1].to(x.dtype))
            normed, res = ops.rmsnorm(x, L["ln1"], cfg.norm_epsilon, res)
            if L["kind"] == "gdn":
                x = self._gdn_prefill(L, li, normed, in_call, cu_q, gdn_states, self.last_gdn_states)
                normed, res = ops.rmsnorm(x, L["ln2"], cfg.norm_epsilon, res)
                x = self._mlp(L, normed)
                continue
            if L["kind"] == "mla":
                ctx = self._mla_prefill(L, li, normed, positions, slots, cu_q, kv_gather_slots, cu_k, fresh)
                x = self._tp_reduce(_linear(ctx, L["o"], out_dtype=self._proj_dtype))
                normed, res = ops.rmsnorm(x, L["ln2"], cfg.norm_epsilon, res)
                x = self._mlp(L, normed)
                continue
            qkv = self._qkv(L, normed, positions, slots, li)
            q3 = qkv.view(T, w.hq + 2 * w.hkv, d)
            q, k, v = q3[:, : w.hq], q3[:, w.hq : w.hq + w.hkv], q3[:, w.hq + w.hkv :]
            if fresh:
                ctx = ops.varlen_attention(q, k, v, cu_q, max_q, self.scale, sinks=L.get("sinks"))
            else:
                k_all = self.kv.k[self.kv_of[li]].index_select(0, kv_gather_slots)
                v_all = self.kv.v[self.kv_of[li]].index_select(0, kv_gather_slots)
                ctx = _extend_attention(q, k_all, v_all, cu_q, cu_k, max_q, max_k, self.scale, sinks=L.get("sinks"))
            ctx = ctx.reshape(T, -1)
            if "gate" in L:
                ctx = ctx * torch.sigmoid(ops.gemm(normed, L["gate"]).float()).to(ctx.dtype)
            x = self._tp_reduce(_linear(ctx, L["o"], out_dtype=self._proj_dtype))
            x = self._post_norm(x, L["post_attn_ln"])
            normed, res = ops.rmsnorm(x, L["ln2"], cfg.norm_epsilon, res)
            x = self._post_norm(self._mlp(L, normed), L["post_mlp_ln"])
        h, hidden = ops.rmsnorm(x, w.final_norm, cfg.norm_epsilon, res)
        self.last_hidden = hidden if w.draft else None  # kept for a draft head only: a chunk's stream is tens of megabytes
        if last_rows is not None:
            h = h.index_select(0, last_rows)
        return self._gather_logits(ops.gemm(h, w.lm_head, out_dtype=torch.float32))

    @torch.no_grad()
    def draft_extend(self, depth: int, hidden, next_ids, positions, slots, cu_q, kv_gather_slots, cu_k, max_q, max_k, fresh: bool):
        """Draft head ``depth`` over packed rows: row p joins the residual stream ``hidden[p]`` the trunk (or the previous
        draft step) left at position p with the embedding of the token at position p + 1, runs one transformer layer with
        its own cache slab (written at ``slots``) and returns ``(normed [T, H], stream [T, H])``: the first feeds the shared
        output head (a guess for the token at position p + 2), the second is the next draft step's ``hidden``. Same
        computation as ``models/gpt.py::MTPLayer``; arguments as in ``prefill``."""
        cfg, w, d, eps = self.cfg, self.w, self.cfg.head_dim, self.cfg.norm_epsilon
        L, li = w.draft[depth], cfg.num_layers + depth
        recording, self.record_routed = self.record_routed, False  # a draft head's routing is nobody's training signal
        try:
            emb = ops.embedding(next_ids, w.embed, w.rank * w.vocab_local)
            emb = self._tp_reduce(emb) if w.tp > 1 else emb
            e_n = ops.rmsnorm(emb, L["enorm"], eps)[0]
            h_n = ops.rmsnorm(hidden.to(emb.dtype), L["hnorm"], eps)[0]
            x = ops.gemm(torch.cat([e_n, h_n], dim=-1), L["eh_proj"])
            T = x.shape[0]
            normed, res = ops.rmsnorm(x, L["ln1"], eps, None)
            if L["kind"] == "mla":
                ctx = self._mla_prefill(L, li, normed, positions, slots, cu_q, kv_gather_slots, cu_k, fresh)
                x = self._tp_reduce(_linear(ctx, L["o"], out_dtype=self._proj_dtype))
            else:
                qkv = self._qkv(L, normed, positions, slots, li)
                q3 = qkv.view(T, w.hq + 2 * w.hkv, d)
                q, k, v = q3[:, : w.hq], q3[:, w.hq : w.hq + w.hkv], q3[:, w.hq + w.hkv :]
                if fresh:
                    ctx = ops.varlen_attention(q, k, v, cu_q, max_q, self.scale, sinks=L.get("sinks"))
                else:
                    k_all = self.kv.k[self.kv_of[li]].index_select(0, kv_gather_slots)
                    v_all = self.kv.v[self.kv_of[li]].index_select(0, kv_gather_slots)
                    ctx = _extend_attention(q, k_all, v_all, cu_q, cu_k, max_q, max_k, self.scale, sinks=L.get("sinks"))
                ctx = ctx.reshape(T, -1)
                if "gate" in L:
                    ctx = ctx * torch.sigmoid(ops.gemm(normed, L["gate"]).float()).to(ctx.dtype)
                x = self._post_norm(self._tp_reduce(_linear(ctx, L["o"], out_dtype=self._proj_dtype)), L["post_attn_ln"])
            normed, res = ops.rmsnorm(x, L["ln2"], eps, res)
            x = self._post_norm(self._mlp(L, normed), L["post_mlp_ln"])
            return ops.rmsnorm(x, L["final_ln"], eps, res)
        finally:
            self.record_routed = recording

    def logits_of(self, normed):
        """Output head over already normalised rows -> fp32 logits over the whole vocabulary."""
        return self._gather_logits(ops.gemm(normed, self.w.lm_head, out_dtype=torch.float32))

    # ---------------------------------------------------------------------- decode
    # Per-slot decode state is device-owned (ids / pos / out_pos): the token sampled in step t is the
    # input of step t+1 without touching the host, so steps can be launched back to back while the host
    # lags one step behind reading results. The host owns the block table, the active mask, sampling
    # parameters and "init" records for slots that start decoding; those live in one flat pinned buffer
    # (double-buffered) uploaded with a single copy per step.
    HOST_FIELDS = ("active", "init_mask", "init_ids", "init_pos", "init_out_pos", "top_k", "temperature", "top_p", "min_p")

    def _alloc_static(self):
        B, W, dev = self.max_batch, self.max_pages_per_req, self.device
        nf = len(self.HOST_FIELDS)
        total = (nf + 2) * B + B * W
        self._flat_dev = torch.zeros(total, dtype=torch.int32, device=dev)
        self._flat_hosts = [torch.zeros(total, dtype=torch.int32, pin_memory=(dev.type == "cuda")) for _ in range(2)]
        self._host_events = [None, None]
        self._host_idx = 0

        def views(flat):
            out, off = {}, 0
            for f in self.HOST_FIELDS:
                v = flat[off : off + B]
                out[f] = v.view(torch.float32) if f in ("temperature", "top_p", "min_p") else v
                off += B
            out["seeds"] = flat[off : off + 2 * B].view(torch.int64)
            off += 2 * B
            out["block_table"] = flat[off : off + B * W].view(B, W)
            return out

        self._static = views(self._flat_dev)
        # the scheduler edits `host` (plain numpy, not pinned); upload copies it into the free pinned buffer
        import numpy as np

        self._host_np = np.zeros(total, dtype=np.int32)
        self.host = {k: v.numpy() for k, v in views(torch.from_numpy(self._host_np)).items()}
        self.host["temperature"][:] = 1.0
        self.host["top_p"][:] = 1.0
        i32 = lambda *sh: torch.zeros(*sh, dtype=torch.int32, device=dev)  # noqa: E731
        self._dev_state = dict(ids=i32(B), pos=i32(B), out_pos=i32(B), ids_eff=i32(B), pos_eff=i32(B), seq_lens=i32(B) + 1,
                               slots=i32(B))  # fmt: skip

    def upload_static(self):
        """Copy the scheduler's host state to the device through a pinned staging buffer that is not in
        flight (two alternate; an event guards reuse). ``init_mask`` is consumed by the upload."""
        k = self._host_idx
        ev = self._host_events[k]
        if ev is not None:
            ev.synchronize()
        stage = self._flat_hosts[k]
        stage.numpy()[:] = self._host_np
        self._flat_dev.copy_(stage, non_blocking=True)
        if self.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
            self._host_events[k] = ev
        self._host_idx = 1 - k
        self.host["init_mask"][:] = 0
        return stage.numel() * 4

    def _decode_step(self, n: int, filtered: bool, kept_cap: int):
        """prepare -> model -> sample -> advance for slots [0, n). Returns (tokens, logprobs, kept_ids, kept_cnt)."""
        cfg, w, d = self.cfg, self.w, self.cfg.head_dim
        st, ds = self._static, self._dev_state
        ps, W = self.kv.page_size, self.max_pages_per_req
        ids, pos, seq_lens, slots = ds["ids_eff"][:n], ds["pos_eff"][:n], ds["seq_lens"][:n], ds["slots"][:n]
        bt = st["block_table"][:n]
        if self.device.type == "cuda":
            from slime_b200.ops import _lib

            P = _lib.ptr
            _lib.check(_lib.lib().sb_decode_prepare(
                P(ds["ids"]), P(ds["pos"]), P(ds["out_pos"]), P(st["init_mask"]), P(st["init_ids"]), P(st["init_pos"]),
                P(st["init_out_pos"]), P(st["active"]), P(st["block_table"]), P(ds["ids_eff"]), P(ds["pos_eff"]),
                P(ds["seq_lens"]), P(ds["slots"]), n, ps, W, _lib.stream()), "sb_decode_prepare")  # fmt: skip
        else:
            self._prepare_reference(n)
        if self.rope_delta is not None:
            pos = pos + self.rope_delta[:n]  # rotary position of a request that carries images
        x = ops.embedding(ids, w.embed, w.rank * w.vocab_local)
        x = self._tp_reduce(x) if w.tp > 1 else x
        if self._fused_tp is not None:
            # after the NCCL all-reduce of the vocab-parallel embedding: that collective has already lined the ranks
            # up, so the bounded barrier only ever waits for launch jitter
            self._fused_tp.begin_forward()
        normed, res = ops.rmsnorm(x, w.layers[0]["ln1"], cfg.norm_epsilon, None)
        for li, L in enumerate(w.layers):
            if L["kind"] == "gdn":
                normed, res = ops.rmsnorm(self._gdn_decode(L, li, normed, n), L["ln2"], cfg.norm_epsilon, res)
            elif L["kind"] == "mla":
                ctx = self._mla_decode(L, li, normed, pos, slots, bt, seq_lens, n)
                normed, res = self._row_parallel_norm(ctx, L["o"], L["ln2"], res, n)
            else:
                qkv = self._qkv(L, normed, pos, slots, li)
                q3 = qkv.view(n, w.hq + 2 * w.hkv, d)
                ctx = ops.paged_decode_attention(q3[:, : w.hq], self.kv.k[self.kv_of[li]], self.kv.v[self.kv_of[li]], bt, seq_lens, ps,
                                                 self.scale, sinks=L.get("sinks")).reshape(n, -1)  # fmt: skip
                if "gate" in L:
                    ctx = ctx * torch.sigmoid(ops.gemm(normed, L["gate"]).float()).to(ctx.dtype)
                normed, res = self._row_parallel_norm(ctx, L["o"], L["ln2"], res, n, post=L["post_attn_ln"])
            # the norm that follows the MLP is the next layer's input norm (or the final norm)
            next_ln = w.layers[li + 1]["ln1"] if li + 1 < len(w.layers) else w.final_norm
            if "gate_up" in L:
                act = ops.swiglu(_linear(normed, L["gate_up"]))
                normed, res = self._row_parallel_norm(act, L["down"], next_ln, res, n, post=L["post_mlp_ln"])
            else:
                normed, res = ops.rmsnorm(self._post_norm(self._moe(L, normed), L["post_mlp_ln"]), next_ln, cfg.norm_epsilon, res)
        h = normed
        logits = self._gather_logits(ops.gemm(h, w.lm_head, out_dtype=torch.float32))
        tok, lp, kept_ids, kept_cnt = ops.sample(
            logits, st["temperature"][:n], st["top_k"][:n] if filtered else None, st["top_p"][:n] if filtered else None,
            st["min_p"][:n] if filtered else None, st["seeds"][:n], ds["out_pos"][:n], kept_cap,
        )  # fmt: skip
        routed = self.take_routed()
        if self.device.type == "cuda":
            _lib.check(_lib.lib().sb_decode_advance(P(ds["ids"]), P(ds["pos"]), P(ds["out_pos"]), P(st["active"]), P(tok), n,
                                                    _lib.stream()), "sb_decode_advance")  # fmt: skip
        else:
            act = st["active"][:n].bool()
            ds["ids"][:n] = torch.where(act, tok, ds["ids"][:n])
            ds["pos"][:n] += act.int()
            ds["out_pos"][:n] += act.int()
        return tok, lp, kept_ids, kept_cnt, routed

    def _prepare_reference(self, n):
        st, ds = self._static, self._dev_state
        ps = self.kv.page_size
        init = st["init_mask"][:n].bool()
        for dst, src in (("ids", "init_ids"), ("pos", "init_pos"), ("out_pos", "init_out_pos")):
            ds[dst][:n] = torch.where(init, st[src][:n], ds[dst][:n])
        act = st["active"][:n].bool()
        p = ds["pos"][:n].long()
        slot = st["block_table"][:n].gather(1, (p // ps)[:, None]).squeeze(1).long() * ps + p % ps
        idle = torch.arange(n) % ps
        ds["ids_eff"][:n] = torch.where(act, ds["ids"][:n], torch.zeros_like(ds["ids"][:n]))
        ds["pos_eff"][:n] = torch.where(act, ds["pos"][:n], torch.zeros_like(ds["pos"][:n]))
        ds["seq_lens"][:n] = torch.where(act, ds["pos"][:n] + 1, torch.ones_like(ds["pos"][:n]))
        ds["slots"][:n] = torch.where(act, slot, idle).to(torch.int32)

    @torch.no_grad()
    def decode(self, n: int, filtered: bool, kept_cap: int = 0):
        """One decode step over slots [0, n) (host state must have been uploaded). Under CUDA graphs the
        step is one replay of the bucket that covers ``n``; extra slots are inactive by construction. MoE layers are
        captured too: their expert-sorted layout is built on the device with static shapes. ``last_routed`` holds the
        step's expert choices when ``record_routed`` is set (a buffer of the graph: copy it before the next replay)."""
        if not self.use_cuda_graph:
            *outs, self.last_routed = self._decode_step(n, filtered, kept_cap)
            return tuple(outs)
        bucket = next(b for b in self.graph_buckets if b >= n)
        key = (bucket, filtered, kept_cap)
        if key not in self.graphs:
            self._capture(bucket, filtered, kept_cap)
        graph, outs, n_kernels = self.graphs[key]
        self.replayed_launches += n_kernels
        graph.replay()
        self.last_routed = outs[4]
        return outs[:4]

    def _capture(self, bucket, filtered, kept_cap):
        """Capture one decode step. Warm-up and capture run with every slot inactive, so they only touch the
        reserved scratch page and leave the device-owned request state unchanged."""
        from slime_b200.ops import _lib

        saved_active = self._static["active"].clone()
        saved_init = self._static["init_mask"].clone()
        self._static["active"].zero_()
        self._static["init_mask"].zero_()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._decode_step(bucket, filtered, kept_cap)
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        before = _lib.launch_count()
        with torch.cuda.graph(g):
            outs = self._decode_step(bucket, filtered, kept_cap)
        self.graphs[(bucket, filtered, kept_cap)] = (g, outs, _lib.launch_count() - before)
        self._static["active"].copy_(saved_active)
        self._static["init_mask"].copy_(saved_init)

    def drop_graphs(self):
        """Memory tag ``cuda_graph``: captured graphs pin their private pools."""
        self.graphs.clear()


def _extend_attention(q, k_all, v_all, cu_q, cu_k, max_q, max_k, scale, sinks=None):
    """Attention of new tokens over (cached + new) context, causal aligned to the sequence end."""
    if q.is_cuda or sinks is not None:
        from slime_b200.ops import attention

        return attention.segment_attention(q, k_all, v_all, attention.segments_extend(cu_q, cu_k), scale, sinks)
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
