"""Trainer (Megatron-named) <-> Hugging Face tensor naming and layout.

Forward direction (``convert_to_hf``): a *TP-gathered* trainer tensor becomes one or more
HF tensors: fused qkv -> q_proj / k_proj / v_proj, fused fc1 -> gate_proj / up_proj, expert
``weight{e}`` -> ``experts.{e}.*``. Parity: slime/backends/megatron_utils/megatron_to_hf/
(qwen2.py:5-71, qwen3moe.py:6-117, llama.py, glm4.py, glm4moe.py, ...).
Inverse direction (``hf_to_trainer_name``/``merge_*``) is used by the HF loader
(slime/backends/megatron_utils/hf_to_megatron/common.py:70-134).

In memory this backend keeps fused qkv rows as [q heads | k heads | v heads]; the Megatron
on-disk layout interleaves per KV group ``[g][q_per_g*d | d | d]``. ``qkv_to_megatron_layout``
/ ``qkv_from_megatron_layout`` translate for torch_dist checkpoints.
"""

from __future__ import annotations

import re

import torch

from slime_b200.models.config import ModelConfig

_LAYER = re.compile(r"^decoder\.layers\.(\d+)\.(.+)$")
_EXPERT = re.compile(r"^mlp\.experts\.linear_fc([12])\.weight(\d+)$")
_MTP = re.compile(r"^mtp\.layers\.(\d+)\.(.+)$")
_QWEN_MTP = {"enorm.weight": "mtp.pre_fc_norm_embedding.weight", "hnorm.weight": "mtp.pre_fc_norm_hidden.weight",
             "final_layernorm.weight": "mtp.norm.weight"}  # fmt: skip
_MIMO_MTP = {"enorm.weight": "token_layernorm.weight", "hnorm.weight": "hidden_layernorm.weight",
             "final_layernorm.weight": "final_layernorm.weight"}  # fmt: skip


def split_qkv(cfg: ModelConfig, t: torch.Tensor):
    """Full (all-TP-ranks) fused tensor [ (Hq+2Hkv)*d , ...] -> (q, k, v)."""
    d = cfg.head_dim
    q, k = cfg.num_attention_heads * d, cfg.num_query_groups * d
    return t[:q], t[q : q + k], t[q + k :]


def qkv_to_megatron_layout(cfg: ModelConfig, t: torch.Tensor) -> torch.Tensor:
    """[q | k | v] rows -> per-KV-group interleave [g][q_per_g*d | d | d]."""
    d, g = cfg.head_dim, cfg.num_query_groups
    per = cfg.num_attention_heads // g
    q, k, v = split_qkv(cfg, t)
    rest = t.shape[1:]
    q = q.reshape(g, per * d, *rest)
    k = k.reshape(g, d, *rest)
    v = v.reshape(g, d, *rest)
    return torch.cat([q, k, v], dim=1).reshape(-1, *rest)


def qkv_from_megatron_layout(cfg: ModelConfig, t: torch.Tensor) -> torch.Tensor:
    d, g = cfg.head_dim, cfg.num_query_groups
    per = cfg.num_attention_heads // g
    rest = t.shape[1:]
    x = t.reshape(g, (per + 2) * d, *rest)
    q = x[:, : per * d].reshape(-1, *rest)
    k = x[:, per * d : (per + 1) * d].reshape(-1, *rest)
    v = x[:, (per + 1) * d :].reshape(-1, *rest)
    return torch.cat([q, k, v], dim=0)


def _qkv_pieces(cfg: ModelConfig, tp: int = 1) -> list[int]:
    """Row counts of the pieces of a fused projection shard: q, (gate,) k, v."""
    d = cfg.head_dim
    q, k = cfg.num_attention_heads // tp * d, cfg.num_query_groups // tp * d
    return [q] * (2 if cfg.attention_output_gate else 1) + [k, k]


def _zero_centred(cfg: ModelConfig) -> bool:
    """Qwen3-Next / Qwen3.5 checkpoints store ``w - 1`` for their RMSNorm weights (the layer computes ``1 + w``); the
    trainer keeps the effective weight."""
    return _family(cfg) in ("qwen3next", "qwen3_5")


# trainer name inside ``self_attention.`` -> checkpoint name inside the layer, for the mixers of models/mixers.py
_MIXER_NAMES = {
    # gated delta-net
    "input_layernorm.weight": "input_layernorm.weight", "in_proj_qkvz.weight": "linear_attn.in_proj_qkvz.weight",
    "in_proj_ba.weight": "linear_attn.in_proj_ba.weight", "in_proj_qkv.weight": "linear_attn.in_proj_qkv.weight",
    "in_proj_z.weight": "linear_attn.in_proj_z.weight", "in_proj_b.weight": "linear_attn.in_proj_b.weight",
    "in_proj_a.weight": "linear_attn.in_proj_a.weight", "conv1d.weight": "linear_attn.conv1d.weight",
    "dt_bias": "linear_attn.dt_bias", "A_log": "linear_attn.A_log", "norm.weight": "linear_attn.norm.weight",
    "out_proj.weight": "linear_attn.out_proj.weight",
    # latent attention (DeepSeek-V3 naming)
    "linear_q_down_proj.weight": "self_attn.q_a_proj.weight", "linear_q_up_proj.weight": "self_attn.q_b_proj.weight",
    "linear_q_proj.weight": "self_attn.q_proj.weight", "linear_kv_down_proj.weight": "self_attn.kv_a_proj_with_mqa.weight",
    "kv_layernorm.weight": "self_attn.kv_a_layernorm.weight", "linear_kv_up_proj.weight": "self_attn.kv_b_proj.weight",
    # lightning indexer
    "wq_b.weight": "self_attn.indexer.wq_b.weight", "wk.weight": "self_attn.indexer.wk.weight",
    "k_norm.weight": "self_attn.indexer.k_norm.weight", "k_norm.bias": "self_attn.indexer.k_norm.bias",
    "weights_proj.weight": "self_attn.indexer.weights_proj.weight",
    # learnable sinks
    "softmax_offset": "self_attn.sinks",
}  # fmt: skip
_ZERO_CENTRED = ("input_layernorm.weight", "post_attention_layernorm.weight", "model.norm.weight", "q_norm.weight", "k_norm.weight")


def _mixer_to_hf(cfg: ModelConfig, layer: str, sub: str, t: torch.Tensor):
    """``self_attention.<sub>`` of a non-standard mixer -> checkpoint pairs, or None when ``sub`` is not one of theirs."""
    p = f"model.layers.{layer}"
    latent = cfg.multi_latent_attention
    if sub == "q_layernorm.weight" and latent:
        return [(f"{p}.self_attn.q_a_layernorm.weight", t)]
    if sub not in _MIXER_NAMES:
        return None
    if sub == "conv1d.weight":
        t = t.unsqueeze(1)  # depthwise Conv1d weight [C, 1, K]
    return [(f"{p}.{_MIXER_NAMES[sub]}", t)]


def _gated_q_to_hf(cfg: ModelConfig, q: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """[q heads] + [gate heads] -> the checkpoint's q_proj rows, per head (query, gate)."""
    d, h = cfg.head_dim, cfg.num_attention_heads
    rest = q.shape[1:]
    return torch.cat([q.reshape(h, d, *rest), gate.reshape(h, d, *rest)], dim=1).reshape(2 * h * d, *rest)


def _gated_q_from_hf(cfg: ModelConfig, qg: torch.Tensor):
    d, h = cfg.head_dim, cfg.num_attention_heads
    rest = qg.shape[1:]
    x = qg.reshape(h, 2 * d, *rest)
    return x[:, :d].reshape(h * d, *rest), x[:, d:].reshape(h * d, *rest)


def _family(cfg: ModelConfig) -> str:
    a = (cfg.model_arch or "").lower().replace("vlmoe", "moe").replace("vl", "")  # Qwen3-VL(-MoE): the text model's family
    for key in ("qwen3_5", "qwen3next", "qwen3moe", "qwen2moe", "qwen3", "qwen2", "glm4moe", "glm4", "llama", "mimo",
                "deepseek", "minimax"):  # fmt: skip
        if key in a.replace("_", "").replace("-", "") or key in a:
            return key
    return "qwen2"


def split_stacked_experts(cfg: ModelConfig, name: str, t: torch.Tensor) -> list[tuple[str, torch.Tensor]] | None:
    """Qwen3-VL-MoE files keep a layer's experts in two stacked tensors, ``mlp.experts.gate_up_proj`` of shape
    [experts, hidden, 2 x width] and ``mlp.experts.down_proj`` of shape [experts, width, hidden] (the operands of
    ``x @ W``, i.e. the transposes of linear-layer weights). Returns the per-expert ``gate_proj`` / ``up_proj`` /
    ``down_proj`` linear weights every consumer here names, or None for any other tensor. A stack that already has the
    linear-layer orientation is taken as it is; where hidden = 2 x width makes the two indistinguishable, the files'
    orientation is assumed."""
    if t.dim() != 3 or not name.endswith((".mlp.experts.gate_up_proj", ".mlp.experts.down_proj")):
        return None
    h, w = cfg.hidden_size, cfg.moe_ffn_hidden_size
    out = []
    if name.endswith("gate_up_proj"):
        base = name[: -len("gate_up_proj")]
        if tuple(t.shape[1:]) != (h, 2 * w):
            assert tuple(t.shape[1:]) == (2 * w, h), (name, tuple(t.shape))
            t = t.transpose(1, 2)
        for e in range(t.shape[0]):
            out += [(f"{base}{e}.gate_proj.weight", t[e, :, :w].t()), (f"{base}{e}.up_proj.weight", t[e, :, w:].t())]
    else:
        base = name[: -len("down_proj")]
        if tuple(t.shape[1:]) != (w, h):
            assert tuple(t.shape[1:]) == (h, w), (name, tuple(t.shape))
            t = t.transpose(1, 2)
        out = [(f"{base}{e}.down_proj.weight", t[e].t()) for e in range(t.shape[0])]
    return out


def stacked_expert_source(name: str) -> tuple[str, int, str] | None:
    """For a per-expert name ``....mlp.experts.<e>.<gate|up|down>_proj.weight``: the stacked tensor that would hold it in
    a file of the layout above, the expert index and the part."""
    m = re.match(r"(.*\.mlp\.experts\.)(\d+)\.(gate|up|down)_proj\.weight$", name)
    if m is None:
        return None
    return m.group(1) + ("down_proj" if m.group(3) == "down" else "gate_up_proj"), int(m.group(2)), m.group(3)


def _vl_name(cfg: ModelConfig, hf_name: str) -> str:
    """Checkpoints of models with vision inputs keep the language model under ``model.language_model`` (next to
    ``model.visual``, whose tensors keep their names). Parity: slime/backends/megatron_utils/megatron_to_hf/qwen3_vl.py:5-25."""
    if cfg.vision is not None and hf_name.startswith("model.") and not hf_name.startswith(("model.visual.", "model.language_model.")):
        return "model.language_model." + hf_name[len("model.") :]
    return hf_name


_MINIMAX_MOE = (("mlp.gate.e_score_correction_bias", "block_sparse_moe.e_score_correction_bias"), ("mlp.gate.weight", "block_sparse_moe.gate.weight"),
                ("gate_proj.weight", "w1.weight"), ("up_proj.weight", "w3.weight"), ("down_proj.weight", "w2.weight"),
                ("mlp.experts.", "block_sparse_moe.experts."))  # fmt: skip


def _family_name(cfg: ModelConfig, hf_name: str) -> str:
    """Checkpoint spelling of a family whose files name the same tensors differently: MiniMax-M2 keeps its experts under
    ``block_sparse_moe`` as w1 (gate) / w3 (up) / w2 (down)
    (slime/backends/megatron_utils/megatron_to_hf/minimax_m2.py:31-84 in the reference)."""
    if _family(cfg) == "minimax" and (".mlp.experts." in hf_name or ".mlp.gate." in hf_name):
        for a, b in _MINIMAX_MOE:
            hf_name = hf_name.replace(a, b)
    return _vl_name(cfg, hf_name)


def family_name_to_generic(hf_name: str) -> str:
    """Inverse of the family spellings above (what an engine that only knows the generic names calls it)."""
    if ".block_sparse_moe." in hf_name:
        for a, b in reversed(_MINIMAX_MOE):
            hf_name = hf_name.replace(b, a)
    return hf_name


def convert_to_hf(cfg: ModelConfig, name: str, t: torch.Tensor) -> list[tuple[str, torch.Tensor]]:
    """One gathered trainer tensor -> HF (name, tensor) pairs. Names not handled raise."""
    name = name.removeprefix("module.").removeprefix("module.")
    if name.startswith("vision."):  # the image encoder keeps the checkpoint's own parameter names
        return [("model.visual." + name[len("vision.") :], t)]
    return [(_family_name(cfg, n), x) for n, x in _text_to_hf(cfg, name, t)]


def _text_to_hf(cfg: ModelConfig, name: str, t: torch.Tensor) -> list[tuple[str, torch.Tensor]]:
    if name == "embedding.word_embeddings.weight":
        return [("model.embed_tokens.weight", t[: cfg.vocab_size])]
    if name == "output_layer.weight":
        return [("lm_head.weight", t[: cfg.vocab_size])]
    if name == "decoder.final_layernorm.weight":
        return [("model.norm.weight", t - 1 if _zero_centred(cfg) else t)]
    mm = _MTP.match(name)
    if mm is not None:
        k, sub = int(mm.group(1)), mm.group(2)
        if _family(cfg) == "mimo":
            # MiMo layout: model.mtp_layers.k.*, the joining projection's column halves in (hidden, embedding) order
            # (slime/backends/megatron_utils/megatron_to_hf/mimo.py:18-75 in the reference)
            p = f"model.mtp_layers.{k}"
            if sub == "eh_proj.weight":
                e_half, h_half = t.chunk(2, dim=1)
                return [(f"{p}.input_proj.weight", torch.cat([h_half, e_half], dim=1))]
            if sub in _MIMO_MTP:
                return [(f"{p}.{_MIMO_MTP[sub]}", t)]
            assert sub.startswith("transformer_layer."), name
            return [(n.replace(f"model.layers.{k}.", f"{p}.", 1), x) for n, x in _layer_to_hf(cfg, str(k), sub[len("transformer_layer.") :], t)]
        if _family(cfg) in ("qwen3next", "qwen3_5"):
            # Qwen3-Next / Qwen3.5 layout: a top-level ``mtp`` block; its norms are stored minus one like all norms of the
            # family, Qwen3-Next keeps the joining projection's halves as (hidden, embedding)
            # (slime/backends/megatron_utils/megatron_to_hf/qwen3_next.py:6-41, qwen3_5.py:6-31 in the reference)
            if sub in _QWEN_MTP:
                return [(_QWEN_MTP[sub], t - 1)]
            if sub == "eh_proj.weight":
                if _family(cfg) == "qwen3next":
                    e_half, h_half = t.chunk(2, dim=1)
                    t = torch.cat([h_half, e_half], dim=1)
                return [("mtp.fc.weight", t)]
            assert sub.startswith("transformer_layer."), name
            out = _layer_to_hf(cfg, str(k), sub[len("transformer_layer.") :], t)
            out = [(n, x - 1 if n.endswith(_ZERO_CENTRED) and ".linear_attn." not in n else x) for n, x in out]
            return [(n.replace(f"model.layers.{k}.", f"mtp.layers.{k}.", 1), x) for n, x in out]
        # DeepSeek-V3 layout: draft depth k is checkpoint layer num_layers + k, with its own norms and projection
        i = str(cfg.num_layers + k)
        p = f"model.layers.{i}"
        own = {"enorm.weight": "enorm.weight", "hnorm.weight": "hnorm.weight", "eh_proj.weight": "eh_proj.weight",
               "final_layernorm.weight": "shared_head.norm.weight"}  # fmt: skip
        if sub in own:
            return [(f"{p}.{own[sub]}", t)]
        assert sub.startswith("transformer_layer."), name
        return _layer_to_hf(cfg, i, sub[len("transformer_layer.") :], t)
    m = _LAYER.match(name)
    if m is None:
        raise ValueError(f"unknown trainer parameter name: {name}")
    i, sub = m.group(1), m.group(2)
    out = _layer_to_hf(cfg, i, sub, t)
    if _zero_centred(cfg):
        out = [(n, x - 1 if n.endswith(_ZERO_CENTRED) and ".linear_attn." not in n else x) for n, x in out]
    return out


def _layer_to_hf(cfg: ModelConfig, i: str, sub: str, t: torch.Tensor) -> list[tuple[str, torch.Tensor]]:
    name = f"decoder.layers.{i}.{sub}"
    p = f"model.layers.{i}"
    fam = _family(cfg)
    if sub.startswith("self_attention."):
        got = _mixer_to_hf(cfg, i, sub[len("self_attention.") :], t)
        if got is not None:
            return got
    if sub == "self_attention.linear_qkv.weight" and cfg.attention_output_gate:
        q, gate, k, v = t.split(_qkv_pieces(cfg), dim=0)
        return [(f"{p}.self_attn.q_proj.weight", _gated_q_to_hf(cfg, q, gate)), (f"{p}.self_attn.k_proj.weight", k),
                (f"{p}.self_attn.v_proj.weight", v)]  # fmt: skip
    if sub == "self_attention.linear_qkv.weight":
        q, k, v = split_qkv(cfg, t)
        return [(f"{p}.self_attn.q_proj.weight", q), (f"{p}.self_attn.k_proj.weight", k), (f"{p}.self_attn.v_proj.weight", v)]
    if sub == "self_attention.linear_qkv.bias":
        q, k, v = split_qkv(cfg, t)
        return [(f"{p}.self_attn.q_proj.bias", q), (f"{p}.self_attn.k_proj.bias", k), (f"{p}.self_attn.v_proj.bias", v)]
    if sub == "self_attention.linear_qkv.layer_norm_weight":
        return [(f"{p}.input_layernorm.weight", t)]
    if sub == "self_attention.linear_proj.weight":
        return [(f"{p}.self_attn.o_proj.weight", t)]
    if sub == "self_attention.q_layernorm.weight":
        return [(f"{p}.self_attn.q_norm.weight", t)]
    if sub == "self_attention.k_layernorm.weight":
        return [(f"{p}.self_attn.k_norm.weight", t)]
    if sub == "post_self_attn_layernorm.weight":
        return [(f"{p}.post_self_attn_layernorm.weight", t)]
    if sub == "post_mlp_layernorm.weight":
        return [(f"{p}.post_mlp_layernorm.weight", t)]
    if sub in ("mlp.linear_fc1.layer_norm_weight", "pre_mlp_layernorm.weight", "mlp.pre_mlp_layernorm.weight"):
        return [(f"{p}.post_attention_layernorm.weight", t)]
    if sub == "mlp.linear_fc1.weight":
        if fam == "glm4":
            return [(f"{p}.mlp.gate_up_proj.weight", t)]
        half = t.shape[0] // 2
        return [(f"{p}.mlp.gate_proj.weight", t[:half]), (f"{p}.mlp.up_proj.weight", t[half:])]
    if sub == "mlp.linear_fc2.weight":
        return [(f"{p}.mlp.down_proj.weight", t)]
    if sub == "mlp.router.weight":
        return [(f"{p}.mlp.gate.weight", t)]
    if sub == "mlp.router.expert_bias":
        return [(f"{p}.mlp.gate.e_score_correction_bias", t)]
    em = _EXPERT.match(sub)
    if em:
        which, e = em.group(1), em.group(2)
        if which == "1":
            half = t.shape[0] // 2
            return [(f"{p}.mlp.experts.{e}.gate_proj.weight", t[:half]), (f"{p}.mlp.experts.{e}.up_proj.weight", t[half:])]
        return [(f"{p}.mlp.experts.{e}.down_proj.weight", t)]
    if sub == "mlp.shared_experts.linear_fc1.weight":
        half = t.shape[0] // 2
        sp = "shared_expert" if fam in ("qwen2moe", "qwen3next", "qwen3_5") else "shared_experts"
        return [(f"{p}.mlp.{sp}.gate_proj.weight", t[:half]), (f"{p}.mlp.{sp}.up_proj.weight", t[half:])]
    if sub == "mlp.shared_experts.linear_fc2.weight":
        sp = "shared_expert" if fam in ("qwen2moe", "qwen3next", "qwen3_5") else "shared_experts"
        return [(f"{p}.mlp.{sp}.down_proj.weight", t)]
    if sub == "mlp.shared_experts.gate_weight":
        return [(f"{p}.mlp.shared_expert_gate.weight", t)]
    raise ValueError(f"unknown trainer parameter name: {name}")


# -------------------------------------------------------------------------- TP gather rules
def gather_dim(name: str, param) -> int | None:
    """Dimension along which TP shards of ``param`` concatenate (None: replicated)."""
    if not getattr(param, "tensor_model_parallel", False):
        return None
    return getattr(param, "partition_dim", 0)


def merge_tp_shards(cfg: ModelConfig, name: str, shards: list[torch.Tensor], partition_dim: int, stride: int) -> torch.Tensor:
    """Concatenate TP shards into the full tensor honouring fused layouts.

    * fused fc1 (stride 2): each shard is [gate_r ; up_r] -> full is [gate_0..gate_n ; up_0..up_n].
    * fused qkv: each shard is [q_r | k_r | v_r] -> full is [q_all | k_all | v_all].
    """
    if len(shards) == 1:
        return shards[0]
    if "linear_qkv" in name and partition_dim == 0:
        pieces = [s.split(_qkv_pieces(cfg, len(shards)), dim=0) for s in shards]  # q, (gate,) k, v of every rank
        return torch.cat([torch.cat([pc[j] for pc in pieces], dim=0) for j in range(len(pieces[0]))], dim=0)
    if stride == 2 and partition_dim == 0:
        halves = [s.chunk(2, dim=0) for s in shards]
        return torch.cat([h[0] for h in halves] + [h[1] for h in halves], dim=0)
    return torch.cat(shards, dim=partition_dim)


def shard_for_tp(cfg: ModelConfig, name: str, full: torch.Tensor, partition_dim: int, stride: int, tp: int, rank: int):
    """Inverse of :func:`merge_tp_shards`: this rank's shard of a full tensor."""
    if tp == 1:
        return full
    if "linear_qkv" in name and partition_dim == 0:
        return torch.cat([piece.chunk(tp, 0)[rank] for piece in full.split(_qkv_pieces(cfg), dim=0)], dim=0)
    if stride == 2 and partition_dim == 0:
        g, u = full.chunk(2, dim=0)
        return torch.cat([g.chunk(tp, 0)[rank], u.chunk(tp, 0)[rank]], dim=0)
    return full.chunk(tp, dim=partition_dim)[rank]


# ---------------------------------------------------------------------- HF -> trainer names
def hf_sources_for(cfg: ModelConfig, name: str) -> tuple[list[str], str]:
    """HF tensor names a trainer parameter is assembled from, and the rule that joins them (``merge_hf_sources``)."""
    if name.startswith("vision."):
        return ["model.visual." + name[len("vision.") :]], "copy"
    names, rule = _text_sources_for(cfg, name)
    return [_family_name(cfg, n) for n in names], rule


def _text_sources_for(cfg: ModelConfig, name: str) -> tuple[list[str], str]:
    """HF tensor names needed to build trainer tensor ``name`` and the merge rule
    ('copy' | 'qkv' | 'gate_up')."""
    if name == "embedding.word_embeddings.weight":
        return ["model.embed_tokens.weight"], "copy"
    if name == "output_layer.weight":
        return ["model.embed_tokens.weight" if cfg.tie_word_embeddings else "lm_head.weight"], "copy"
    if name == "decoder.final_layernorm.weight":
        return ["model.norm.weight"], "copy+1" if _zero_centred(cfg) else "copy"
    mm = _MTP.match(name)
    if mm is not None:
        k, sub = int(mm.group(1)), mm.group(2)
        if _family(cfg) == "mimo":
            p = f"model.mtp_layers.{k}"
            if sub == "eh_proj.weight":
                return [f"{p}.input_proj.weight"], "swap_halves"
            if sub in _MIMO_MTP:
                return [f"{p}.{_MIMO_MTP[sub]}"], "copy"
            names, rule = _text_sources_for(cfg, f"decoder.layers.{k}.{sub[len('transformer_layer.'):]}")
            return [n.replace(f"model.layers.{k}.", f"{p}.", 1) for n in names], rule
        if _family(cfg) in ("qwen3next", "qwen3_5"):
            if sub in _QWEN_MTP:
                return [_QWEN_MTP[sub]], "copy+1"
            if sub == "eh_proj.weight":
                return ["mtp.fc.weight"], "swap_halves" if _family(cfg) == "qwen3next" else "copy"
            names, rule = _text_sources_for(cfg, f"decoder.layers.{k}.{sub[len('transformer_layer.'):]}")
            return [n.replace(f"model.layers.{k}.", f"mtp.layers.{k}.", 1) for n in names], rule
        p = f"model.layers.{cfg.num_layers + k}"
        own = {"enorm.weight": "enorm.weight", "hnorm.weight": "hnorm.weight", "eh_proj.weight": "eh_proj.weight",
               "final_layernorm.weight": "shared_head.norm.weight"}  # fmt: skip
        if sub in own:
            return [f"{p}.{own[sub]}"], "copy"
        return _text_sources_for(cfg, f"decoder.layers.{cfg.num_layers + k}.{sub[len('transformer_layer.'):]}")
    m = _LAYER.match(name)
    if m is None:
        raise ValueError(f"unknown trainer parameter name: {name}")
    i, sub = m.group(1), m.group(2)
    p = f"model.layers.{i}"
    simple = {
        "self_attention.linear_qkv.layer_norm_weight": "input_layernorm.weight",
        "self_attention.linear_proj.weight": "self_attn.o_proj.weight",
        "self_attention.q_layernorm.weight": "self_attn.q_norm.weight",
        "self_attention.k_layernorm.weight": "self_attn.k_norm.weight",
        "mlp.linear_fc1.layer_norm_weight": "post_attention_layernorm.weight",
        "pre_mlp_layernorm.weight": "post_attention_layernorm.weight",
        "mlp.pre_mlp_layernorm.weight": "post_attention_layernorm.weight",
        "mlp.linear_fc2.weight": "mlp.down_proj.weight",
        "mlp.router.weight": "mlp.gate.weight",
        "mlp.router.expert_bias": "mlp.gate.e_score_correction_bias",
        "post_self_attn_layernorm.weight": "post_self_attn_layernorm.weight",
        "post_mlp_layernorm.weight": "post_mlp_layernorm.weight",
    }
    plus1 = "+1" if _zero_centred(cfg) else ""
    if sub.startswith("self_attention."):
        inner = sub[len("self_attention.") :]
        if inner == "q_layernorm.weight" and cfg.multi_latent_attention:
            return [f"{p}.self_attn.q_a_layernorm.weight"], "copy"
        if inner in _MIXER_NAMES and not (inner == "input_layernorm.weight" and cfg.mixer(int(i)) == "attention"):
            rule = "conv" if inner == "conv1d.weight" else ("copy" + plus1 if inner == "input_layernorm.weight" else "copy")
            return [f"{p}.{_MIXER_NAMES[inner]}"], rule
    if sub in simple:
        norm = simple[sub].endswith(_ZERO_CENTRED)
        return [f"{p}.{simple[sub]}"], "copy" + (plus1 if norm else "")
    if sub == "self_attention.linear_qkv.weight" and cfg.attention_output_gate:
        return [f"{p}.self_attn.{x}_proj.weight" for x in "qkv"], "gated_qkv"
    if sub == "self_attention.linear_qkv.weight":
        return [f"{p}.self_attn.{x}_proj.weight" for x in "qkv"], "qkv"
    if sub == "self_attention.linear_qkv.bias":
        return [f"{p}.self_attn.{x}_proj.bias" for x in "qkv"], "qkv"
    if sub == "mlp.linear_fc1.weight":
        if _family(cfg) == "glm4":  # GLM-4 dense checkpoints store the fused [gate; up] matrix
            return [f"{p}.mlp.gate_up_proj.weight"], "copy"
        return [f"{p}.mlp.gate_proj.weight", f"{p}.mlp.up_proj.weight"], "gate_up"
    sp = "shared_expert" if _family(cfg) in ("qwen2moe", "qwen3next", "qwen3_5") else "shared_experts"
    if sub == "mlp.shared_experts.linear_fc1.weight":
        return [f"{p}.mlp.{sp}.gate_proj.weight", f"{p}.mlp.{sp}.up_proj.weight"], "gate_up"
    if sub == "mlp.shared_experts.linear_fc2.weight":
        return [f"{p}.mlp.{sp}.down_proj.weight"], "copy"
    if sub == "mlp.shared_experts.gate_weight":
        return [f"{p}.mlp.shared_expert_gate.weight"], "copy"
    em = _EXPERT.match(sub)
    if em:
        which, e = em.group(1), em.group(2)
        if which == "1":
            return [f"{p}.mlp.experts.{e}.gate_proj.weight", f"{p}.mlp.experts.{e}.up_proj.weight"], "gate_up"
        return [f"{p}.mlp.experts.{e}.down_proj.weight"], "copy"
    raise ValueError(f"unknown trainer parameter name: {name}")


def merge_hf_sources(rule: str, tensors: list[torch.Tensor], cfg: ModelConfig | None = None) -> torch.Tensor:
    if rule == "copy":
        return tensors[0]
    if rule == "copy+1":  # zero-centred norm weight -> effective weight
        return tensors[0] + 1
    if rule == "swap_halves":  # MiMo's joining projection: (hidden, embedding) columns -> (embedding, hidden)
        a, b = tensors[0].chunk(2, dim=1)
        return torch.cat([b, a], dim=1)
    if rule == "conv":  # depthwise Conv1d weight [C, 1, K] -> [C, K]
        return tensors[0].squeeze(1)
    if rule == "gated_qkv":  # q_proj rows are per head (query, gate)
        q, gate = _gated_q_from_hf(cfg, tensors[0])
        return torch.cat([q, gate, tensors[1], tensors[2]], dim=0)
    return torch.cat(tensors, dim=0)  # qkv -> [q|k|v], gate_up -> [gate;up]


def pad_vocab(t: torch.Tensor, padded: int) -> torch.Tensor:
    if t.shape[0] >= padded:
        return t[:padded]
    return torch.cat([t, t.new_zeros(padded - t.shape[0], *t.shape[1:])], dim=0)
