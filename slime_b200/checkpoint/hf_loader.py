"""Load Hugging Face safetensors straight into the trainer's local shards.

``SafetensorReader`` resolves tensors through ``model.safetensors.index.json`` (or by scanning
``*.safetensors``) and dequantises block-FP8 checkpoints on the fly (``<w>`` e4m3 +
``<w>_scale_inv`` fp32, 128x128 blocks). Each trainer parameter is assembled from its HF sources
(q/k/v -> fused qkv, gate/up -> fused fc1), vocab-padded and TP-sharded with the GLU / fused-qkv
rules. Parity: slime/backends/megatron_utils/hf_to_megatron/common.py:13-167, qwen.py:56-129.
"""

from __future__ import annotations

import glob
import json
import os

import torch

from slime_b200.parallel import state as mpu
from slime_b200.weight_sync import convert


class SafetensorReader:
    def __init__(self, path: str):
        from safetensors import safe_open

        self.path, self._open = path, safe_open
        self.index: dict[str, str] = {}
        idx = os.path.join(path, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                self.index = json.load(f)["weight_map"]
        else:
            for fn in sorted(glob.glob(os.path.join(path, "*.safetensors"))):
                with safe_open(fn, framework="pt") as f:
                    for k in f.keys():
                        self.index[k] = os.path.basename(fn)
        self._handles = {}

    def keys(self):
        return self.index.keys()

    def __contains__(self, name):
        if name in self.index:
            return True
        stacked = convert.stacked_expert_source(name)  # files that keep a layer's experts in one tensor
        return stacked is not None and stacked[0] in self.index

    def _file(self, name):
        fn = self.index[name]
        if fn not in self._handles:
            self._handles[fn] = self._open(os.path.join(self.path, fn), framework="pt")
        return self._handles[fn]

    def get(self, name: str, cfg=None) -> torch.Tensor:
        if name not in self.index:
            stacked, e, part = convert.stacked_expert_source(name)
            if cfg is None:
                raise KeyError(f"{name} is held in the stacked tensor {stacked}: pass the model configuration to slice it")
            sl = self._file(stacked).get_slice(stacked)
            one = sl[e : e + 1]  # one expert's block only: the stack of a layer can be gigabytes
            return dict(convert.split_stacked_experts(cfg, stacked, one))[name.replace(f".experts.{e}.", ".experts.0.")].contiguous()
        t = self._file(name).get_tensor(name)
        scale_name = name + "_scale_inv"
        if t.dtype == torch.float8_e4m3fn and scale_name in self.index:
            from slime_b200.ops import reference

            s = self._file(scale_name).get_tensor(scale_name)
            t = reference.block_fp8_dequant(t, s, (128, 128), torch.bfloat16)
        return t


def supports_hf_weight_loading(path: str) -> bool:
    try:
        with open(os.path.join(path, "config.json")) as f:
            arch = (json.load(f).get("architectures") or [""])[0].lower()
    except OSError:
        return False
    return any(k in arch for k in ("qwen2", "qwen3", "llama", "glm", "mimo", "minimax", "deepseek", "kimi"))


@torch.no_grad()
def load_hf_weights(path: str, model) -> list[str]:
    reader = SafetensorReader(path)
    cfg = model.cfg
    tp, tpr = mpu.get_tensor_model_parallel_world_size(), mpu.get_tensor_model_parallel_rank()
    ep, epr = mpu.get_expert_model_parallel_world_size(), mpu.get_expert_model_parallel_rank()
    missing = []
    from slime_b200.backends.train.checkpoint import global_param_name

    # parameters, and the buffers a checkpoint carries (the router's score-correction bias)
    tensors = list(model.named_parameters()) + [(n, b) for n, b in model.named_buffers() if n.endswith("expert_bias")]
    for name, p in tensors:
        gname = global_param_name(name, p)
        try:
            sources, rule = convert.hf_sources_for(cfg, gname)
        except ValueError:
            missing.append(name)
            continue
        if not all(s in reader for s in sources):
            missing.append(name)
            continue
        full = convert.merge_hf_sources(rule, [reader.get(s, cfg) for s in sources], cfg)
        if name in ("embedding.word_embeddings.weight", "output_layer.weight"):
            full = convert.pad_vocab(full, cfg.padded_vocab_size)
        if getattr(p, "tensor_model_parallel", False) and tp > 1 and not getattr(p, "is_expert", False):
            full = convert.shard_for_tp(cfg, name, full, p.partition_dim, getattr(p, "partition_stride", 1), tp, tpr)
        assert full.shape == p.shape, f"{name}: HF-derived shape {tuple(full.shape)} != {tuple(p.shape)}"
        p.copy_(full.to(p.device, p.dtype))
    return missing
