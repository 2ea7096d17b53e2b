"""Quantise a Hugging Face bf16 checkpoint to fp8 (e4m3) weights with fp32 scales.

    python -m slime_b200.tools.convert_hf_to_fp8 --model-dir /ckpt/Qwen3-30B-A3B --save-dir /ckpt/Qwen3-30B-A3B-FP8 \\
        --strategy block --block-size 128 128

``block``: one scale per 128x128 tile, ``weight_scale_inv[i, j] = max|W_tile| / 448`` (clamped at 1e-12), stored as
``<name>_scale_inv``; ``channel``: one scale per output row (``<name>_scale``); ``tensor``: one scale. Only 2-D linear
weights of attention / MLP / experts are quantised; embeddings, norms, the LM head, routers (gates) and biases stay in
bf16. ``config.json`` gains the matching ``quantization_config``. On a GPU the block strategy runs the same kernel the
weight-sync path uses (``ops.block_fp8_quant``). Parity: tools/convert_hf_to_fp8.py:30-269.
"""

from __future__ import annotations

import argparse
import json
import os
import shutil

import torch

FP8_MAX = torch.finfo(torch.float8_e4m3fn).max
SKIP_SUBSTRINGS = ("embed_tokens", "lm_head", "norm", "mlp.gate.", "router", "e_score_correction_bias", "indexer.weights_proj")


def block_fp8(w: torch.Tensor, block=(128, 128)):
    from slime_b200 import ops

    if w.is_cuda and tuple(block) == (128, 128) and w.dtype == torch.bfloat16:
        return ops.block_fp8_quant(w, block)
    bn, bk = block
    n, k = w.shape
    tn, tk = -(-n // bn), -(-k // bk)
    pad = torch.nn.functional.pad(w.float(), (0, tk * bk - k, 0, tn * bn - n)).reshape(tn, bn, tk, bk)
    scale = pad.abs().amax(dim=(1, 3), keepdim=True).clamp(min=1e-12) / FP8_MAX
    q = (pad / scale).clamp(-FP8_MAX, FP8_MAX).reshape(tn * bn, tk * bk)[:n, :k].to(torch.float8_e4m3fn)
    return q.contiguous(), scale.reshape(tn, tk)


def channel_fp8(w: torch.Tensor):
    scale = w.float().abs().amax(dim=-1, keepdim=True).clamp(min=1e-12) / FP8_MAX
    return (w.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), scale


def tensor_fp8(w: torch.Tensor):
    scale = w.float().abs().max().clamp(min=1e-12) / FP8_MAX
    return (w.float() / scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn), scale.view(1)


def should_quantise(name: str, t: torch.Tensor) -> bool:
    return name.endswith(".weight") and t.dim() == 2 and not any(s in name for s in SKIP_SUBSTRINGS)


def convert(model_dir: str, save_dir: str, strategy: str = "block", block=(128, 128), device: str | None = None) -> dict:
    from safetensors import safe_open
    from safetensors.torch import save_file

    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    os.makedirs(save_dir, exist_ok=True)
    weight_map, kept_bf16 = {}, []
    files = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    for fname in files:
        out = {}
        with safe_open(os.path.join(model_dir, fname), framework="pt") as f:
            for name in f.keys():
                t = f.get_tensor(name)
                if not should_quantise(name, t):
                    out[name] = t
                    if name.endswith(".weight") and t.dim() == 2:
                        kept_bf16.append(name[: -len(".weight")])
                    continue
                w = t.to(device)
                if strategy == "block":
                    q, s = block_fp8(w, block)
                    out[name], out[name + "_scale_inv"] = q.cpu(), s.float().cpu()
                elif strategy == "channel":
                    q, s = channel_fp8(w)
                    out[name], out[name + "_scale"] = q.cpu(), s.float().cpu()
                else:
                    q, s = tensor_fp8(w)
                    out[name], out[name + "_scale"] = q.cpu(), s.float().cpu()
        save_file({k: v.contiguous() for k, v in out.items()}, os.path.join(save_dir, fname), metadata={"format": "pt"})
        weight_map.update({k: fname for k in out})
    with open(os.path.join(save_dir, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f, indent=2)
    for fn in os.listdir(model_dir):
        src = os.path.join(model_dir, fn)
        if os.path.isfile(src) and not fn.endswith(".safetensors") and fn != "model.safetensors.index.json":
            shutil.copyfile(src, os.path.join(save_dir, fn))
    cfg_path = os.path.join(save_dir, "config.json")
    cfg = json.load(open(cfg_path)) if os.path.exists(cfg_path) else {}
    qc = {"quant_method": "fp8", "fmt": "e4m3", "activation_scheme": "dynamic", "modules_to_not_convert": sorted(set(kept_bf16))}
    if strategy == "block":
        qc["weight_block_size"] = list(block)
    else:
        qc["strategy"] = strategy
    cfg["quantization_config"] = qc
    with open(cfg_path, "w") as f:
        json.dump(cfg, f, indent=2)
    return weight_map


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--model-dir", required=True)
    p.add_argument("--save-dir", required=True)
    p.add_argument("--strategy", choices=["block", "channel", "tensor"], default="block")
    p.add_argument("--block-size", type=int, nargs=2, default=[128, 128])
    p.add_argument("--device", default=None)
    a = p.parse_args(argv)
    wm = convert(a.model_dir, a.save_dir, a.strategy, tuple(a.block_size), a.device)
    print(f"wrote {len(wm)} tensors to {a.save_dir}")


if __name__ == "__main__":
    main()
