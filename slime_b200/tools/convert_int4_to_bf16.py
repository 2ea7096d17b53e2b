"""Undo W4A16 ``pack-quantized`` compression of a Hugging Face checkpoint: packed INT4 codes + group scales -> bf16 weights.

    python -m slime_b200.tools.convert_int4_to_bf16 --model-dir /ckpt/Kimi-K2-Thinking --save-dir /ckpt/Kimi-K2-Thinking-bf16

For checkpoints that ship their expert weights as compressed-tensors INT4 (``<name>.weight_packed`` int32 with eight
codes per word, ``<name>.weight_scale``, ``<name>.weight_shape``), which the trainer cannot load directly: every such
triple becomes ``<name>.weight`` in bf16, everything else is copied, and ``quantization_config`` is dropped from
``config.json``. Codes are stored with an offset of 8 (element i of a word at bits [4i, 4i + 4)); the group size follows
from the shapes of the codes and the scales. Same role as tools/convert_k2_thinking_int4_to_bf16.py in the reference.
"""

from __future__ import annotations

import argparse
import json
import os
import shutil

import torch


def unpack_int4(packed: torch.Tensor, scale: torch.Tensor, shape) -> torch.Tensor:
    """``packed`` [N, K/8] int32, ``scale`` [N, K/group] -> [N, K] bf16."""
    n, k = int(shape[0]), int(shape[1])
    shifts = torch.arange(0, 32, 4, device=packed.device, dtype=torch.int32)
    codes = (((packed.to(torch.int32)[..., None] >> shifts) & 0xF) - 8).reshape(n, -1)[:, :k].float()
    group = k // scale.shape[1]
    return (codes.view(n, -1, group) * scale.float()[..., None]).view(n, k).to(torch.bfloat16)


def convert(model_dir: str, save_dir: str, device: str | None = None) -> dict:
    from safetensors import safe_open
    from safetensors.torch import save_file

    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    os.makedirs(save_dir, exist_ok=True)
    weight_map, restored = {}, 0
    files = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    # a triple may be split over files: index every tensor first
    where = {}
    for fname in files:
        with safe_open(os.path.join(model_dir, fname), framework="pt") as f:
            for name in f.keys():
                where[name] = fname

    def fetch(name):
        with safe_open(os.path.join(model_dir, where[name]), framework="pt") as f:
            return f.get_tensor(name)

    for fname in files:
        out = {}
        with safe_open(os.path.join(model_dir, fname), framework="pt") as f:
            for name in f.keys():
                if name.endswith(".weight_scale") or name.endswith(".weight_shape"):
                    base = name.rsplit(".weight_", 1)[0]
                    if f"{base}.weight_packed" in where:
                        continue  # consumed with its packed partner
                if name.endswith(".weight_packed"):
                    base = name[: -len(".weight_packed")]
                    w = unpack_int4(f.get_tensor(name).to(device), fetch(f"{base}.weight_scale").to(device), fetch(f"{base}.weight_shape").tolist())
                    out[f"{base}.weight"] = w.cpu()
                    restored += 1
                else:
                    out[name] = f.get_tensor(name)
        save_file({k: v.contiguous() for k, v in out.items()}, os.path.join(save_dir, fname), metadata={"format": "pt"})
        weight_map.update({k: fname for k in out})
    with open(os.path.join(save_dir, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f, indent=2)
    for fn in os.listdir(model_dir):
        p = os.path.join(model_dir, fn)
        if os.path.isfile(p) and not fn.endswith(".safetensors") and fn != "model.safetensors.index.json":
            shutil.copyfile(p, os.path.join(save_dir, fn))
    cfg_path = os.path.join(save_dir, "config.json")
    if os.path.exists(cfg_path):
        cfg = json.load(open(cfg_path))
        cfg.pop("quantization_config", None)
        cfg["torch_dtype"] = "bfloat16"
        with open(cfg_path, "w") as f:
            json.dump(cfg, f, indent=2)
    return {"tensors": len(weight_map), "restored": restored}


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--model-dir", required=True)
    p.add_argument("--save-dir", required=True)
    p.add_argument("--device", default=None)
    a = p.parse_args(argv)
    print(convert(a.model_dir, a.save_dir, a.device))


if __name__ == "__main__":
    main()
