"""Block-fp8 checkpoint -> bf16 checkpoint: ``W = q * scale_inv[tile]`` for every tensor that has a ``_scale_inv``.

    python -m slime_b200.tools.fp8_cast_bf16 --input-fp8-hf-path /ckpt/model-FP8 --output-bf16-hf-path /ckpt/model-bf16

The ``quantization_config`` entry is removed from ``config.json``. On a GPU the dequantisation runs the
``block_fp8_dequant`` kernel of this package. Parity: tools/fp8_cast_bf16.py:1-117.
"""

from __future__ import annotations

import argparse
import json
import os
import shutil

import torch


def dequant(q: torch.Tensor, scale_inv: torch.Tensor, block=(128, 128)) -> torch.Tensor:
    from slime_b200 import ops

    if q.is_cuda:
        return ops.block_fp8_dequant(q, scale_inv, block)
    n, k = q.shape
    s = scale_inv.float().repeat_interleave(block[0], 0)[:n].repeat_interleave(block[1], 1)[:, :k]
    return (q.float() * s).to(torch.bfloat16)


def convert(src: str, dst: str, device: str | None = None) -> int:
    from safetensors import safe_open
    from safetensors.torch import save_file

    from slime_b200.checkpoint.hf_loader import SafetensorReader

    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    os.makedirs(dst, exist_ok=True)
    cfg = json.load(open(os.path.join(src, "config.json")))
    block = tuple((cfg.get("quantization_config") or {}).get("weight_block_size") or (128, 128))
    reader = SafetensorReader(src)  # scales may sit in a different shard than their weight
    weight_map, n = {}, 0
    for fname in sorted(f for f in os.listdir(src) if f.endswith(".safetensors")):
        out = {}
        with safe_open(os.path.join(src, fname), framework="pt") as f:
            for name in f.keys():
                if name.endswith("_scale_inv"):
                    continue
                t = f.get_tensor(name)
                if t.dtype == torch.float8_e4m3fn and (name + "_scale_inv") in reader:
                    t = dequant(t.to(device), reader.get(name + "_scale_inv").to(device), block).cpu()
                    n += 1
                out[name] = t.contiguous()
        save_file(out, os.path.join(dst, fname), metadata={"format": "pt"})
        weight_map.update({k: fname for k in out})
    with open(os.path.join(dst, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f, indent=2)
    for fn in os.listdir(src):
        p = os.path.join(src, fn)
        if os.path.isfile(p) and not fn.endswith(".safetensors") and fn != "model.safetensors.index.json":
            shutil.copyfile(p, os.path.join(dst, fn))
    cfg.pop("quantization_config", None)
    with open(os.path.join(dst, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    return n


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--input-fp8-hf-path", required=True)
    p.add_argument("--output-bf16-hf-path", required=True)
    p.add_argument("--device", default=None)
    a = p.parse_args(argv)
    print(f"dequantised {convert(a.input_fp8_hf_path, a.output_bf16_hf_path, a.device)} tensors")


if __name__ == "__main__":
    main()
