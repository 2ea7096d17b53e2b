"""Round-to-nearest INT4 (W4A16, compressed-tensors ``pack-quantized``) conversion of a Hugging Face checkpoint.

    python -m slime_b200.tools.convert_hf_to_int4_direct --model-dir /ckpt/moe-bf16 --save-dir /ckpt/moe-int4 --group-size 32

Symmetric, one scale per group of ``--group-size`` input channels (scale = absmax / 7, codes = round(w / scale) in [-8, 7]),
eight codes packed per int32 (``<name>_packed``), scales in bf16 (``<name>_scale``) and the original shape
(``<name>_shape``). By default only routed-expert weights are quantised (the bulk of a MoE model); attention, shared
experts, dense MLPs, routers, embeddings, norms and the LM head stay bf16 -- the same ignore list a calibrated GPTQ run
would use. No calibration data is needed, which is what makes this the variant used inside weight sync.
Parity: tools/convert_hf_to_int4_direct.py:1-326 (and the ignore list of tools/convert_hf_to_int4.py:72-80).
"""

from __future__ import annotations

import argparse
import json
import os
import re
import shutil

import torch

DEFAULT_IGNORE = [r".*lm_head.*", r".*norm.*", r".*embed.*", r".*self_attn.*", r".*shared_experts.*",
                  r".*mlp\.(gate|up|gate_up|down)_proj.*", r".*mlp\.gate\..*"]  # fmt: skip


def quantise_weight(w: torch.Tensor, group_size: int):
    from slime_b200.weight_sync.quantizer import quantize_param_int4

    return quantize_param_int4("w.weight", w, group_size)


def convert(model_dir: str, save_dir: str, group_size: int = 32, ignore=None, device: str | None = None) -> dict:
    from safetensors import safe_open
    from safetensors.torch import save_file

    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    ignore = [re.compile(p) for p in (DEFAULT_IGNORE if ignore is None else ignore)]
    os.makedirs(save_dir, exist_ok=True)
    weight_map, n_q = {}, 0
    for fname in sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors")):
        out = {}
        with safe_open(os.path.join(model_dir, fname), framework="pt") as f:
            for name in f.keys():
                t = f.get_tensor(name)
                if not (name.endswith(".weight") and t.dim() == 2 and t.shape[1] % max(group_size, 8) == 0) or any(
                        p.fullmatch(name) for p in ignore):  # fmt: skip
                    out[name] = t
                    continue
                for k, v in quantise_weight(t.to(device), group_size):
                    out[name[: -len("weight")] + k.split(".", 1)[1]] = v.cpu()
                n_q += 1
        save_file({k: v.contiguous() for k, v in out.items()}, os.path.join(save_dir, fname), metadata={"format": "pt"})
        weight_map.update({k: fname for k in out})
    with open(os.path.join(save_dir, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f, indent=2)
    for fn in os.listdir(model_dir):
        p = os.path.join(model_dir, fn)
        if os.path.isfile(p) and not fn.endswith(".safetensors") and fn != "model.safetensors.index.json":
            shutil.copyfile(p, os.path.join(save_dir, fn))
    cfg_path = os.path.join(save_dir, "config.json")
    cfg = json.load(open(cfg_path)) if os.path.exists(cfg_path) else {}
    cfg["quantization_config"] = {
        "quant_method": "compressed-tensors", "format": "pack-quantized",
        "config_groups": {"group_0": {"targets": ["Linear"], "weights": {
            "num_bits": 4, "type": "int", "symmetric": True, "strategy": "group", "group_size": group_size}}},
        "ignore": [p.pattern for p in ignore],
    }  # fmt: skip
    with open(cfg_path, "w") as f:
        json.dump(cfg, f, indent=2)
    return {"tensors": len(weight_map), "quantised": n_q}


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--model-dir", required=True)
    p.add_argument("--save-dir", required=True)
    p.add_argument("--group-size", type=int, default=32)
    p.add_argument("--ignore", nargs="*", default=None, help="regexes of tensor names to keep in bf16")
    p.add_argument("--device", default=None)
    a = p.parse_args(argv)
    print(convert(a.model_dir, a.save_dir, a.group_size, a.ignore, a.device))


if __name__ == "__main__":
    main()
