"""Native ``torch_dist`` checkpoint -> Hugging Face safetensors directory.

    python -m slime_b200.tools.convert_torch_dist_to_hf --input-dir /ckpt/run/iter_0000100 --output-dir /ckpt/hf_100 \\
        --origin-hf-dir /ckpt/Qwen3-4B

Single process: the DCP shards are read tensor by tensor (no model is built, nothing needs a GPU), renamed and re-laid
out (fused qkv de-interleaved, gate/up split, experts unstacked) and written in shards of ``--chunk-size`` bytes with a
``model.safetensors.index.json``. Config and tokenizer files are copied from ``--origin-hf-dir``. Vocabulary padding
rows are dropped. Parity: tools/convert_torch_dist_to_hf.py:1-244.
"""

from __future__ import annotations

import argparse
import json
import os
import shutil

import torch


def _load_common_args(input_dir: str):
    path = os.path.join(input_dir, "common.pt")
    if os.path.exists(path):
        return torch.load(path, weights_only=False).get("args")
    return None


def convert(input_dir: str, output_dir: str, origin_hf_dir: str | None, chunk_size: int = 5 * 1024**3, vocab_size: int | None = None):
    from safetensors.torch import save_file

    from slime_b200.backends.train.checkpoint import _dcp_load, _read_dcp_keys
    from slime_b200.models.config import ModelConfig
    from slime_b200.weight_sync import convert as cv

    if origin_hf_dir:
        cfg = ModelConfig.from_hf(origin_hf_dir)
    else:
        cfg = ModelConfig.from_args(_load_common_args(input_dir))
    if vocab_size:
        cfg.vocab_size = vocab_size
    meta = _read_dcp_keys(input_dir)
    names = sorted(k for k in meta if not k.startswith("optimizer.") and not k.startswith("rng"))
    os.makedirs(output_dir, exist_ok=True)
    weight_map, shard, used, n_shards = {}, {}, 0, 0
    files = []

    def flush():
        nonlocal shard, used, n_shards
        if not shard:
            return
        n_shards += 1
        fname = f"model-{n_shards:05d}.safetensors"
        save_file({k: v.contiguous() for k, v in shard.items()}, os.path.join(output_dir, fname), metadata={"format": "pt"})
        files.append((fname, list(shard)))
        shard, used = {}, 0

    for name in names:
        spec = meta[name]
        t = torch.empty(spec.size, dtype=spec.properties.dtype)
        _dcp_load(input_dir, {name: t})
        key = name[len("model.") :] if name.startswith("model.") else name
        if key == "output_layer.weight" and cfg.tie_word_embeddings:
            continue
        if key.endswith("linear_qkv.weight") or key.endswith("linear_qkv.bias"):
            t = cv.qkv_from_megatron_layout(cfg, t)  # the checkpoint interleaves q/k/v per kv group
        for hf_name, ht in cv.convert_to_hf(cfg, key, t):
            if hf_name in ("model.embed_tokens.weight", "lm_head.weight"):
                ht = ht[: cfg.vocab_size]
            nbytes = ht.numel() * ht.element_size()
            if shard and used + nbytes > chunk_size:
                flush()
            shard[hf_name] = ht
            used += nbytes
    flush()
    total = len(files)
    for i, (fname, keys) in enumerate(files, 1):
        final = f"model-{i:05d}-of-{total:05d}.safetensors"
        os.replace(os.path.join(output_dir, fname), os.path.join(output_dir, final))
        for k in keys:
            weight_map[k] = final
    with open(os.path.join(output_dir, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f, indent=2)
    if origin_hf_dir:
        for fn in os.listdir(origin_hf_dir):
            if fn.endswith(".safetensors") or fn == "model.safetensors.index.json":
                continue
            src = os.path.join(origin_hf_dir, fn)
            if os.path.isfile(src):
                shutil.copyfile(src, os.path.join(output_dir, fn))
    else:
        with open(os.path.join(output_dir, "config.json"), "w") as f:
            json.dump(cfg.to_hf_dict(), f, indent=2)
    return weight_map


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--input-dir", required=True, help="an iter_NNNNNNN or release directory")
    p.add_argument("--output-dir", required=True)
    p.add_argument("--origin-hf-dir", default=None, help="config / tokenizer files are copied from here")
    p.add_argument("--chunk-size", type=int, default=5 * 1024**3)
    p.add_argument("--vocab-size", type=int, default=None)
    p.add_argument("-f", "--force", action="store_true")
    a = p.parse_args(argv)
    if os.path.exists(a.output_dir) and os.listdir(a.output_dir) and not a.force:
        raise SystemExit(f"{a.output_dir} is not empty (use --force)")
    wm = convert(a.input_dir, a.output_dir, a.origin_hf_dir, a.chunk_size, a.vocab_size)
    print(f"wrote {len(wm)} tensors to {a.output_dir}")


if __name__ == "__main__":
    main()
