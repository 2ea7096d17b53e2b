"""Layer-by-layer tensor dumps of a forward pass, and a comparison of two dump folders.

For chasing a train / rollout mismatch down to the layer where it starts: the trainer (and the rollout engine's model
runner, which exposes the same per-layer call) records the output of every selected layer into
``<dump_dir>/<prefix>rank<r>/layer<i>.pt``; ``compare`` walks two such folders and reports, per layer, the largest and
the mean absolute difference and the first layer whose difference exceeds a threshold.

    SLIME_B200_LAYERWISE_DUMP_DIR=/tmp/dump SLIME_B200_LAYERWISE_DUMP_LAYERS=0,1,23 python train.py ...
    python -m slime_b200.observability.layerwise_dump /tmp/dump/actor_rank0 /tmp/dump/engine_rank0

Only the first forward pass after ``enable`` is recorded per layer (a dump of every micro-batch would be useless and
huge). Same role as slime/backends/megatron_utils/alignment/layerwise_alignment.py:42-145 and the engine-side
debug_utils/tensor_dump_forward_hook.py of the reference's SGLang patch.
"""

from __future__ import annotations

import os
import sys

import torch


def _first_tensor(value):
    if torch.is_tensor(value):
        return value
    if isinstance(value, (list, tuple)):
        for v in value:
            t = _first_tensor(v)
            if t is not None:
                return t
    return None


class LayerDump:
    def __init__(self, dump_dir: str, layers: set[int] | None, prefix: str = ""):
        rank = int(os.environ.get("RANK", "0"))
        self.dir = os.path.join(dump_dir, f"{prefix}rank{rank}")
        os.makedirs(self.dir, exist_ok=True)
        self.layers, self.seen, self.handles = layers, set(), []

    def record(self, layer: int, output, residual=None):
        """Store the layer's hidden state (output plus the residual stream it will be added to, when given)."""
        if (self.layers is not None and layer not in self.layers) or layer in self.seen:
            return
        t = _first_tensor(output)
        if t is None:
            return
        self.seen.add(layer)
        h = t.detach().float()
        if residual is not None:
            h = h + residual.detach().float()
        torch.save({"layer": layer, "hidden": h.cpu()}, os.path.join(self.dir, f"layer{layer}.pt"))

    def register(self, model_chunk) -> int:
        """Forward hooks on every transformer layer of a trainer model chunk; returns how many were hooked."""
        n = 0
        for layer in model_chunk.decoder.layers:
            idx = layer.layer_number

            def hook(_m, _args, out, idx=idx):
                res = out[1] if isinstance(out, (list, tuple)) and len(out) > 1 and torch.is_tensor(out[1]) else None
                self.record(idx, out, res)

            self.handles.append(layer.register_forward_hook(hook))
            n += 1
        return n

    def remove(self):
        for h in self.handles:
            h.remove()
        self.handles = []


def enable_from_env(model, prefix: str = "") -> LayerDump | None:
    """Install the dump on a ``TrainModel`` when ``SLIME_B200_LAYERWISE_DUMP_DIR`` is set."""
    d = os.environ.get("SLIME_B200_LAYERWISE_DUMP_DIR")
    if not d:
        return None
    sel = os.environ.get("SLIME_B200_LAYERWISE_DUMP_LAYERS", "")
    layers = {int(x) for x in sel.split(",") if x.strip()} or None
    dump = LayerDump(d, layers, prefix)
    for chunk in getattr(model, "chunks", [model]):
        dump.register(chunk)
    return dump


def compare(dir_a: str, dir_b: str, threshold: float = 1e-2) -> list[dict]:
    rows = []
    names = sorted((n for n in os.listdir(dir_a) if n.startswith("layer") and os.path.exists(os.path.join(dir_b, n))),
                   key=lambda n: int(n[5:-3]))  # fmt: skip
    for n in names:
        a, b = torch.load(os.path.join(dir_a, n))["hidden"], torch.load(os.path.join(dir_b, n))["hidden"]
        rows_n = min(a.shape[0], b.shape[0])
        d = (a[:rows_n] - b[:rows_n]).abs()
        rows.append({"layer": int(n[5:-3]), "max_abs": float(d.max()), "mean_abs": float(d.mean()),
                     "ref_mean_abs": float(a[:rows_n].abs().mean()), "over": bool(d.max() > threshold)})  # fmt: skip
    return rows


def main(argv=None) -> int:
    argv = argv if argv is not None else sys.argv[1:]
    if len(argv) < 2:
        print("usage: python -m slime_b200.observability.layerwise_dump <dump dir A> <dump dir B> [threshold]")
        return 2
    rows = compare(argv[0], argv[1], float(argv[2]) if len(argv) > 2 else 1e-2)
    for r in rows:
        print(f"layer {r['layer']:3d}  max |a-b| {r['max_abs']:.3e}  mean {r['mean_abs']:.3e}  (mean |a| {r['ref_mean_abs']:.3e})"
              + ("  <-- over threshold" if r["over"] else ""))
    first = next((r["layer"] for r in rows if r["over"]), None)
    print("first layer over the threshold:", first)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
