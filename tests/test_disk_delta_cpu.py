"""Delta weight sync over a directory: codec round trips, and trainer-side publish -> engine-side pull on real files."""

import json
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from slime_b200.weight_sync import delta_codec, local_checkpoint


@pytest.mark.parametrize("encoding", ["xor", "overwrite"])
@pytest.mark.parametrize("fmt", ["zlib", "none"])
def test_codec_roundtrip(encoding, fmt):
    rng = np.random.default_rng(0)
    old = rng.integers(0, 256, 4096, dtype=np.uint8)
    new = old.copy()
    new[rng.choice(4096, 37, replace=False)] ^= 0x5A
    enc, changed = delta_codec.encode_delta(new, old, encoding)
    assert changed == 37
    wire = delta_codec.compress(enc, fmt)
    patched = old.copy()
    delta_codec.apply_delta(patched, delta_codec.decompress(wire, fmt), encoding)
    assert np.array_equal(patched, new)
    assert delta_codec.encode_delta(old, old, encoding) == (None, 0)
    for algo in ("xxh3-128", "blake3", "adler32"):
        assert delta_codec.checksum(algo, patched) == delta_codec.checksum(algo, new) != delta_codec.checksum(algo, old)


def _save_ckpt(path, tensors):
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    save_file(tensors, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump({"model_type": "toy"}, f)


def _load_ckpt(path):
    from safetensors.torch import load_file

    return load_file(os.path.join(path, "model.safetensors"))


class _ToyUpdater:
    """The real updater with the model walk replaced by a dict of HF tensors."""

    def __new__(cls, args, tensors):
        from slime_b200.weight_sync.disk_delta import UpdateWeightFromDiskDelta

        class U(UpdateWeightFromDiskDelta):
            def _iter_hf(self):
                yield from tensors.items()

        model = SimpleNamespace(device=torch.device("cpu"), cfg=None)
        u = U(args, model)
        u.is_src = True
        return u


class _FakeEngine:
    """What an engine does with the two calls: patch its local directory, then 'reload' (remember the version)."""

    def __init__(self, base_dir):
        self.base_dir, self.loaded, self.paused = base_dir, None, 0

    def pull_weights(self, local_dir, source_dir, version):
        return local_checkpoint.pull_weights(local_dir, source_dir, version, self.base_dir)

    def update_weights_from_disk(self, path, weight_version=None):
        self.loaded = (path, weight_version, _load_ckpt(path))

    def pause_generation(self):
        self.paused += 1

    def flush_cache(self):
        pass

    def continue_generation(self):
        self.paused -= 1


@pytest.mark.parametrize("encoding", ["xor", "overwrite"])
def test_publish_then_pull(tmp_path, encoding):
    torch.manual_seed(0)
    base = {"a.weight": torch.randn(64, 32).to(torch.bfloat16), "b.weight": torch.randn(128).to(torch.bfloat16),
            "frozen.weight": torch.randn(16, 16).to(torch.bfloat16)}  # fmt: skip
    hf = str(tmp_path / "hf")
    _save_ckpt(hf, base)
    args = SimpleNamespace(update_weight_disk_dir=str(tmp_path / "stream"), update_weight_delta_encoding=encoding,
                           update_weight_delta_checksum="xxh3-128", custom_update_weight_post_write_path=None,
                           update_weight_local_checkpoint_dir=str(tmp_path / "local"), hf_checkpoint=hf,
                           update_weight_disk_keep_files=False, sglang_quantization=None)  # fmt: skip
    live = {k: v.clone() for k, v in base.items()}
    up = _ToyUpdater(args, live)
    eng = _FakeEngine(hf)
    up.connect_rollout_engines([eng])
    up.is_src = True
    up.update_weights()  # baseline only: engines materialise version 0, nothing is published
    assert local_checkpoint.current_version(args.update_weight_local_checkpoint_dir) == 0
    assert not os.path.exists(local_checkpoint.version_dir(args.update_weight_disk_dir, 1))

    for step in (1, 2):
        live["a.weight"][step, :5] += 1.0  # a sparse change, as after a small optimizer step
        live["b.weight"][10 * step] = 3.0
        up.update_weights()
        vdir = local_checkpoint.version_dir(args.update_weight_disk_dir, step)
        index = json.load(open(os.path.join(vdir, "model.safetensors.index.json")))
        assert index["metadata"]["delta_encoding"] == encoding and int(index["metadata"]["base_version"]) == step - 1
        assert set(index["weight_map"]) == {"a.weight", "b.weight"}  # the frozen tensor is not on the wire
        path, version, loaded = eng.loaded
        assert version == str(step) and eng.paused == 0
        for k in live:
            assert torch.equal(loaded[k], live[k]), k
        assert 0 < up.metrics["perf/update_weights_density"] < 0.05

    # a fresh host catches up from the base by replaying every delta
    late = str(tmp_path / "late")
    local_checkpoint.pull_weights(late, args.update_weight_disk_dir, 2, hf)
    assert all(torch.equal(_load_ckpt(late)[k], live[k]) for k in live)
    # corruption is caught by the checksum
    bad = str(tmp_path / "bad")
    local_checkpoint.pull_weights(bad, args.update_weight_disk_dir, 1, hf)
    where = local_checkpoint.tensor_locations(bad)["a.weight"]
    with open(where[0], "r+b") as f:
        f.seek(where[1] + 64 * 2)  # a byte inside row 2, which delta 2 touches (xor) / leaves wrong (overwrite elsewhere)
        f.write(b"\x7f")
    if encoding == "xor":
        with pytest.raises(ValueError, match="checksum"):
            local_checkpoint.pull_weights(bad, args.update_weight_disk_dir, 2, hf)
