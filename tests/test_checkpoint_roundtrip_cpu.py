"""Native (torch_dist) checkpoints: save after two optimizer steps, load into a fresh trainer, continue identically."""

import os

import torch

from slime_b200.backends.train import checkpoint as ckpt
from slime_b200.backends.train.model import TrainModel
from slime_b200.utils.arguments import namespace_from_dict


def _args(tmp, **kw):
    base = dict(hf_checkpoint="preset:tiny", num_rollout=4, rollout_batch_size=2, n_samples_per_prompt=2, global_batch_size=4,
                seed=11, lr=1e-2, weight_decay=0.1, clip_grad=1.0, save=str(tmp / "ckpt"), load=None)
    base.update(kw)
    return namespace_from_dict(base)


def _fake_step(model, seed):
    """Deterministic gradients straight into main_grad, then the framework's own finalize + optimizer step."""
    g = torch.Generator().manual_seed(seed)
    model.zero_grad_buffer()
    for _, p in model.named_parameters():
        p.main_grad.copy_(torch.randn(p.shape, generator=g) * 0.1)
    model.finalize_grads()
    model.optimizer.step(grad_scale=1.0)
    model.scheduler.step(4)


def _params(model):
    return {n: p.detach().clone() for n, p in model.named_parameters()}


def test_save_load_continue_identically(tmp_path):
    a = _args(tmp_path)
    m1 = TrainModel(a, device=torch.device("cpu"))
    _fake_step(m1, 1)
    _fake_step(m1, 2)
    path = ckpt.save_checkpoint(a, 2, m1)
    assert os.path.isdir(path) and ckpt.read_tracker(a.save) == 2 and ckpt.is_native_checkpoint(a.save)
    before = _params(m1)

    a2 = _args(tmp_path, load=a.save, seed=999)  # a different seed: everything must come from the checkpoint
    m2 = TrainModel(a2, device=torch.device("cpu"))
    it = ckpt.load_checkpoint(a2, m2)
    assert it == 2 and m2.optimizer.step_count == m1.optimizer.step_count == 2
    assert m2.scheduler.num_steps == m1.scheduler.num_steps
    for n, p in m2.named_parameters():
        assert torch.equal(p, before[n]), n
    for s1, s2 in zip(m1.optimizer.state, m2.optimizer.state):
        for k in s1:
            assert torch.equal(s1[k], s2[k]), k
    _fake_step(m1, 3)
    _fake_step(m2, 3)
    for (n, p1), (_, p2) in zip(m1.named_parameters(), m2.named_parameters()):
        assert torch.equal(p1, p2), n
    # every random stream of the rank came back: host generator, python, numpy and the model-parallel generators
    import random

    import numpy as np

    from slime_b200.parallel import tensor_parallel as tp

    assert os.path.exists(os.path.join(path, "rng_rank00000.pt"))
    saved = torch.load(os.path.join(path, "rng_rank00000.pt"), weights_only=False)
    ckpt.restore_rng_state(saved)
    draws = (torch.rand(3), random.random(), np.random.rand(), {k: torch.rand(2, generator=g) for k, g in tp.get_rng_tracker().states.items()})
    torch.rand(5), random.random(), np.random.rand()
    ckpt.restore_rng_state(saved)
    again = (torch.rand(3), random.random(), np.random.rand(), {k: torch.rand(2, generator=g) for k, g in tp.get_rng_tracker().states.items()})
    assert torch.equal(draws[0], again[0]) and draws[1:3] == again[1:3] and all(torch.equal(draws[3][k], again[3][k]) for k in draws[3])

    # --ckpt-step picks an older iteration; --finetune / no optimizer keeps fresh optimizer state
    ckpt.save_checkpoint(a, 3, m1)
    a3 = _args(tmp_path, load=a.save, ckpt_step=2, finetune=True)
    m3 = TrainModel(a3, device=torch.device("cpu"))
    assert ckpt.load_checkpoint(a3, m3) == 2
    assert all(torch.equal(p, before[n]) for n, p in m3.named_parameters()) and m3.optimizer.step_count == 0


def test_partial_load_and_async_save(tmp_path):
    import torch.distributed.checkpoint as dcp

    a = _args(tmp_path)
    m1 = TrainModel(a, device=torch.device("cpu"))
    _fake_step(m1, 5)
    ckpt.save_checkpoint(a, 1, m1, async_save=True)
    ckpt.finalize_async_saves()
    assert ckpt.read_tracker(a.save) == 1
    # drop one tensor from the checkpoint: the loader keeps the initialised value for it and loads the rest
    path = ckpt.checkpoint_dir(a.save, 1)
    keys = ckpt._read_dcp_keys(path)
    victim = next(k for k in keys if k.endswith("final_layernorm.weight") or k.endswith("final_norm.weight"))
    state = {k: torch.empty(tuple(v.size), dtype=torch.float32 if "optimizer" in k else torch.bfloat16) for k, v in keys.items()
             if hasattr(v, "size")}
    ckpt._dcp_load(path, state)
    state.pop(victim)
    pruned = tmp_path / "pruned" / "iter_0000001"
    pruned.mkdir(parents=True)
    dcp.save(state, storage_writer=dcp.FileSystemWriter(str(pruned), single_file_per_rank=True), no_dist=True)
    (tmp_path / "pruned" / ckpt.TRACKER).write_text("1")
    a2 = _args(tmp_path, load=str(tmp_path / "pruned"), finetune=True)
    m2 = TrainModel(a2, device=torch.device("cpu"))
    fresh = _params(m2)
    ckpt.load_checkpoint(a2, m2, load_optimizer=False)
    p1 = dict(m1.named_parameters())
    for n, p in m2.named_parameters():
        if ckpt.global_param_name(n, p) == victim:
            assert torch.equal(p, fresh[n])
        else:
            assert torch.equal(p, p1[n]), n
