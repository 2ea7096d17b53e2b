"""Plug-in hook contracts: every built-in hook resolves by the dotted path users write (``slime.*`` names included) and
has the call shape its call site uses. A user hook is a drop-in replacement for one of these, so this pins the API."""

import inspect

import pytest

from slime_b200.utils.misc import load_function


def params(fn):
    return list(inspect.signature(fn).parameters)


@pytest.mark.parametrize("path", [
    "slime.rollout.sglang_rollout.generate_rollout", "slime.rollout.sft_rollout.generate_rollout",
    "slime.rollout.fully_async_rollout.generate_rollout_fully_async", "slime.rollout.sleep_rollout.sleep",
    "slime_b200.plugins.rollout_buffer.rollout_buffer_example.generate_rollout",
])
def test_rollout_functions(path):
    fn = load_function(path)
    p = params(fn)
    assert p[:3] == ["args", "rollout_id", p[2]] and p[2] in ("data_source", "data_buffer")
    assert "evaluation" in p and inspect.signature(fn).parameters["evaluation"].default is False


def test_generate_rm_filter_and_hook_shapes():
    gen = load_function("slime.rollout.sglang_rollout.generate")
    assert inspect.iscoroutinefunction(gen) and params(gen) == ["args", "sample", "sampling_params"]
    for path in ("examples.search_r1.generate_with_search.generate", "examples.multi_agent.agent_system.generate_with_multi_agents",
                 "slime.rollout.sglang_streaming_rollout.generate_streaming"):
        fn = load_function(path)
        assert inspect.iscoroutinefunction(fn) and params(fn)[:3] == ["args", "sample", "sampling_params"]
    rm = load_function("slime.rollout.rm_hub.async_rm")
    brm = load_function("slime.rollout.rm_hub.batched_async_rm")
    assert inspect.iscoroutinefunction(rm) and params(rm)[:2] == ["args", "sample"]
    assert inspect.iscoroutinefunction(brm) and params(brm)[:2] == ["args", "samples"]
    flt = load_function("slime.rollout.filter_hub.dynamic_sampling_filters.check_reward_nonzero_std")
    assert params(flt)[:2] == ["args", "samples"]
    from slime_b200.rollout.filter_hub.base_types import DynamicFilterOutput
    from slime_b200.utils.types import Sample

    out = flt(None, [Sample(reward=1.0), Sample(reward=1.0)])
    assert isinstance(out, DynamicFilterOutput) and out.keep is False
    assert flt(None, [Sample(reward=1.0), Sample(reward=0.0)]).keep is True
    hooks = load_function("slime.rollout.sample_hooks.apply_rollout_sample_hooks")
    assert inspect.iscoroutinefunction(hooks) and params(hooks)[:2] == ["args", "samples"]  # the rest is free-form context


def test_data_source_and_buffer_filter_contract():
    cls = load_function("slime.rollout.data_source.RolloutDataSourceWithBuffer")
    for m in ("get_samples", "add_samples", "save", "load", "__len__", "get_buffer_length", "update_metadata", "get_metadata"):
        assert callable(getattr(cls, m)), m
    assert params(cls.get_samples)[1] == "num_samples" and params(cls.add_samples)[1] == "samples"
    pop = load_function("slime.rollout.data_source.pop_first")
    assert params(pop) == ["args", "rollout_id", "buffer", "num_samples"]


def test_training_side_hooks():
    loss = load_function("slime.backends.megatron_utils.loss.policy_loss_function")
    assert params(loss) == ["args", "batch", "logits", "sum_of_sample_mean"]
    for path in ("slime.backends.megatron_utils.loss.vanilla_tis_function", "slime.backends.megatron_utils.loss.icepop_function",
                 "slime_b200.utils.mis.compute_mis_weights_with_cp", "examples.train_infer_mismatch_helper.mis.compute_mis_weights_with_cp"):
        fn = load_function(path)
        sig = inspect.signature(fn)
        assert params(fn)[0] == "args"
        for kw in ("pg_loss", "train_log_probs", "rollout_log_probs", "loss_masks"):
            assert sig.parameters[kw].kind is inspect.Parameter.KEYWORD_ONLY, (path, kw)
        assert any(p.kind is inspect.Parameter.VAR_KEYWORD for p in sig.parameters.values()), path
    adv = load_function("slime.backends.megatron_utils.loss.compute_advantages_and_returns")
    assert params(adv)[:2] == ["args", "rollout_data"]
    reducer = load_function("slime.backends.megatron_utils.cp_utils.get_sum_of_sample_mean")
    assert params(reducer)[:3] == ["total_lengths", "response_lengths", "loss_masks"]


def test_moved_modules_are_the_same_objects():
    import slime.utils.types as a
    import slime_b200.utils.types as b
    from slime.ray.rollout import RolloutManager as R1
    from slime_b200.runtime.rollout_manager import RolloutManager as R2

    assert a.Sample is b.Sample and R1 is R2
    with pytest.raises(ImportError):
        load_function("slime.does_not_exist.fn")


def test_sample_hooks_receive_the_context_they_name(monkeypatch):
    import asyncio
    import sys
    import types

    from slime_b200.rollout.sample_hooks import apply_rollout_sample_hooks, set_current_rollout_id
    from slime_b200.utils.types import Sample

    def sync_hook(args, sample, *, rollout_id=None):
        sample.metadata["sync_hook"] = (args.marker, rollout_id)

    async def async_hook(args, sample, *, evaluation=False):
        sample.metadata["async_hook"] = evaluation
        return sample

    def bare_hook(args, sample):
        sample.metadata["bare"] = True

    def invalid_hook(args, sample):
        return {"sample": sample}

    mod = types.ModuleType("_sample_hook_cases")
    for f in (sync_hook, async_hook, bare_hook, invalid_hook):
        setattr(mod, f.__name__, f)
    monkeypatch.setitem(sys.modules, "_sample_hook_cases", mod)
    args = types.SimpleNamespace(marker="seen", rollout_sample_hook_path=[f"_sample_hook_cases.{n}" for n in ("sync_hook", "async_hook", "bare_hook")])
    samples = [[Sample(index=0, metadata={})], [Sample(index=1, metadata={})]]
    set_current_rollout_id(7)
    out = asyncio.run(apply_rollout_sample_hooks(args, samples, evaluation=True, ignored="value"))
    assert out is not samples and [[s.index for s in g] for g in out] == [[0], [1]]
    assert all(g[0].metadata == {"sync_hook": ("seen", 7), "async_hook": True, "bare": True} for g in out)
    with pytest.raises(TypeError, match="expected Sample or None"):
        asyncio.run(apply_rollout_sample_hooks(types.SimpleNamespace(rollout_sample_hook_path=["_sample_hook_cases.invalid_hook"]), Sample(index=0)))
    one = Sample(index=0)
    assert asyncio.run(apply_rollout_sample_hooks(types.SimpleNamespace(rollout_sample_hook_path=[]), one)) is one
    set_current_rollout_id(None)


def test_server_group_gpu_ranges_are_checked_with_context():
    from slime_b200.runtime.rollout_validation import validate_server_group_gpu_indices as check

    common = dict(num_gpus_per_engine_on_node=1, num_available_gpus=4, rollout_num_gpus=4)
    check(worker_type="regular", gpu_offset=2, num_gpus_per_engine=1, num_engines=2, rollout_num_gpus_per_engine=1, **common)
    check(worker_type="placeholder", gpu_offset=4, num_gpus_per_engine=1, num_engines=0, rollout_num_gpus_per_engine=1, **common)
    with pytest.raises(ValueError) as e:
        check(worker_type="regular", gpu_offset=3, num_gpus_per_engine=2, num_engines=1, rollout_num_gpus_per_engine=2, **{**common, "num_gpus_per_engine_on_node": 2})
    for part in ("worker_type=regular", "gpu_offset=3", "num_gpus_per_engine=2", "num_engines=1", "required_gpu_slots=5", "len(reordered_gpu_ids)=4",
                 "rollout_num_gpus=4", "rollout_num_gpus_per_engine=2"):  # fmt: skip
        assert part in str(e.value)
