"""Small pure-Python utilities against closed-form expectations: scheduling invariants, partitioners, reward rules,
evaluation configs, the stateless optimizer, zero blocks in fp8 quantisation."""

import asyncio
import math
import random
from argparse import Namespace

import pytest
import torch

from slime_b200.utils import seqlen_balancing as sb
from slime_b200.utils.dp_schedule import build_dp_schedule
from slime_b200.utils.types import Sample


# ------------------------------------------------------------------------------------------------ dp schedule
def _sched_args(**kw):
    base = dict(use_dynamic_batch_size=True, max_tokens_per_gpu=100, micro_batch_size=None, balance_data=False, balance_by_flops=False,
                num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=2, kv_channels=16, ffn_hidden_size=128,
                vocab_size=256, num_experts=None)  # fmt: skip
    base.update(kw)
    return Namespace(**base)


@pytest.mark.parametrize("dp,vpp,group,balance", [(1, 1, 1, False), (2, 1, 1, False), (3, 1, 1, True), (2, 2, 2, False), (4, 1, 1, True)])
def test_dp_schedule_invariants(dp, vpp, group, balance):
    """Same micro-batch count on every rank and step; every kept sample placed exactly once; micro-batch indices tile each
    rank's partition; only a single over-long sample may exceed the token cap; samples of a rollout stay in one step."""
    rng = random.Random(dp * 10 + vpp)
    n_rollouts, per = 12, 3
    lengths = [rng.randint(5, 60) for _ in range(n_rollouts * per)]
    lengths[7] = 250  # longer than the cap on its own
    rollout_ids = [i // per for i in range(n_rollouts * per)]
    args = _sched_args(balance_data=balance)
    cfgp = {"dp_size": dp, "cp_size": 1, "vpp_size": vpp, "microbatch_group_size_per_vp_stage": group}
    parts, mbi, num_mb, gbs = build_dp_schedule(args, cfgp, lengths, global_batch_size=4, rollout_indices=rollout_ids)
    assert gbs == [4, 4, 4] and len(num_mb) == 3
    placed = sorted(p for part in parts for p in part)
    assert placed == list(range(len(lengths)))
    align = group if vpp > 1 else 1
    for r in range(dp):
        assert len(mbi[r]) == sum(num_mb) and all(n % align == 0 for n in num_mb)
        flat = [i for mb in mbi[r] for i in mb]
        assert flat == list(range(len(parts[r])))
        for mb in mbi[r]:
            tokens = sum(lengths[parts[r][i]] for i in mb)
            assert tokens <= 100 or len(mb) == 1
    # steps do not mix rollouts: step s holds rollouts 4s .. 4s+3
    k = 0
    for s, n in enumerate(num_mb):
        step_samples = {parts[r][i] for r in range(dp) for mb in mbi[r][k : k + n] for i in mb}
        assert {rollout_ids[p] for p in step_samples} == set(range(4 * s, 4 * s + 4))
        k += n


def test_dp_schedule_static_batching_and_errors():
    args = _sched_args(use_dynamic_batch_size=False, micro_batch_size=2, max_tokens_per_gpu=None)
    cfgp = {"dp_size": 2, "cp_size": 1, "vpp_size": 1, "microbatch_group_size_per_vp_stage": 1}
    parts, mbi, num_mb, _ = build_dp_schedule(args, cfgp, [10] * 8, global_batch_size=8, rollout_indices=list(range(8)))
    assert num_mb == [2] and all(len(mb) == 2 for r in range(2) for mb in mbi[r])
    with pytest.raises(AssertionError, match="not a multiple"):
        build_dp_schedule(args, {**cfgp, "dp_size": 3}, [10] * 8, global_batch_size=8, rollout_indices=list(range(8)))
    with pytest.raises(AssertionError, match="need at least one rollout"):
        build_dp_schedule(args, cfgp, [10] * 2, global_batch_size=8, rollout_indices=[0, 1])


# ------------------------------------------------------------------------------------------------ partitioners
def test_partitioners_cover_everything_and_balance():
    rng = random.Random(0)
    lens = [rng.randint(1, 1000) for _ in range(64)]
    for k, equal in ((4, True), (4, False), (7, False), (8, True)):
        for fn in (sb.karmarkar_karp, sb.greedy_partition, sb.get_seqlen_balanced_partitions):
            parts = fn(lens, k, equal)
            assert len(parts) == k and sorted(i for p in parts for i in p) == list(range(len(lens)))
            if equal:
                assert {len(p) for p in parts} == {len(lens) // k}
        sums = [sum(lens[i] for i in p) for p in sb.get_seqlen_balanced_partitions(lens, k, equal)]
        assert max(sums) - min(sums) <= max(lens)  # within one item of perfectly even
    bins = sb.first_fit_pack([60, 50, 40, 30, 200, 10], 100)
    assert sorted(i for b in bins for i in b) == list(range(6))
    assert all(sum([60, 50, 40, 30, 200, 10][i] for i in b) <= 100 or len(b) == 1 for b in bins)
    sb.expand_bins_by_splitting(bins, len(bins) + 2, [60, 50, 40, 30, 200, 10])
    assert sorted(i for b in bins for i in b) == list(range(6)) and all(bins)
    idx = [3, 0, 2, 1]
    rev = sb.get_reverse_idx(idx)
    assert [idx[rev[i]] for i in range(4)] == [0, 1, 2, 3]


# ------------------------------------------------------------------------------------------------ reward rules
def _rm(run_rm_type, response, label, md=None):
    from slime_b200.rollout.rm_hub import async_rm

    s = Sample(index=0, prompt="q", response=response, label=label, metadata=md)
    return asyncio.run(async_rm(Namespace(rm_type=run_rm_type, custom_rm_path=None), s))


def test_rule_based_rewards():
    assert _rm("math", "so the answer is \\boxed{\\frac{1}{2}}", "0.5") == 1
    assert _rm("math", "the answer is \\boxed{3}", "4") == 0
    assert _rm("deepscaler", "thinking </think> therefore \\boxed{42}", "42") == 1
    assert _rm("deepscaler", "no think close \\boxed{42}", "42") == 0  # the reasoning block must be closed
    assert _rm("dapo", "Answer: 7", "7")["score"] == 1.0 and _rm("dapo", "Answer: 8", "7")["score"] == -1.0
    assert _rm("f1", "The capital is Paris", "Paris") == pytest.approx(2 * (1 / 3) * 1 / (1 / 3 + 1), rel=1e-6)
    assert _rm("gpqa", "I think (B) is right. Answer: B", "B") == 1.0 and _rm("gpqa", "Answer: C", "B") == 0.0
    assert _rm("boxed_f1", "x \\boxed{10}", "10") == 1.0  # the boxed_ prefix hands the boxed content to the rule
    assert _rm("random", "x", "y") in (0, 1)
    with pytest.raises(NotImplementedError):
        _rm("nope", "x", "y")
    # per-sample metadata overrides the run's reward type
    assert _rm("math", "Answer: B", "B", {"rm_type": "gpqa"}) == 1.0


# ------------------------------------------------------------------------------------------------ eval configs
def test_eval_dataset_configs_merge_defaults_and_args():
    from slime_b200.utils.eval_config import EvalDatasetConfig, build_eval_dataset_configs, ensure_dataset_list

    raw = ensure_dataset_list({"aime": {"path": "/d/aime.jsonl", "rm_type": "deepscaler"}, "gpqa": {"path": "/d/gpqa.jsonl", "top_p": 0.9}})
    assert [d["name"] for d in raw] == ["aime", "gpqa"]
    args = Namespace(eval_max_response_len=4096, rollout_max_response_len=1024, n_samples_per_eval_prompt=4, eval_temperature=None,
                     rollout_temperature=0.8, eval_top_p=None, rollout_top_p=1.0, input_key="prompt", eval_input_key=None)  # fmt: skip
    cfgs = build_eval_dataset_configs(args, raw, {"n_samples_per_eval_prompt": 8})
    assert all(isinstance(c, EvalDatasetConfig) for c in cfgs)
    assert cfgs[0].n_samples_per_eval_prompt == 8 and cfgs[1].top_p == 0.9
    assert cfgs[0].inject_metadata({"a": 1}) == {"a": 1, "rm_type": "deepscaler"}
    with pytest.raises(ValueError, match="Unknown key"):
        build_eval_dataset_configs(args, raw, {"not_a_field": 1})
    with pytest.raises(ValueError, match="include a `name`"):
        ensure_dataset_list([{"path": "x"}])
    with pytest.raises(ValueError, match="min_eval_samples"):
        EvalDatasetConfig(name="x", path="y", min_eval_samples=0)


# ------------------------------------------------------------------------------------------------ optimizer
def test_stateless_adam_is_a_sign_like_step_and_keeps_no_state():
    from slime_b200.backends.train.optimizer import StatelessAdam

    p = torch.nn.Parameter(torch.tensor([1.0, -2.0, 3.0, 0.5]))
    opt = StatelessAdam([p], lr=0.1, betas=(0.9, 0.999), eps=1e-12, weight_decay=0.0)
    p.grad = torch.tensor([0.3, -5.0, 1e-3, 0.0])
    opt.step()
    # moments restart from zero, so the bias-corrected update is g / |g|: a step of lr against the gradient's sign
    assert torch.allclose(p.detach(), torch.tensor([0.9, -1.9, 2.9, 0.5]), atol=1e-6)
    assert not opt.state  # nothing is remembered between steps
    p.grad = torch.tensor([0.3, -5.0, 1e-3, 0.0])
    opt.step()
    assert torch.allclose(p.detach(), torch.tensor([0.8, -1.8, 2.8, 0.5]), atol=1e-6)
    q = torch.nn.Parameter(torch.ones(2))
    StatelessAdam([q], lr=0.1, weight_decay=0.5).step()  # no gradient: untouched, decay included
    assert torch.equal(q.detach(), torch.ones(2))
    # every step is the first step of a freshly created torch optimizer, with decoupled or coupled weight decay
    for decoupled, cls in ((True, torch.optim.AdamW), (False, torch.optim.Adam)):
        torch.manual_seed(0)
        start = torch.randn(8, dtype=torch.float64)
        grads = [torch.randn_like(start) for _ in range(4)]
        ours, kw = start.clone(), dict(lr=0.03, betas=(0.9, 0.98), eps=1e-6, weight_decay=0.1)
        opt = StatelessAdam([ours], adam_w_mode=decoupled, **kw)
        ref = start.clone()
        for g in grads:
            ours.grad = g.clone()
            opt.step()
            opt.zero_grad()
            ref = ref.detach().requires_grad_(True)
            fresh = cls([ref], **kw)
            ref.grad = g.clone()
            fresh.step()
        assert torch.allclose(ours, ref.detach(), atol=1e-12) and opt.state_dict()["state"] == {}


# ------------------------------------------------------------------------------------------------ quantisation
def test_block_fp8_quantisation_of_zero_blocks_and_ragged_edges():
    from slime_b200 import ops

    x = torch.zeros(300, 260)
    x[:128, :128] = torch.randn(128, 128)
    x[299, 259] = 5.0
    q, s = ops.block_fp8_quant(x, (128, 128))
    assert q.shape == x.shape and s.shape == (3, 3) and torch.isfinite(s).all() and (s > 0).all()
    back = ops.block_fp8_dequant(q, s, (128, 128), torch.float32)
    assert torch.isfinite(back).all() and float(back[128:256, 128:256].abs().max()) == 0.0  # an all-zero block stays zero
    assert abs(float(back[299, 259]) - 5.0) < 1e-6 and (back[:128, :128] - x[:128, :128]).abs().max() <= x.abs().max() / 16
    q2, s2 = ops.block_fp8_quant(x, (128, 128), pow2_scale=True)
    assert torch.allclose(torch.log2(s2), torch.log2(s2).round())  # UE8M0-style scales are powers of two


# ------------------------------------------------------------------------------------------------ samples
def test_sample_round_trip_and_response_bookkeeping():
    s = Sample(index=3, group_index=1, prompt="p", tokens=[1, 2, 3], label="x", metadata={"k": 1})
    args = Namespace(rollout_max_response_len=8)
    s.append_response_tokens(args, tokens=[4, 5], log_probs=[-0.1, -0.2], trainable=True, text="ab")
    s.append_response_tokens(args, tokens=[6], trainable=False, text="o")
    assert s.tokens == [1, 2, 3, 4, 5, 6] and s.response_length == 3 and s.loss_mask == [1, 1, 0]
    assert s.rollout_log_probs == [-0.1, -0.2, 0.0] and s.response == "abo"
    d = s.to_dict()
    back = Sample.from_dict(d)
    assert back.tokens == s.tokens and back.loss_mask == s.loss_mask and back.metadata == {"k": 1} and back.status == s.status
    assert math.isclose(sum(back.rollout_log_probs), -0.3)


# ------------------------------------------------------------------------------------------------ debug index checks
def test_debug_mode_catches_bad_indices_before_any_launch(monkeypatch):
    """SLIME_B200_CHECKS=1: every op with a data-dependent index validates it on the host and names the offender."""
    from slime_b200 import ops
    from slime_b200.ops import _checks, attention, grouped

    k_cache, v_cache = torch.zeros(32, 2, 4), torch.zeros(32, 2, 4)
    good_slots = torch.tensor([0, 5, -1], dtype=torch.int32)
    k, v = torch.randn(3, 8), torch.randn(3, 8)
    bt = torch.tensor([[0, 1, 7, 0]], dtype=torch.int32)
    q = torch.randn(1, 2, 4)
    # off: the same calls run (or fail later, in the op itself); on: they are refused up front
    monkeypatch.setenv("SLIME_B200_CHECKS", "1")
    ops.kv_write(k, v, good_slots, k_cache, v_cache)  # -1 = "skip this row" stays legal
    with pytest.raises(_checks.IndexCheckError, match=r"kv_write: slots\[1\] = 99 is outside"):
        ops.kv_write(k, v, torch.tensor([0, 99, 1], dtype=torch.int32), k_cache, v_cache)
    ops.paged_decode_attention(q, k_cache, v_cache, bt, torch.tensor([9], dtype=torch.int32), 4)
    with pytest.raises(_checks.IndexCheckError, match=r"block_table\[0, 2\] = 9 is not one of the cache's 8 pages"):
        ops.paged_decode_attention(q, k_cache, v_cache, torch.tensor([[0, 1, 9, 0]], dtype=torch.int32), torch.tensor([9], dtype=torch.int32), 4)
    with pytest.raises(_checks.IndexCheckError, match="does not fit a block table of 16 tokens"):
        ops.paged_decode_attention(q, k_cache, v_cache, bt, torch.tensor([17], dtype=torch.int32), 4)
    # an entry past the used length is never read, so it may hold anything
    ops.paged_decode_attention(q, k_cache, v_cache, torch.tensor([[0, 1, 99, 99]], dtype=torch.int32), torch.tensor([8], dtype=torch.int32), 4)
    with pytest.raises(_checks.IndexCheckError, match="embedding: ids"):
        ops.embedding(torch.tensor([3, -2]), torch.randn(8, 4))
    with pytest.raises(_checks.IndexCheckError, match="scatter_rows: dest"):
        grouped.scatter_rows(torch.randn(2, 8), torch.tensor([0, 7], dtype=torch.int32), 1, 4)
    with pytest.raises(_checks.IndexCheckError, match=r"segment 0 covers key rows \[2, 9\) of 6"):
        attention.segment_attention(torch.randn(6, 2, 4), torch.randn(6, 1, 4), torch.randn(6, 1, 4), torch.tensor([[0, 3, 2, 7]], dtype=torch.int32))
    monkeypatch.setenv("SLIME_B200_CHECKS", "0")
    _checks.index_range("x", "y", torch.tensor([5]), upper=2)  # switched off: no check, no cost


def test_dp_schedule_fixed_cases():
    """Static / balanced / dynamic / interleaved-pipeline / grouped-rollout schedules on fixed inputs: every rank's
    micro-batches tile its partition, partitions are disjoint and cover what is expected, a micro-batch above the token cap
    holds a single sample. The FLOPs-balanced split of [1, 2, 3, 4, 5, 7, 9, 10] over two ranks is [[1, 2, 5, 6], [0, 3, 4, 7]]
    (heavier part first), as in the reference's tests/test_dp_schedule.py."""
    from types import SimpleNamespace

    def A(**k):
        d = dict(micro_batch_size=1, use_dynamic_batch_size=False, max_tokens_per_gpu=None, balance_data=False, balance_by_flops=False,
                 hidden_size=16, num_attention_heads=2, num_query_groups=2, vocab_size=32, ffn_hidden_size=64, num_experts=None,
                 num_layers=2, kv_channels=8)  # fmt: skip
        d.update(k)
        return SimpleNamespace(**d)

    def P(dp=1, vpp=1, group=1):
        return {"dp_size": dp, "cp_size": 1, "vpp_size": vpp, "microbatch_group_size_per_vp_stage": group}

    def check(parts, mbi, nmb, dp, expect, lengths, cap=None):
        seen = set()
        for r in range(dp):
            assert len(mbi[r]) == sum(nmb) and [i for m in mbi[r] for i in m] == list(range(len(parts[r])))
            assert seen.isdisjoint(parts[r])
            seen.update(parts[r])
            for m in mbi[r]:
                assert cap is None or sum(lengths[parts[r][i]] for i in m) <= cap or len(m) == 1
        assert seen == set(expect)

    tl = [10] * 16
    p, m, n, g = build_dp_schedule(A(micro_batch_size=2), P(4), tl, global_batch_size=16, rollout_indices=list(range(16)))
    assert n == [2] and g == [16]
    check(p, m, n, 4, range(16), tl)
    tl = [1, 2, 3, 4, 5, 6, 7, 8, 8, 7, 6, 5, 4, 3, 2, 1]
    p, m, n, g = build_dp_schedule(A(micro_batch_size=2, balance_data=True), P(2), tl, global_batch_size=8, rollout_indices=list(range(16)))
    assert n == [2, 2] and g == [8, 8]
    check(p, m, n, 2, range(16), tl)
    p, m, n, g = build_dp_schedule(A(balance_data=True), P(2), [1, 2, 3, 4, 5, 7, 9, 10], global_batch_size=8, rollout_indices=list(range(8)))
    assert p == [[1, 2, 5, 6], [0, 3, 4, 7]] and n == [4] and g == [8]
    dyn = A(use_dynamic_batch_size=True, max_tokens_per_gpu=10)
    tl = [15, 3, 3, 3, 3, 3, 3, 3]  # the oversized sample gets a micro-batch of its own
    p, m, n, g = build_dp_schedule(dyn, P(2), tl, global_batch_size=8, rollout_indices=list(range(8)))
    check(p, m, n, 2, range(8), tl, cap=10)
    tl = [4] * 32
    p, m, n, g = build_dp_schedule(A(use_dynamic_batch_size=True, max_tokens_per_gpu=8), P(2, vpp=2, group=2), tl, global_batch_size=16,
                                   rollout_indices=list(range(32)))  # fmt: skip
    assert all(x % 2 == 0 for x in n)
    check(p, m, n, 2, range(32), tl, cap=8)
    dyn = A(use_dynamic_batch_size=True, max_tokens_per_gpu=12)
    p, m, n, g = build_dp_schedule(dyn, P(1), [3] * 9, global_batch_size=1, rollout_indices=[0, 0, 0, 1, 1, 2, 2, 2, 2])
    assert g == [1, 1, 1]  # a rollout's samples stay in one step
    cur = 0
    for step, k in enumerate(n):
        assert sorted(p[0][j] for mb in m[0][cur : cur + k] for j in mb) == [[0, 1, 2], [3, 4], [5, 6, 7, 8]][step]
        cur += k
    p, m, n, g = build_dp_schedule(dyn, P(1), [3] * 8, global_batch_size=2, rollout_indices=[0, 0, 1, 2, 2, 3, 4, 4])
    assert g == [2, 2]  # the fifth rollout does not fill a step and is dropped
    check(p, m, n, 1, range(6), [3] * 8, cap=12)
    with pytest.raises(AssertionError, match="num_rollouts"):
        build_dp_schedule(dyn, P(1), [3] * 6, global_batch_size=4, rollout_indices=[0, 0, 1, 1, 2, 2])


# ------------------------------------------------------------------------------------------------ argument validation
_ARGV = ["--rollout-batch-size", "4", "--num-rollout", "2", "--hf-checkpoint", "preset:qwen2.5-0.5b", "--rollout-num-gpus", "4"]


@pytest.mark.parametrize("extra,message", [
    (["--update-weight-transport", "disk"], "update-weight-disk-dir"),
    (["--save-debug-rollout-data", "/tmp/d_{rollout_id}.pt", "--save-debug-train-data", "/tmp/d_{rollout_id}.pt"], "--save-debug-train-data must not be equal"),
    (["--rollout-temperature", "0.0"], "--rollout-temperature must be > 0"),
    (["--rollout-temperature", "-0.1"], "--rollout-temperature must be > 0"),
    (["--update-weight-mode", "delta", "--update-weight-transport", "nccl", "--update-weight-local-checkpoint-dir", "/l"], "requires --update-weight-transport=disk"),
    (["--update-weight-mode", "delta", "--update-weight-transport", "disk", "--update-weight-disk-dir", "/s", "--update-weight-local-checkpoint-dir", "/l",
      "--colocate"], "not supported with --colocate"),
    (["--update-weight-mode", "delta", "--update-weight-transport", "disk", "--update-weight-disk-dir", "/s"], "requires --update-weight-local-checkpoint-dir"),
    (["--allgather-cp", "--context-parallel-size", "2"], "only supported for DSA attention models"),
])  # fmt: skip
def test_argument_combinations_that_are_refused(extra, message):
    from slime_b200.utils.arguments import parse_args

    with pytest.raises(ValueError, match=message):
        parse_args(_ARGV + extra)


def test_argument_defaults_that_are_kept_or_filled():
    from slime_b200.utils.arguments import parse_args

    assert parse_args(_ARGV + ["--start-rollout-id", "100"]).start_rollout_id == 100 and parse_args(_ARGV).start_rollout_id == 0
    a = parse_args(_ARGV[:-2] + ["--colocate", "--rollout-num-gpus", "0"])
    assert a.rollout_num_gpus == 0 and a.offload_train is True and a.offload_rollout is True
    a = parse_args(_ARGV[:-2] + ["--colocate", "--actor-num-gpus-per-node", "8", "--actor-num-nodes", "1", "--rollout-num-gpus", "12"])
    assert a.rollout_num_gpus == 12 and a.offload_train and a.offload_rollout
    a = parse_args(_ARGV[:-2] + ["--rollout-num-gpus", "0"])
    assert (a.rollout_num_gpus, a.actor_num_gpus_per_node, a.actor_num_nodes, a.offload_train, a.offload_rollout) == (0, 8, 1, False, False)
    assert parse_args(_ARGV + ["--allgather-cp"]).allgather_cp  # without context parallelism the flag has nothing to refuse


def test_route_records_are_validated_and_rollout_payloads_normalised(tmp_path):
    import numpy as np

    from slime_b200.observability.rollout_data_utils import (
        load_debug_rollout_data, save_debug_rollout_data, validate_rollout_routed_experts_for_replay)
    from slime_b200.rollout.train_data import tensorize_rollout_data_for_training

    args = Namespace(num_layers=6, moe_router_topk=2, moe_layer_freq=[0, 0, 0, 1, 1, 1])
    routes = torch.zeros((4, 6, 2), dtype=torch.uint8)
    routes[:, 3:, 1] = 7
    validate_rollout_routed_experts_for_replay([routes], args)  # dense layers are zero by construction
    routes = torch.zeros((4, 6, 2), dtype=torch.uint8)
    routes[:, 3, 1] = 7
    with pytest.raises(ValueError, match=r"all zero.*\[4, 5\]"):  # an engine stage that did not report its layers
        validate_rollout_routed_experts_for_replay([routes], args)
    with pytest.raises(ValueError, match="Invalid rollout routed-experts shape"):
        validate_rollout_routed_experts_for_replay([torch.zeros((4, 5, 2), dtype=torch.uint8)], args)
    with pytest.raises(ValueError, match="no rollout routed-experts"):
        validate_rollout_routed_experts_for_replay([], args)
    frozen = np.array([1, 2, 3])
    frozen.flags.writeable = False
    data = {"tokens": [frozen], "loss_masks": [[1, 0]], "rollout_mask_sums": [2],
            "multimodal_train_inputs": [{"pixel_values": torch.tensor([1.0], requires_grad=True), "metadata": "unchanged"}]}  # fmt: skip
    tensorize_rollout_data_for_training(data)
    assert data["tokens"][0].dtype == torch.long and data["loss_masks"][0].dtype == torch.int and data["rollout_mask_sums"].dtype == torch.float32
    mm = data["multimodal_train_inputs"][0]
    assert mm["metadata"] == "unchanged" and not mm["pixel_values"].requires_grad
    template = str(tmp_path / "rollout_{rollout_id}.pt")
    save_debug_rollout_data(template, [Sample(index=1, rollout_id=3, prompt="question", response="answer", response_length=1)], rollout_id=3, evaluation=False)
    back = load_debug_rollout_data(template, rollout_id=3)
    assert (len(back), back[0].index, back[0].rollout_id, back[0].prompt, back[0].response) == (1, 1, 3, "question", "answer")
    save_debug_rollout_data(template, {"math": {"samples": [Sample(index=1)]}, "code": {"samples": [Sample(index=2)]}}, rollout_id=4, evaluation=True)
    saved = torch.load(tmp_path / "rollout_eval_4.pt", weights_only=False)
    assert saved["rollout_id"] == 4 and [s["index"] for s in saved["samples"]] == [1, 2]
