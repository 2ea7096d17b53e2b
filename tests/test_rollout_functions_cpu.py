"""Rollout functions that need no engine: fully-async worker, forge replay, SFT rollout, OPD reward post-processing."""

import asyncio
import threading

import pytest
import torch

from slime_b200.utils.arguments import namespace_from_dict
from slime_b200.utils.types import Sample


class _Buffer:
    """Thread-safe stand-in for the data source: hands out single-sample groups with increasing index."""

    def __init__(self, n_samples=1):
        self.lock, self.next, self.n, self.returned = threading.Lock(), 0, n_samples, []

    def get_samples(self, k):
        with self.lock:
            if self.returned:
                return [self.returned.pop(0) for _ in range(min(k, len(self.returned)))]
            out = []
            for _ in range(k):
                out.append([Sample(index=self.next * self.n + j, group_index=self.next, prompt="p") for j in range(self.n)])
                self.next += 1
            return out

    def add_samples(self, groups):
        with self.lock:
            self.returned += groups


def _args(**kw):
    base = dict(rollout_batch_size=4, n_samples_per_prompt=1, num_rollout=2, sglang_server_concurrency=3, rollout_num_gpus=1,
                rollout_num_gpus_per_engine=1, hf_checkpoint=None, rollout_global_dataset=True)  # fmt: skip
    return namespace_from_dict({**base, **kw})


def test_fully_async_worker_runs_ahead_and_requeues_aborted_groups():
    from slime_b200.rollout import fully_async_rollout as fa

    aborted_once = set()

    async def fake_group(args, group, sampling_params, evaluation=False):
        await asyncio.sleep(0.01 * (1 + group[0].index % 3))  # uneven latencies: completion order != submission order
        for s in group:
            if s.index == 2 and s.index not in aborted_once:
                aborted_once.add(s.index)
                s.status = Sample.Status.ABORTED  # e.g. cut short by a weight update
            else:
                s.status, s.response_length, s.reward = Sample.Status.COMPLETED, 3, 1.0
        return group

    buf = _Buffer()
    w = fa.AsyncRolloutWorker(_args(), buf, concurrency=3, generate_group=fake_group)
    w.start()
    try:
        first = fa.collect_groups(w, 4)
        second = fa.collect_groups(w, 4)
    finally:
        w.stop()
    for batch in (first, second):
        assert len(batch) == 4
        assert [g[0].index for g in batch] == sorted(g[0].index for g in batch)
        assert all(s.status == Sample.Status.COMPLETED for g in batch for s in g)
    seen = [g[0].index for g in first + second]
    assert len(set(seen)) == 8 and 2 in seen  # the aborted group was regenerated, not lost and not duplicated
    assert w.requeued == 1
    # submission stops while `concurrency` finished groups wait, so at most that many more (those in flight) can pile up
    assert w.queue_size() <= 2 * 3 - 1


def test_forge_load_replays_dumps(tmp_path):
    from slime_b200.observability.rollout_data_utils import save_debug_rollout_data
    from slime_b200.rollout import forge_load

    samples = [Sample(index=i, tokens=[1, 2, 3, 4], response_length=2, reward=float(i), status=Sample.Status.COMPLETED)
               for i in range(3)]  # fmt: skip
    tpl = str(tmp_path / "dump_{rollout_id}.pt")
    save_debug_rollout_data(tpl, samples, rollout_id=0, evaluation=False)
    save_debug_rollout_data(tpl, {"ds": {"samples": samples[:2]}}, rollout_id=0, evaluation=True)
    args = _args(load_forge_rollout_data=tpl, eval_reward_key=None, reward_key=None)
    out = forge_load.generate_rollout(args, 0, None)
    assert [s.reward for s in out.samples] == [0.0, 1.0, 2.0] and out.samples[0].tokens == [1, 2, 3, 4]
    assert len(forge_load.generate_rollout(args, 5, None).samples) == 3  # missing rollout -> falls back to rollout 0
    ev = forge_load.generate_rollout(args, 0, None, evaluation=True)
    assert ev.data["forge_eval"]["rewards"] == [0.0, 1.0]
    assert forge_load.generate_rollout(args, 7, None, evaluation=True).data == {}
    literal = _args(load_forge_rollout_data=tpl.format(rollout_id=0), eval_reward_key=None, reward_key=None)
    assert len(forge_load.generate_rollout(literal, 3, None).samples) == 3
    with pytest.raises(RuntimeError):
        forge_load.generate_rollout(_args(load_forge_rollout_data=None), 0, None)


def test_opd_post_process_keeps_response_logprobs():
    from slime_b200.rollout.on_policy_distillation import post_process_rewards

    def teacher_reply(n):
        return {"meta_info": {"input_token_logprobs": [[None, 0]] + [[-0.1 * i, i] for i in range(1, n)]}}

    samples = [Sample(index=0, tokens=list(range(6)), response_length=2, reward=teacher_reply(6)),
               Sample(index=1, tokens=list(range(4)), response_length=3, reward=teacher_reply(4))]  # fmt: skip
    raw, rewards = post_process_rewards(_args(reward_key=None), samples)
    assert raw == rewards == [0.0, 0.0]
    assert torch.allclose(samples[0].teacher_log_probs, torch.tensor([-0.4, -0.5]))
    assert torch.allclose(samples[1].teacher_log_probs, torch.tensor([-0.1, -0.2, -0.3]))


def test_streaming_snapshot_rewind_roundtrip():
    from slime_b200.rollout.sglang_streaming_rollout import _rewind, _snapshot, _sse_payloads

    s = Sample(index=0, tokens=[1, 2], response="ab", response_length=1, rollout_log_probs=[-0.5], loss_mask=[1])
    snap = _snapshot(s)
    s.tokens += [9, 9]
    s.response += "zz"
    s.response_length = 3
    s.rollout_log_probs += [-1.0, -2.0]
    s.loss_mask += [1, 1]
    _rewind(s, snap)
    assert (s.tokens, s.response, s.response_length, s.rollout_log_probs, s.loss_mask) == ([1, 2], "ab", 1, [-0.5], [1])
    s.tokens.append(5)
    assert snap["tokens"] == [1, 2]  # rewinding hands out copies
    assert _sse_payloads('data: {"text": "x"}') == {"text": "x"}
    assert _sse_payloads("data: [DONE]") is None and _sse_payloads(": keep-alive") is None and _sse_payloads("data: {oops") is None
