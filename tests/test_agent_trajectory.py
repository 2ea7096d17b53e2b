"""Session tree -> training rows: clean extension, realign, fork, shared prefixes, assistant rewrites."""

from slime_b200.agent.trajectory import TrajectoryManager, TurnRecord
from slime_b200.utils.types import Sample

BASE = Sample(index=3, group_index=1, prompt="task", label="42")
U1, U2 = {"role": "user", "content": "hi"}, {"role": "user", "content": "more"}


def _turn(prompt, out, lp=None, finish="stop"):
    return TurnRecord(prompt_ids=list(prompt), output_ids=list(out), finish_reason=finish,
                      output_log_probs=lp if lp is not None else [-0.1 * (i + 1) for i in range(len(out))])  # fmt: skip


def test_clean_two_turn_session_is_one_row():
    tm = TrajectoryManager()
    a1 = {"role": "assistant", "content": "a1"}
    tm.record_turn("s", turn=_turn([1, 2, 3], [10, 11]), prompt_messages=[U1], response_message=a1)
    tm.record_turn("s", turn=_turn([1, 2, 3, 10, 11, 4, 5], [12]), prompt_messages=[U1, a1, U2],
                   response_message={"role": "assistant", "content": "a2"})  # fmt: skip
    assert tm.turn_count("s") == 2 and tm.has_session("s")
    (row,) = tm.get_trajectory("s", base_sample=BASE, reward=1.5)
    assert row.tokens == [1, 2, 3, 10, 11, 4, 5, 12]
    assert row.response_length == 5 and row.loss_mask == [1, 1, 0, 0, 1]
    assert row.rollout_log_probs == [-0.1, -0.2, 0.0, 0.0, -0.1]
    assert row.reward == 1.5 and row.index == 3 and row.rollout_id == 3 and row.metadata["truncated"] is False
    assert not tm.has_session("s") and tm.get_trajectory("s", base_sample=BASE) == []


def test_drift_in_last_response_realigns_and_early_drift_forks():
    tm = TrajectoryManager(fork_threshold_tokens=8)
    a1 = {"role": "assistant", "content": "a1"}
    tm.record_turn("s", turn=_turn([1, 2, 3], [10, 11]), prompt_messages=[U1], response_message=a1)
    # the harness re-tokenised a1 as [10, 99]: the second prompt disagrees inside the last response only
    tm.record_turn("s", turn=_turn([1, 2, 3, 10, 99, 4], [12, 13]), prompt_messages=[U1, a1, U2],
                   response_message={"role": "assistant", "content": "a2"})  # fmt: skip
    (row,) = tm.get_trajectory("s", base_sample=BASE)
    assert row.tokens == [1, 2, 3, 10, 99, 4, 12, 13]
    assert row.loss_mask == [0, 0, 0, 1, 1]  # the drifted response no longer trains; the new one does

    tm2 = TrajectoryManager(fork_threshold_tokens=8)
    tm2.record_turn("s", turn=_turn([1, 2, 3], [10, 11]), prompt_messages=[U1], response_message=a1)
    # disagreement inside the first prompt: cannot be absorbed -> a second row that starts with its own prompt
    tm2.record_turn("s", turn=_turn([1, 7, 3, 10, 11, 4], [12]), prompt_messages=[U1, a1, U2],
                    response_message={"role": "assistant", "content": "a2"})  # fmt: skip
    rows = tm2.get_trajectory("s", base_sample=BASE)
    assert [r.tokens for r in rows] == [[1, 2, 3, 10, 11], [1, 7, 3, 10, 11, 4, 12]]
    assert rows[1].response_length == 1 and rows[1].loss_mask == [1]


def test_shared_prefix_is_trained_once():
    tm = TrajectoryManager()
    a1 = {"role": "assistant", "content": "a1"}
    tm.record_turn("s", turn=_turn([1], [10]), prompt_messages=[U1], response_message=a1)
    for k, user in enumerate(({"role": "user", "content": "left"}, {"role": "user", "content": "right"})):
        tm.record_turn("s", turn=_turn([1, 10, 20 + k], [30 + k]), prompt_messages=[U1, a1, user],
                       response_message={"role": "assistant", "content": f"b{k}"})  # fmt: skip
    rows = tm.get_trajectory("s", base_sample=BASE, reward=1.0)
    assert [r.tokens for r in rows] == [[1, 10, 20, 30], [1, 10, 21, 31]]
    assert rows[0].loss_mask == [1, 0, 1] and rows[1].loss_mask == [0, 0, 1]  # a1 trains on the first path only
    assert all(r.reward == 1.0 for r in rows)


def test_short_assistant_rewrite_is_merged_not_stranded():
    tm = TrajectoryManager()
    a1 = {"role": "assistant", "content": "a1"}
    a1_rerendered = {"role": "assistant", "content": "a1 "}
    tm.record_turn("s", turn=_turn([1], [10]), prompt_messages=[U1], response_message=a1)
    tm.record_turn("s", turn=_turn([1, 10, 5], [11]), prompt_messages=[U1, a1_rerendered, U2],
                   response_message={"role": "assistant", "content": "a2"})  # fmt: skip
    rows = tm.get_trajectory("s", base_sample=BASE)
    assert len(rows) == 1 and rows[0].tokens == [1, 10, 5, 11]  # one live branch; a1 survives only as prompt context
    assert rows[0].response_length == 1 and rows[0].loss_mask == [1]


def test_metadata_flags_and_token_cap():
    tm = TrajectoryManager()
    call = {"role": "assistant", "content": "", "tool_calls": [{"id": "t"}]}
    tm.record_turn("s", turn=_turn([1, 2], [3, 4, 5, 6], finish="length"), prompt_messages=[U1], response_message=call)
    (row,) = tm.get_trajectory("s", base_sample=BASE, extra_metadata={"k": 1}, max_sample_tokens=4)
    assert row.tokens == [1, 2, 3, 4] and row.response_length == 2 and len(row.loss_mask) == 2
    assert row.metadata == {"k": 1, "truncated": True, "use_tool": True, "ill_formed": False}
