"""Turn multi-turn agent sessions into loss-masked training rows.

An agent harness talks to the policy through a chat API (``slime_b200/agent/adapters``). Every model call is recorded
as a ``TurnRecord``: the exact prompt token ids the engine saw, the token ids and log-probs it produced. Calls of one
session form a tree, because harnesses branch: they retry, summarise history, or run sub-agents from a shared prefix.
``TrajectoryManager`` keeps that tree per session id and, at the end, walks every root-to-leaf path and packs the
generated turns on it into as few ``Sample`` rows as possible:

* consecutive turns whose prompt exactly extends the tokens already collected are appended (prompt tail with loss
  mask 0, generated tokens with loss mask 1 and their rollout log-probs);
* text -> tokens -> text round trips rarely reproduce ids exactly. If a later prompt disagrees with the collected
  tokens only inside the most recent response and the new response is short, that response span is *replaced* by
  what the prompt says (loss mask 0: drifted tokens carry no learning signal) and packing continues;
* any other disagreement *forks*: the row is closed and a new one starts with this turn's full prompt.

A generated turn shared by several leaves is trained once; other paths carry it as context. A short assistant message
that a later prompt replays slightly re-rendered is merged onto the node that generated it (which stops training it)
instead of stranding the original as a dead-end branch.
Parity: slime/agent/trajectory.py:27-508 (same public surface and packing rules).
"""

from __future__ import annotations

import dataclasses
import enum
import logging
from typing import Any

from slime_b200.utils.types import Sample

logger = logging.getLogger(__name__)
__all__ = ["TrajectoryManager", "TurnRecord"]


@dataclasses.dataclass(frozen=True)
class TurnRecord:
    """One engine ``/generate`` call as the adapters saw it."""

    prompt_ids: list[int]
    output_ids: list[int]
    finish_reason: str
    output_log_probs: list[float] = dataclasses.field(default_factory=list)
    ill_formed: bool = False


class MessageNode:
    """A chat message in a session tree. ``turn`` is set only on assistant messages this framework generated."""

    __slots__ = ("role", "message", "metadata", "parent", "children", "turn", "turn_index", "response_trained")

    def __init__(self, role=None, message=None, metadata=None, parent=None):
        self.role, self.message, self.metadata, self.parent = role, message, dict(metadata or {}), parent
        self.children: list[MessageNode] = []
        self.turn: TurnRecord | None = None
        self.turn_index: int | None = None
        self.response_trained = False

    @property
    def is_root(self) -> bool:
        return self.parent is None

    def add_child(self, child: "MessageNode") -> "MessageNode":
        child.parent = self
        self.children.append(child)
        return child

    def path_from_root(self) -> list["MessageNode"]:
        out, n = [], self
        while n is not None and not n.is_root:
            out.append(n)
            n = n.parent
        return out[::-1]

    def leaves(self):
        stack = [self]
        while stack:
            n = stack.pop()
            if n.children:
                stack.extend(reversed(n.children))
            else:
                yield n


def _common_prefix_len(a: list[int], b: list[int], block: int = 4096) -> int:
    """Length of the shared prefix; compares slices first so long equal prefixes cost one memcmp per block."""
    n = min(len(a), len(b))
    i = 0
    while i < n:
        j = min(i + block, n)
        if a[i:j] == b[i:j]:
            i = j
            continue
        while a[i] == b[i]:
            i += 1
        return i
    return n


class DriftKind(enum.Enum):
    CLEAN = "clean"
    REALIGN = "realign"
    FORK = "fork"


class _SampleBuilder:
    """Tokens, loss mask and log-probs of one output row while turns are being packed into it."""

    def __init__(self, fork_threshold: int):
        self.fork_threshold = fork_threshold
        self.tokens: list[int] = []
        self.loss_mask: list[int] = []
        self.logprobs: list[float] = []
        self.last_response_start_idx: int | None = None
        self.leading_prompt_len = 0

    def classify_token_drift(self, turn: TurnRecord) -> DriftKind:
        agree = _common_prefix_len(self.tokens, turn.prompt_ids)
        if agree == len(self.tokens):
            return DriftKind.CLEAN
        start = self.last_response_start_idx
        if start is not None and agree >= start and len(turn.output_ids) < self.fork_threshold:
            return DriftKind.REALIGN
        return DriftKind.FORK

    def _extend(self, ids, mask: int, lps=None):
        self.tokens += ids
        self.loss_mask += [mask] * len(ids)
        self.logprobs += list(lps) if lps else [0.0] * len(ids)

    def append_turn(self, turn: TurnRecord, kind: DriftKind, *, trained: bool = True):
        assert kind is not DriftKind.FORK
        first = self.last_response_start_idx is None
        if kind is DriftKind.REALIGN:
            s = self.last_response_start_idx
            tail = turn.prompt_ids[s:]
            self.tokens[s:], self.loss_mask[s:], self.logprobs[s:] = tail, [0] * len(tail), [0.0] * len(tail)
        else:
            self._extend(turn.prompt_ids[len(self.tokens) :], 0)
        self.last_response_start_idx = len(self.tokens)
        self._extend(turn.output_ids, int(trained), turn.output_log_probs if trained else None)
        if first:
            self.leading_prompt_len = len(turn.prompt_ids)

    def has_trained_response(self) -> bool:
        return any(self.loss_mask[self.leading_prompt_len :])

    def to_sample(self, base: Sample, metadata: dict | None, max_sample_tokens: int = 0) -> Sample:
        cut = max_sample_tokens if max_sample_tokens and len(self.tokens) > max_sample_tokens else len(self.tokens)
        p = self.leading_prompt_len
        return Sample(index=base.index, group_index=base.group_index,
                      rollout_id=base.rollout_id if base.rollout_id is not None else base.index,
                      prompt=base.prompt, label=base.label, tokens=self.tokens[:cut], response_length=max(cut - p, 0),
                      loss_mask=self.loss_mask[p:cut], rollout_log_probs=self.logprobs[p:cut], reward=0.0,
                      status=Sample.Status.COMPLETED, metadata=dict(metadata or {}))  # fmt: skip


class TrajectoryManager:
    def __init__(self, *, fork_threshold_tokens: int | None = None):
        self._fork_threshold = 1024 if fork_threshold_tokens is None else fork_threshold_tokens
        self._trees: dict[str, MessageNode] = {}
        self._turn_count: dict[str, int] = {}

    # ---------------------------------------------------------------------- sessions
    def has_session(self, sid: str) -> bool:
        return sid in self._trees

    def turn_count(self, sid: str) -> int:
        return self._turn_count.get(sid, 0)

    def drop_session(self, sid: str) -> None:
        self._trees.pop(sid, None)
        self._turn_count.pop(sid, None)

    # ------------------------------------------------------------------------ record
    def record_turn(self, sid: str, *, turn: TurnRecord, prompt_messages: list[dict[str, Any]],
                    response_message: dict[str, Any] | None, metadata: dict[str, Any] | None = None) -> None:  # fmt: skip
        if not prompt_messages:
            logger.warning("record_turn(%s): no prompt messages, turn ignored", sid)
            return
        if turn.output_log_probs and len(turn.output_log_probs) != len(turn.output_ids):
            raise AssertionError(f"{len(turn.output_log_probs)} log-probs for {len(turn.output_ids)} output tokens")
        root = self._trees.setdefault(sid, MessageNode())
        node, depth = self._find_mount_point(root, prompt_messages)
        node, depth = self._try_merge_assistant_rewrite(sid, node, prompt_messages, depth)
        for m in prompt_messages[depth:]:
            node = node.add_child(MessageNode(m.get("role"), m))
        leaf = node.add_child(MessageNode("assistant", response_message, metadata))
        leaf.turn = turn
        leaf.turn_index = self._turn_count[sid] = self._turn_count.get(sid, 0) + 1

    @staticmethod
    def _find_mount_point(root: MessageNode, messages: list[dict]) -> tuple[MessageNode, int]:
        node, depth = root, 0
        for msg in messages:
            nxt = next((c for c in node.children if c.role == msg.get("role") and c.message == msg), None)
            if nxt is None:
                break
            node, depth = nxt, depth + 1
        return node, depth

    def _try_merge_assistant_rewrite(self, sid, node, prompt_messages, depth):
        if self._fork_threshold <= 0 or depth >= len(prompt_messages) or prompt_messages[depth].get("role") != "assistant":
            return node, depth
        candidates = [c for c in node.children if c.role == "assistant"]
        if len(candidates) != 1:
            if len(candidates) > 1:
                logger.warning("record_turn(%s): %d assistant children at the mount point, forking", sid, len(candidates))
            return node, depth
        old = candidates[0]
        if old.children or old.turn is None or len(old.turn.output_ids) >= self._fork_threshold:
            return node, depth  # has descendants, was not generated here, or is long enough to deserve its own row
        old.metadata["merged_rewrite"] = {"abandoned_turn_index": old.turn_index,
                                          "abandoned_response_tokens": len(old.turn.output_ids)}  # fmt: skip
        old.turn = old.turn_index = None
        old.message = prompt_messages[depth]
        return old, depth + 1

    # --------------------------------------------------------------------- linearise
    def get_trajectory(self, sid: str, *, base_sample: Sample, reward: float = 0.0, extra_metadata: dict | None = None,
                       max_sample_tokens: int = 0) -> list[Sample]:  # fmt: skip
        """Rows of the whole session (every row gets the full outcome ``reward``); the session is consumed."""
        root = self._trees.get(sid)
        if root is None:
            return []
        out: list[Sample] = []
        for leaf in root.leaves():
            if not leaf.is_root:
                out += self._chain_to_samples(leaf.path_from_root(), base_sample, extra_metadata, max_sample_tokens)
        for s in out:
            s.reward = reward
        self.drop_session(sid)
        return out

    def _split_chain_into_builders(self, chain: list[MessageNode]) -> list[_SampleBuilder]:
        rows: list[_SampleBuilder] = []
        for n in chain:
            if n.role != "assistant" or n.turn is None:
                continue
            trained, n.response_trained = not n.response_trained, True
            kind = rows[-1].classify_token_drift(n.turn) if rows else DriftKind.FORK
            if kind is DriftKind.FORK:
                rows.append(_SampleBuilder(self._fork_threshold))
                kind = DriftKind.CLEAN
            rows[-1].append_turn(n.turn, kind, trained=trained)
        return rows

    def _chain_to_samples(self, chain, base_sample, extra_metadata, max_sample_tokens=0) -> list[Sample]:
        gen = [n for n in chain if n.role == "assistant" and n.turn is not None]
        md = {**(extra_metadata or {}),
              "truncated": bool(gen) and gen[-1].turn.finish_reason == "length",
              "use_tool": any(bool((n.message or {}).get("tool_calls")) for n in gen),
              "ill_formed": any(n.turn.ill_formed for n in gen)}  # fmt: skip
        return [b.to_sample(base_sample, md, max_sample_tokens) for b in self._split_chain_into_builders(chain)
                if b.has_trained_response()]  # fmt: skip
