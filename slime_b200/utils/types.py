"""The rollout <-> training data contract.

``Sample`` is what a rollout function produces and what the trainer consumes.
Field names, ``to_dict``/``from_dict`` and ``append_response_tokens`` follow the
public contract of slime/utils/types.py:93-443 so custom rollout functions and
reward hooks written against it keep working.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from enum import Enum
from typing import Any

import torch

from slime_b200.utils.misc import decode_int32_meta_array

_TOPP_ID_KEYS = ("top_p_token_ids", "top_p_kept_token_ids")
_TOPP_OFF_KEYS = ("top_p_token_offsets", "top_p_kept_token_offsets")

_FINISH_TO_STATUS = {"length": "truncated", "abort": "aborted", "stop": "completed"}


def _ints(x) -> list[int]:
    if x is None:
        return []
    if torch.is_tensor(x):
        return [int(v) for v in x.detach().cpu().reshape(-1).tolist()]
    return [int(v) for v in x]


def _floats(x) -> list[float] | None:
    if x is None:
        return None
    if torch.is_tensor(x):
        return [float(v) for v in x.detach().cpu().reshape(-1).tolist()]
    return [float(v) for v in x]


def _i32(x, default) -> torch.Tensor:
    return torch.as_tensor(default if x is None else x, dtype=torch.int32).reshape(-1)


class RaggedTopP:
    """Ragged per-token id lists (CSR form) used by top-p keep-mask replay.

    Token ``i`` kept ids are ``ids[offsets[i]:offsets[i+1]]``.
    """

    @staticmethod
    def parse(meta_info: dict, expected_tokens: int | None):
        ids = decode_int32_meta_array(meta_info, _TOPP_ID_KEYS)
        offs = decode_int32_meta_array(meta_info, _TOPP_OFF_KEYS)
        if ids is None and offs is None:
            return None
        if ids is None or offs is None:
            raise ValueError("top-p token replay must include both token ids and offsets.")
        if offs.numel() == 0 or int(offs[0]) != 0:
            raise ValueError(f"top-p token offsets must start with 0, got {offs[:1].tolist()}.")
        if int(offs[-1]) != ids.numel():
            raise ValueError(
                f"top-p token ids/offsets mismatch: offsets[-1]={int(offs[-1])}, len(token_ids)={ids.numel()}."
            )
        if expected_tokens is not None and offs.numel() != expected_tokens + 1:
            raise ValueError(
                "top-p token offsets length must equal generated token count + 1: "
                f"len(offsets)={offs.numel()}, generated={expected_tokens}."
            )
        return ids, offs

    @staticmethod
    def concat(base_ids, base_offs, ids, offs):
        b_ids = _i32(base_ids, [])
        b_offs = _i32(base_offs, [0])
        shift = int(b_offs[-1])
        return torch.cat([b_ids, ids]), torch.cat([b_offs, offs[1:] + shift])

    @staticmethod
    def pad_empty(ids, offs, n: int):
        if ids is None or offs is None:
            raise ValueError("Cannot append empty top-p spans without existing token ids and offsets.")
        if n < 0:
            raise ValueError(f"num_tokens must be non-negative, got {n}.")
        ids_t, offs_t = _i32(ids, []), _i32(offs, [])
        if offs_t.numel() == 0:
            raise ValueError("Cannot append empty top-p spans to empty offsets.")
        if n == 0:
            return ids_t, offs_t
        return ids_t, torch.cat([offs_t, offs_t.new_full((n,), int(offs_t[-1]))])


class SampleStatus(Enum):
    PENDING = "pending"
    COMPLETED = "completed"
    TRUNCATED = "truncated"
    ABORTED = "aborted"
    # recoverable failure (tool error, API error): partial output may be valid
    FAILED = "failed"


@dataclass
class SpecInfo:
    """Speculative-decoding counters accumulated over the turns of one sample."""

    spec_accept_token_num: int = 0
    spec_draft_token_num: int = 0
    spec_verify_ct: int = 0
    completion_token_num: int = 0

    @property
    def spec_accept_rate(self) -> float:
        return self.spec_accept_token_num / self.spec_draft_token_num if self.spec_draft_token_num > 0 else 0.0

    @property
    def spec_accept_length(self) -> float:
        return self.completion_token_num / self.spec_verify_ct if self.spec_verify_ct > 0 else 0.0

    def add(self, meta_info: dict):
        self.spec_accept_token_num += meta_info.get("spec_accept_token_num", 0)
        self.spec_draft_token_num += meta_info.get("spec_draft_token_num", 0)
        self.spec_verify_ct += meta_info.get("spec_verify_ct", 0)
        self.completion_token_num += meta_info.get("completion_tokens", 0)

    def to_dict(self):
        return dataclasses.asdict(self)

    @staticmethod
    def from_dict(data: dict):
        return SpecInfo(**{f.name: data.get(f.name, 0) for f in dataclasses.fields(SpecInfo)})


@dataclass
class PrefixCacheInfo:
    cached_tokens: int = 0
    total_prompt_tokens: int = 0

    @property
    def prefix_cache_hit_rate(self) -> float:
        return self.cached_tokens / self.total_prompt_tokens if self.total_prompt_tokens > 0 else 0.0

    def add(self, meta_info: dict):
        self.cached_tokens += meta_info.get("cached_tokens", 0)
        self.total_prompt_tokens += meta_info.get("prompt_tokens", 0)

    def to_dict(self):
        return dataclasses.asdict(self)

    @staticmethod
    def from_dict(data: dict):
        return PrefixCacheInfo(data.get("cached_tokens", 0), data.get("total_prompt_tokens", 0))


@dataclass
class Sample:
    """One generated (or to-be-generated) sequence plus its training metadata."""

    group_index: int | None = None
    index: int | None = None
    # All training samples split out of one rollout execution share rollout_id;
    # consumers fall back to ``index`` when it is None.
    rollout_id: int | None = None
    prompt: str | list[dict[str, str]] = ""
    tokens: list[int] = field(default_factory=list)  # prompt + response ids
    multimodal_inputs: dict[str, Any] | None = None
    multimodal_train_inputs: dict[str, Any] | None = None
    multimodal_train_input_id: str | None = None
    apply_chat_template_kwargs: dict = field(default_factory=dict)
    response: str = ""
    response_length: int = 0
    label: str | None = None
    reward: float | dict[str, Any] | None = None
    loss_mask: list[int] | None = None
    weight_versions: list[str] = field(default_factory=list)
    rollout_log_probs: list[float] | None = None
    rollout_top_p_token_ids: list[int] | torch.Tensor | None = None
    rollout_top_p_token_offsets: list[int] | torch.Tensor | None = None
    rollout_routed_experts: list[list[int]] | torch.Tensor | None = None
    remove_sample: bool = False
    teacher_log_probs: list[float] | None = None

    Status = SampleStatus
    SpecInfo = SpecInfo
    PrefixCacheInfo = PrefixCacheInfo

    status: SampleStatus = SampleStatus.PENDING
    metadata: dict = field(default_factory=dict)
    generate_function_path: str | None = None
    custom_rm_path: str | None = None
    train_metadata: dict | None = None
    session_id: str | None = None
    non_generation_time: float = 0.0
    spec_info: SpecInfo = field(default_factory=SpecInfo)
    prefix_cache_info: PrefixCacheInfo = field(default_factory=PrefixCacheInfo)

    # ------------------------------------------------------------------ serde
    def to_dict(self) -> dict:
        out = dict(self.__dict__)
        out["status"] = self.status.value
        out["spec_info"] = self.spec_info.to_dict()
        out["prefix_cache_info"] = self.prefix_cache_info.to_dict()
        return out

    @staticmethod
    def from_dict(data: dict) -> "Sample":
        known = {f.name for f in dataclasses.fields(Sample)}
        kw, extra = {}, {}
        for k, v in data.items():
            (kw if k in known else extra)[k] = v
        kw["status"] = SampleStatus(kw["status"])
        kw["spec_info"] = SpecInfo.from_dict(kw.get("spec_info") or {})
        kw["prefix_cache_info"] = PrefixCacheInfo.from_dict(kw.get("prefix_cache_info") or {})
        s = Sample(**kw)
        for k, v in extra.items():
            setattr(s, k, v)
        return s

    # --------------------------------------------------------------- accessors
    def get_reward_value(self, args) -> float:
        key = getattr(args, "reward_key", None)
        return self.reward[key] if key else self.reward

    @property
    def effective_response_length(self) -> int:
        return self.response_length if self.loss_mask is None else sum(self.loss_mask)

    # ---------------------------------------------------------------- mutation
    def append_response_tokens(
        self,
        args=None,
        *,
        tokens=None,
        log_probs=None,
        trainable: bool = True,
        meta_info: dict | None = None,
        text: str | None = None,
        update_terminal_info: bool = True,
    ):
        """Append response-side tokens keeping loss mask / logprobs / top-p spans aligned.

        Model tokens: ``trainable=True`` with engine ``meta_info`` and logprobs.
        Tool/environment tokens: ``trainable=False``; they get loss-mask zeros,
        logprob 0.0 and empty top-p spans.
        """
        new_tokens = _ints(tokens)
        lps = _floats(log_probs)
        n_new = len(new_tokens)
        if lps is not None and len(lps) != n_new:
            raise ValueError(f"log_probs length {len(lps)} != tokens length {n_new}")
        if n_new and trainable and lps is None:
            raise ValueError("trainable response tokens require rollout log probabilities.")
        if n_new and not trainable:
            if lps is not None:
                raise ValueError("non-trainable response tokens should not pass rollout log probabilities.")
            lps = [0.0] * n_new

        if text is not None:
            self.response += text

        prev_len = self.response_length
        if n_new:
            self.tokens = self.tokens + new_tokens
            self.response_length = prev_len + n_new
            if self.loss_mask is None:
                self.loss_mask = [1] * prev_len
            self.loss_mask = self.loss_mask + [int(trainable)] * n_new

        if lps is not None:
            if self.rollout_log_probs is None:
                if trainable and prev_len:
                    raise ValueError(
                        "Cannot append trainable rollout log probabilities to a sample with existing response "
                        "tokens but no existing rollout_log_probs."
                    )
                self.rollout_log_probs = [0.0] * prev_len
            self.rollout_log_probs = self.rollout_log_probs + lps

        pad_topp = bool(n_new and not trainable)
        if meta_info is not None or pad_topp:
            self._absorb_meta(args, meta_info or {}, n_new, pad_topp, update_terminal_info)
        self._check_lengths()

    def _absorb_meta(self, args, meta: dict, n_new: int, pad_topp: bool, terminal: bool) -> None:
        got_topp = False
        if n_new:
            parsed = RaggedTopP.parse(meta, n_new)
            if parsed is not None:
                got_topp = True
                if self.rollout_top_p_token_ids is None and self.rollout_top_p_token_offsets is None:
                    self.rollout_top_p_token_ids, self.rollout_top_p_token_offsets = parsed
                else:
                    self.rollout_top_p_token_ids, self.rollout_top_p_token_offsets = RaggedTopP.concat(
                        self.rollout_top_p_token_ids, self.rollout_top_p_token_offsets, *parsed
                    )
        if pad_topp and n_new and not got_topp and self.rollout_top_p_token_offsets is not None:
            self.rollout_top_p_token_ids, self.rollout_top_p_token_offsets = RaggedTopP.pad_empty(
                self.rollout_top_p_token_ids, self.rollout_top_p_token_offsets, n_new
            )

        self._absorb_routed_experts(args, meta)

        if not terminal or "finish_reason" not in meta:
            return
        if getattr(args, "sglang_speculative_algorithm", False):
            self.spec_info.add(meta)
        self.prefix_cache_info.add(meta)
        if "weight_version" in meta:
            self.weight_versions.append(meta["weight_version"])
        mapped = _FINISH_TO_STATUS.get(meta["finish_reason"].get("type"))
        if mapped is not None:
            self.status = SampleStatus(mapped)

    def _absorb_routed_experts(self, args, meta: dict) -> None:
        flat = decode_int32_meta_array(meta, "routed_experts")
        if flat is None:
            return
        if args is None:
            raise ValueError("args is required to decode routed experts metadata.")
        start = int(meta.get("routed_experts_start_len", 0) or 0)
        if start < 0:
            raise ValueError(f"routed_experts_start_len must be non-negative, got {start}.")
        rows = max(0, len(self.tokens) - 1 - start)
        want = rows * args.num_layers * args.moe_router_topk
        if flat.numel() != want:
            raise ValueError(
                f"routed_experts element count does not match sample tokens: got={flat.numel()}, expected={want} "
                f"(tokens={len(self.tokens)}, routed_experts_start_len={start}, num_layers={args.num_layers}, "
                f"moe_router_topk={args.moe_router_topk})."
            )
        block = flat.reshape(rows, args.num_layers, args.moe_router_topk)
        if start == 0:
            self.rollout_routed_experts = block
            return
        prev = self.rollout_routed_experts
        if prev is None:
            raise ValueError(
                f"Cannot append partial routed experts without existing routed experts (routed_experts_start_len={start})."
            )
        prev = prev if torch.is_tensor(prev) else torch.as_tensor(prev, dtype=block.dtype)
        if prev.shape[0] < start:
            raise ValueError(
                f"Existing routed experts shorter than routed_experts_start_len: existing_rows={prev.shape[0]}, "
                f"routed_experts_start_len={start}."
            )
        self.rollout_routed_experts = torch.cat([prev[:start], block], dim=0)

    def _check_lengths(self) -> None:
        if self.loss_mask is not None and len(self.loss_mask) != self.response_length:
            raise ValueError(f"loss_mask length {len(self.loss_mask)} != response_length {self.response_length}")
        if self.rollout_log_probs is not None and len(self.rollout_log_probs) != self.response_length:
            raise ValueError(
                f"rollout_log_probs length {len(self.rollout_log_probs)} != response_length {self.response_length}"
            )
        ids, offs = self.rollout_top_p_token_ids, self.rollout_top_p_token_offsets
        if ids is None and offs is None:
            return
        if ids is None or offs is None:
            raise ValueError("rollout top-p replay must include both token ids and offsets.")
        offs_t = _i32(offs, [])
        if offs_t.numel() != self.response_length + 1:
            raise ValueError(
                "rollout_top_p_token_offsets length must equal response_length + 1: "
                f"len(offsets)={offs_t.numel()}, response_length={self.response_length}."
            )
        n_ids = int(torch.as_tensor(ids).reshape(-1).numel())
        if int(offs_t[-1]) != n_ids:
            raise ValueError(
                f"rollout top-p token ids/offsets mismatch: offsets[-1]={int(offs_t[-1])}, len(token_ids)={n_ids}."
            )


@dataclass(frozen=True)
class ParamInfo:
    """Metadata of one trainer parameter exchanged once before weight sync."""

    name: str
    dtype: torch.dtype
    shape: torch.Size
    attrs: dict
    size: int
    src_rank: int


RolloutBatch = dict[str, "list[torch.Tensor] | list[int] | list[float] | list[str]"]


@dataclass
class MultimodalType:
    name: str
    placeholder: str


class MultimodalTypes:
    IMAGE = MultimodalType("image", "<image>")
    VIDEO = MultimodalType("video", "<video>")
    AUDIO = MultimodalType("audio", "<audio>")

    @classmethod
    def all(cls) -> list[MultimodalType]:
        return [cls.IMAGE, cls.VIDEO, cls.AUDIO]

    @classmethod
    def get(cls, name: str) -> MultimodalType | None:
        for m in cls.all():
            if m.name == name:
                return m
        return None
