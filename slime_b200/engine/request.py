"""Request and sampling-parameter types of the rollout engine (wire-compatible with the
``/generate`` payload described in slime/rollout/sglang_rollout.py:152-221)."""

from __future__ import annotations

import dataclasses
import time
from dataclasses import dataclass, field
from enum import Enum
from typing import Any


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    max_new_tokens: int = 128
    min_new_tokens: int = 0
    stop: list[str] | str | None = None
    stop_token_ids: list[int] | None = None
    ignore_eos: bool = False
    skip_special_tokens: bool = True
    no_stop_trim: bool = False
    spaces_between_special_tokens: bool = True
    sampling_seed: int | None = None
    repetition_penalty: float = 1.0
    n: int = 1
    custom_params: dict[str, Any] | None = None

    @classmethod
    def from_dict(cls, d: dict | None) -> "SamplingParams":
        d = dict(d or {})
        names = {f.name for f in dataclasses.fields(cls)}
        sp = cls(**{k: v for k, v in d.items() if k in names})
        if isinstance(sp.stop, str):
            sp.stop = [sp.stop]
        if sp.top_k is None or sp.top_k <= 0:
            sp.top_k = -1
        return sp

    @property
    def return_top_p_token_ids(self) -> bool:
        return bool((self.custom_params or {}).get("return_top_p_token_ids"))


class ReqState(Enum):
    WAITING = 0
    RUNNING = 1
    FINISHED = 2


@dataclass
class Request:
    rid: str
    input_ids: list[int]
    sampling: SamplingParams
    return_logprob: bool = True
    logprob_start_len: int = -1  # >=0: also return input-token log-probs from this position
    return_routed_experts: bool = False
    stream: bool = False
    prefill_only: bool = False  # prefill / decode disaggregation: stop after the first token and export the prompt's KV
    kv_export: Any = None  # (k, v) [layers, tokens, kv heads, head dim] of a finished prefill-only request
    gdn_state: Any = None  # {layer: (recurrent state, convolution history)} between prefill chunks, until a decode slot takes it
    mm: dict | None = None  # vision inputs: pixel_values + image_grid_thw (and the video pair) for the placeholder tokens of input_ids
    extra_meta: dict = field(default_factory=dict)  # added verbatim to meta_info (e.g. the pd_* transfer figures)
    # ---- engine state ----
    state: ReqState = ReqState.WAITING
    output_ids: list[int] = field(default_factory=list)
    output_logprobs: list[float] = field(default_factory=list)
    input_logprobs: list[float] | None = None
    pages: list[int] = field(default_factory=list)
    num_cached_tokens: int = 0  # prompt tokens served from the prefix cache
    num_computed: int = 0  # tokens whose KV is in the cache
    committed_pages: int = 0
    chain_hash: bytes = b""
    finish_reason: dict | None = None
    seed: int = 0
    kept_ids: list[int] = field(default_factory=list)
    kept_offsets: list[int] = field(default_factory=lambda: [0])
    routed_experts: list = field(default_factory=list)
    arrival: float = field(default_factory=time.time)
    first_scheduled: float | None = None
    first_token_time: float | None = None
    finish_time: float | None = None
    weight_version: str = "default"
    on_token: Any = None  # callback(req) for streaming
    done_event: Any = None
    text_so_far: str = ""
    # decode-slot bookkeeping (see Engine._start_decoding)
    ctx_ids: list[int] = field(default_factory=list)  # tokens to prefill (prompt, plus outputs after a retraction)
    slot: int | None = None
    decode_from_step: int = 0
    harvested: int = 0
    end_step: int | None = None
    end_reason: dict | None = None
    # speculative decoding (engine/speculative.py): guesses for the tokens after the last one, the draft head's stream
    mm_rows: Any = None  # positions of the placeholder tokens in input_ids (long tensor) ...
    mm_embeds: Any = None  # ... and the encoder's vector for each, computed at the first prefill pass
    mm_deepstack: Any = None  # vectors of the same rows that join the stream after the first layers (list, often empty)
    mm_positions: Any = None  # [3, len(input_ids)] temporal / height / width position streams of the prompt
    rope_delta: int = 0  # rotary position of a generated token = its index + rope_delta
    spec_draft: list[int] = field(default_factory=list)
    spec_hidden: Any = None

    @property
    def seq_len(self) -> int:
        return len(self.input_ids) + len(self.output_ids)

    def all_ids(self) -> list[int]:
        return self.input_ids + self.output_ids

    def finished(self) -> bool:
        return self.state == ReqState.FINISHED
