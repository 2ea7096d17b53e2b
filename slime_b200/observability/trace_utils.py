"""Per-sample tracing: spans and events recorded on ``Sample.trace`` and persisted with rollout dumps.

``Sample.trace = {"version", "trace_id", "sample_id", "group_id", "attempt", "events": [...]}``; a span is a
``span_start`` / ``span_end`` event pair linked by ``span_id`` with ``parent_span_id`` taken from a
``contextvars`` stack, so nested ``with trace_span(...)`` blocks form a tree per sample. Engine
``meta_info`` timings are folded into span attributes (and synthetic prefill/decode child spans for
disaggregated engines). Tracing never raises into the rollout path.
Parity: slime/observability/trace_utils.py:47-54 (schema), :146-216 (meta attrs), :351-431 (spans),
:457-619 (decorator, carrier helpers).
"""

from __future__ import annotations

import contextvars
import functools
import inspect
import logging
import time
import uuid
from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Any

logger = logging.getLogger(__name__)
TRACE_VERSION = 1
_span_stack: contextvars.ContextVar[tuple[str, ...]] = contextvars.ContextVar("slime_trace_span_stack", default=())

_META_KEYS = ("e2e_latency", "queue_time", "decode_throughput", "prompt_tokens", "completion_tokens", "cached_tokens",
              "weight_version", "spec_accept_token_num", "spec_draft_token_num", "spec_verify_ct")  # fmt: skip
_PD_KEYS = ("pd_prefill_queue_time", "pd_prefill_forward_time", "pd_bootstrap_time", "pd_transfer_time",
            "pd_decode_queue_time", "pd_transfer_speed_gb_s", "pd_transfer_total_mb", "pd_prefill_retry_count")  # fmt: skip


def _log_trace_error(where: str, e: BaseException):
    logger.debug("trace error in %s: %r", where, e)


def _new_id() -> str:
    return uuid.uuid4().hex[:16]


def _targets(target) -> list:
    """Normalise Sample | list[Sample] | nested lists into a flat list of trace carriers."""
    if target is None:
        return []
    if isinstance(target, (list, tuple)):
        out = []
        for t in target:
            out += _targets(t)
        return out
    return [target]


def ensure_trace(sample, attempt: int | None = None) -> dict:
    tr = getattr(sample, "trace", None)
    if not isinstance(tr, dict):
        tr = {"version": TRACE_VERSION, "trace_id": _new_id(), "sample_id": getattr(sample, "index", None),
              "group_id": getattr(sample, "group_index", None), "attempt": 0, "events": []}  # fmt: skip
        sample.trace = tr
    if attempt is not None:
        tr["attempt"] = attempt
    return tr


def trace_event(target, name: str, attrs: dict | None = None):
    try:
        now = time.time()
        for s in _targets(target):
            ensure_trace(s)["events"].append({"type": "event", "name": name, "ts": now, "attrs": dict(attrs or {}),
                                              "parent_span_id": (_span_stack.get() or (None,))[-1]})  # fmt: skip
    except Exception as e:  # noqa: BLE001
        _log_trace_error("trace_event", e)


@dataclass
class TraceHandle:
    """Returned by ``trace_span``: lets the body attach attributes that land on the ``span_end`` event."""

    span_id: str
    attrs: dict = field(default_factory=dict)

    def update(self, more: dict | None):
        if more:
            self.attrs.update(more)

    def set(self, key: str, value: Any):
        self.attrs[key] = value


@contextmanager
def trace_span(target, name: str, attrs: dict | None = None):
    handle = TraceHandle(_new_id())
    carriers = []
    token = None
    try:
        carriers = _targets(target)
        parent = (_span_stack.get() or (None,))[-1]
        start = time.time()
        for s in carriers:
            ensure_trace(s)["events"].append({"type": "span_start", "name": name, "span_id": handle.span_id,
                                              "parent_span_id": parent, "ts": start, "attrs": dict(attrs or {})})  # fmt: skip
        token = _span_stack.set(_span_stack.get() + (handle.span_id,))
    except Exception as e:  # noqa: BLE001
        _log_trace_error("trace_span.enter", e)
    error = None
    try:
        yield handle
    except BaseException as e:
        error = repr(e)
        raise
    finally:
        try:
            if token is not None:
                _span_stack.reset(token)
            end = time.time()
            for s in carriers:
                ev = {"type": "span_end", "name": name, "span_id": handle.span_id, "ts": end, "attrs": dict(handle.attrs)}
                if error:
                    ev["error"] = error
                ensure_trace(s)["events"].append(ev)
        except Exception as e:  # noqa: BLE001
            _log_trace_error("trace_span.exit", e)


def trace_function(name: str, target: str = "sample", attrs_getter=None):
    """Decorator for (async) functions whose argument ``target`` is a Sample / group: wraps the call in a span."""

    def deco(fn):
        sig = inspect.signature(fn)

        def carrier(args, kwargs):
            try:
                bound = sig.bind_partial(*args, **kwargs)
                return bound.arguments.get(target) or bound.arguments.get("group") or bound.arguments.get("sample")
            except TypeError:
                return None

        def span_attrs(args, kwargs):
            try:
                return attrs_getter(*args, **kwargs) if attrs_getter else None
            except Exception:  # noqa: BLE001
                return None

        if inspect.iscoroutinefunction(fn):

            @functools.wraps(fn)
            async def awrapper(*args, **kwargs):
                with trace_span(carrier(args, kwargs), name, span_attrs(args, kwargs)):
                    return await fn(*args, **kwargs)

            return awrapper

        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            with trace_span(carrier(args, kwargs), name, span_attrs(args, kwargs)):
                return fn(*args, **kwargs)

        return wrapper

    return deco


def build_sglang_meta_trace_attrs(meta_info: dict | None) -> dict:
    """Engine timings worth keeping on the generate span."""
    if not meta_info:
        return {}
    out = {k: meta_info[k] for k in _META_KEYS + _PD_KEYS if k in meta_info}
    fr = meta_info.get("finish_reason")
    if isinstance(fr, dict):
        out["finish_reason"] = fr.get("type")
    return out


def build_pd_child_spans(meta_info: dict, start_ts: float) -> list[dict]:
    """Synthetic prefill -> transfer -> decode child spans from ``pd_*`` durations of a disaggregated engine."""
    spans, t = [], start_ts
    for name, key in (("pd_prefill_queue", "pd_prefill_queue_time"), ("pd_prefill_forward", "pd_prefill_forward_time"),
                      ("pd_bootstrap", "pd_bootstrap_time"), ("pd_transfer", "pd_transfer_time"),
                      ("pd_decode_queue", "pd_decode_queue_time")):  # fmt: skip
        d = meta_info.get(key)
        if d is None:
            continue
        spans.append({"name": name, "start": t, "end": t + float(d)})
        t += float(d)
    return spans


def export_spans(sample) -> list[dict]:
    """Pair span_start / span_end events into ``{name, span_id, parent_span_id, start, end, attrs}`` records."""
    tr = getattr(sample, "trace", None)
    if not isinstance(tr, dict):
        return []
    open_, out = {}, []
    for ev in tr.get("events", []):
        if ev.get("type") == "span_start":
            open_[ev["span_id"]] = ev
        elif ev.get("type") == "span_end" and ev.get("span_id") in open_:
            st = open_.pop(ev["span_id"])
            out.append({"name": st["name"], "span_id": st["span_id"], "parent_span_id": st.get("parent_span_id"),
                        "start": st["ts"], "end": ev["ts"], "attrs": {**st.get("attrs", {}), **ev.get("attrs", {})},
                        **({"error": ev["error"]} if "error" in ev else {})})  # fmt: skip
    return out
