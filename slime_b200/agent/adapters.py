"""Chat-protocol front ends for agent harnesses: OpenAI ``/v1/chat/completions`` and Anthropic ``/v1/messages``.

An agent framework (a coding agent, a tool-use loop, ...) is pointed at one of these servers instead of a vendor API.
Every request is one *turn* of a session:

    request -> normalise to chat messages (+ tool schemas) -> chat template -> token ids
            -> rollout engine ``/generate`` with ``return_logprob`` (token ids in, token ids and log-probs out)
            -> parse reasoning / tool calls out of the text -> protocol-shaped reply (JSON or SSE)
            -> ``TrajectoryManager.record_turn`` with the exact ids and log-probs

so that when the episode ends ``finish_session`` returns loss-masked ``Sample`` rows built from what the engine really
produced, never from re-tokenised text. Sessions are keyed by the bearer token (``Authorization: Bearer <sid>``), the
``user`` / ``metadata.user_id`` body field, or ``"default"``. A reply is flushed to the client *before* the turn is
recorded: a client that disconnected mid-generation never acted on that turn, so it must not be trained on.
Parity: slime/agent/adapters/{common,openai,anthropic}.py.
"""

from __future__ import annotations

import asyncio
import dataclasses
import json
import logging
import time
import uuid
from typing import Any, Callable

import aiohttp
from aiohttp import web

from slime_b200.agent.parsing import ParsedModelOutput, parse_model_output
from slime_b200.agent.trajectory import TrajectoryManager, TurnRecord

logger = logging.getLogger(__name__)


@dataclasses.dataclass
class Session:
    sampling_defaults: dict = dataclasses.field(default_factory=dict)
    max_context_tokens: int = 0


@dataclasses.dataclass
class Reply:
    """What goes back on the wire plus the chat message stored in the session tree."""

    manager_message: dict
    wire: Any
    finish: str


def flatten_content(c: Any) -> str:
    """Chat content as plain text: strings pass, lists of typed parts keep their text parts."""
    if c is None:
        return ""
    if isinstance(c, str):
        return c
    if isinstance(c, list):
        parts = []
        for p in c:
            if isinstance(p, str):
                parts.append(p)
            elif isinstance(p, dict):
                if p.get("type") in ("text", "input_text", "output_text"):
                    parts.append(p.get("text", ""))
                elif p.get("type") == "tool_result":
                    parts.append(flatten_content(p.get("content")))
        return "\n".join(x for x in parts if x)
    return str(c)


def tool_call_dict(name: str, arguments: dict | None, call_id: str | None = None) -> dict:
    return {"id": call_id or f"call_{uuid.uuid4().hex[:24]}", "type": "function",
            "function": {"name": name, "arguments": arguments or {}}}  # fmt: skip


def sid_from_bearer(request: web.Request) -> str | None:
    auth = request.headers.get("Authorization", "")
    if auth.lower().startswith("bearer "):
        return auth[7:].strip() or None
    return request.headers.get("x-api-key") or None


def sid_from_body(body: dict | None) -> str | None:
    if not isinstance(body, dict):
        return None
    if isinstance(body.get("user"), str):
        return body["user"]
    md = body.get("metadata")
    if isinstance(md, dict):
        return md.get("user_id") or md.get("session_id")
    return None


def _render_token_ids(messages, tokenizer, tools=None, add_generation_prompt=True) -> list[int]:
    kw = {"tools": tools} if tools else {}
    ids = tokenizer.apply_chat_template(messages, tokenize=True, add_generation_prompt=add_generation_prompt, **kw)
    return list(ids["input_ids"] if isinstance(ids, dict) else ids)


def _sampling_params(session: Session, body: dict, max_token_keys, stop_keys) -> dict:
    sp = {"skip_special_tokens": False, "spaces_between_special_tokens": False, "no_stop_trim": True,
          "max_new_tokens": 4096, **(session.sampling_defaults or {})}  # fmt: skip
    for k in max_token_keys:
        if body.get(k) is not None:
            sp["max_new_tokens"] = min(int(sp["max_new_tokens"]), int(body[k]))
            break
    for k in ("temperature", "top_p", "top_k"):
        if k in body and body[k] is not None:
            sp[k] = body[k]
    for k in stop_keys:
        if body.get(k):
            sp["stop"] = body[k]
            break
    return sp


async def call_engine_generate(prompt_ids: list[int], session: Session, body: dict, *, adapter: "BaseAdapter",
                               session_id: str | None = None) -> TurnRecord:  # fmt: skip
    """One ``/generate`` round trip. Module-level so tests can replace it. On cancel / transport errors the request
    is aborted on the engine so an orphaned generation does not sit on KV pages until its length cap."""
    sp = _sampling_params(session, body, adapter.max_token_keys, adapter.stop_keys)
    if session.max_context_tokens > 0:
        room = session.max_context_tokens - len(prompt_ids)
        if room <= 0:
            return TurnRecord(prompt_ids=list(prompt_ids), output_ids=[], finish_reason="length")
        sp["max_new_tokens"] = min(int(sp["max_new_tokens"]), room)
    rid = uuid.uuid4().hex
    headers = {"X-SMG-Routing-Key": session_id} if session_id and session_id != "default" else None
    url = adapter.engine_url
    try:
        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=None, sock_read=900)) as http:
            async with http.post(f"{url}/generate", headers=headers, json={
                    "rid": rid, "input_ids": prompt_ids, "sampling_params": sp, "return_logprob": True}) as r:  # fmt: skip
                if r.status >= 400:
                    raise RuntimeError(f"engine answered {r.status}: {(await r.text())[:400]}")
                data = await r.json(content_type=None)
    except (asyncio.CancelledError, aiohttp.ClientError, asyncio.TimeoutError):
        try:
            async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=5)) as http:
                await http.post(f"{url}/abort_request", json={"rid": rid})
        except Exception:  # noqa: BLE001
            pass
        raise
    meta = data.get("meta_info") or {}
    pairs = meta.get("output_token_logprobs") or []
    return TurnRecord(prompt_ids=list(prompt_ids), output_ids=[p[1] for p in pairs], finish_reason=(meta.get("finish_reason") or {}).get("type") or "stop",
                      output_log_probs=[float(p[0]) for p in pairs])  # fmt: skip


class BaseAdapter:
    log_prefix = "adapter"
    max_token_keys: tuple[str, ...] = ()
    stop_keys: tuple[str, ...] = ()

    def __init__(self, *, tokenizer, engine_url: str, tool_parser=None, reasoning_parser=None, max_turns_per_sid: int | None = None,
                 fork_threshold_tokens: int | None = None, debug_callback: Callable[..., None] | None = None):  # fmt: skip
        self.tokenizer, self.engine_url = tokenizer, engine_url.rstrip("/")
        self.tool_parser, self.reasoning_parser = tool_parser, reasoning_parser
        self.store: dict[str, Session] = {}
        self.inflight: dict[str, set[asyncio.Task]] = {}
        self.closed: set[str] = set()
        self.manager = TrajectoryManager(fork_threshold_tokens=fork_threshold_tokens)
        self.max_turns_per_sid, self.debug_callback = max_turns_per_sid, debug_callback
        self._turns: dict[str, int] = {}
        self.app = web.Application(client_max_size=64 * 1024 * 1024)
        self.app.router.add_get("/healthz", self._health)
        self.app.router.add_get("/v1/models", self._health)
        self._register_routes(self.app)

    async def _health(self, _request):
        return web.json_response({"ok": True, "object": "list", "data": [{"id": "policy", "object": "model"}]})

    # -- protocol hooks --------------------------------------------------------
    def _register_routes(self, app):
        raise NotImplementedError

    def _session_id(self, request, body) -> str:
        return sid_from_bearer(request) or sid_from_body(body) or "default"

    def _preprocess_body(self, body: dict) -> None:
        pass

    def _translate(self, body: dict) -> tuple[list[dict], list[dict] | None]:
        raise NotImplementedError

    def _build_reply(self, parsed: ParsedModelOutput, raw_finish: str, translated, tools_schema) -> Reply:
        raise NotImplementedError

    async def _respond(self, request, body, reply: Reply, in_tok: int, out_tok: int, stream: bool):
        raise NotImplementedError

    # -- sessions ----------------------------------------------------------------
    def open_session(self, sid: str, *, sampling_defaults: dict | None = None, max_context_tokens: int = 0) -> None:
        if sid in self.store:
            raise ValueError(f"session id {sid!r} is already open; ids must be unique per agent run")
        self.closed.discard(sid)
        self.store[sid] = Session(dict(sampling_defaults or {}), int(max_context_tokens or 0))

    async def shutdown_session(self, sid: str, *, wait_timeout: float = 5.0) -> None:
        """Refuse new requests for ``sid`` and give requests in flight ``wait_timeout`` seconds, then cancel them."""
        self.closed.add(sid)
        tasks = [t for t in self.inflight.get(sid, ()) if not t.done()]
        if tasks:
            _done, pending = await asyncio.wait(tasks, timeout=wait_timeout)
            for t in pending:
                t.cancel()
        self.inflight.pop(sid, None)

    async def finish_session(self, sid: str, *, base_sample, reward: float = 0.0, extra_metadata: dict | None = None,
                             wait_timeout: float = 5.0) -> list:  # fmt: skip
        await self.shutdown_session(sid, wait_timeout=wait_timeout)
        session = self.store.pop(sid, None)
        self._turns.pop(sid, None)
        samples = self.manager.get_trajectory(sid, base_sample=base_sample, reward=reward, extra_metadata=extra_metadata,
                                              max_sample_tokens=session.max_context_tokens if session else 0)  # fmt: skip
        for s in samples:
            n = int(s.response_length or 0)
            s.response = self.tokenizer.decode(s.tokens[-n:], skip_special_tokens=False) if n and s.tokens else ""
        return samples

    async def drop_session(self, sid: str, *, wait_timeout: float = 5.0) -> None:
        await self.shutdown_session(sid, wait_timeout=wait_timeout)
        self.store.pop(sid, None)
        self._turns.pop(sid, None)
        self.manager.drop_session(sid)

    # -- one turn ------------------------------------------------------------------
    async def _run_turn(self, request: web.Request) -> web.StreamResponse:
        body = await request.json()
        self._preprocess_body(body)
        sid = self._session_id(request, body)
        if sid in self.closed:
            return web.Response(status=503, text="session closed")
        if self.max_turns_per_sid is not None:
            self._turns[sid] = self._turns.get(sid, 0) + 1
            if self._turns[sid] > self.max_turns_per_sid:
                return web.json_response({"error": {"type": "rate_limit_error", "message": f"turn cap {self.max_turns_per_sid} reached"}},
                                         status=429)  # fmt: skip
        session = self.store.setdefault(sid, Session())
        task = asyncio.current_task()
        self.inflight.setdefault(sid, set()).add(task)
        t0 = time.monotonic()
        try:
            translated, tools = self._translate(body)
            prompt_ids = _render_token_ids(translated, self.tokenizer, tools)
            turn = await call_engine_generate(prompt_ids, session, body, adapter=self, session_id=sid)
            raw = self.tokenizer.decode(turn.output_ids, skip_special_tokens=False) if turn.output_ids else ""
            parsed = parse_model_output(raw, tools, self.tool_parser, self.reasoning_parser)
            reply = self._build_reply(parsed, turn.finish_reason, translated, tools)
            turn = dataclasses.replace(turn, ill_formed=parsed.ill_formed)
            stream = body.get("stream") is True or "text/event-stream" in request.headers.get("Accept", "")
            try:
                response = await self._respond(request, body, reply, len(prompt_ids), len(turn.output_ids), stream)
            except ConnectionResetError:
                logger.warning("[%s] sid=%s client went away before the reply was flushed (%.1fs)", self.log_prefix, sid,
                               time.monotonic() - t0)  # fmt: skip
                return web.Response(status=499, text="client disconnected")
            if self.debug_callback is not None:
                try:
                    self.debug_callback(sid, translated, tools, reply.manager_message, turn)
                except Exception:  # noqa: BLE001
                    logger.exception("debug callback failed")
            self.manager.record_turn(sid, turn=turn, prompt_messages=translated, response_message=reply.manager_message,
                                     metadata={"sid": sid})  # fmt: skip
            return response
        finally:
            self.inflight.get(sid, set()).discard(task)


async def _sse(request, events) -> web.StreamResponse:
    resp = web.StreamResponse(headers={"Content-Type": "text/event-stream", "Cache-Control": "no-cache"})
    await resp.prepare(request)
    for name, data in events:
        head = f"event: {name}\n" if name else ""
        payload = data if isinstance(data, str) else json.dumps(data)
        await resp.write(f"{head}data: {payload}\n\n".encode())
    await resp.write_eof()
    return resp


# ------------------------------------------------------------------------------------- OpenAI
def _openai_messages(messages: list[dict]) -> list[dict]:
    out = []
    for m in messages:
        role = "system" if m.get("role") == "developer" else m.get("role")
        msg = {"role": role, "content": flatten_content(m.get("content"))}
        if role == "assistant" and m.get("tool_calls"):
            calls = []
            for c in m["tool_calls"]:
                fn = c.get("function", {})
                args = fn.get("arguments")
                if isinstance(args, str):
                    try:
                        args = json.loads(args) if args.strip() else {}
                    except ValueError:
                        args = {"_raw": args}
                calls.append(tool_call_dict(fn.get("name", ""), args, c.get("id")))
            msg["tool_calls"] = calls
        if role == "tool" and m.get("tool_call_id"):
            msg["tool_call_id"] = m["tool_call_id"]
        out.append(msg)
    return out


class OpenAIAdapter(BaseAdapter):
    log_prefix = "openai"
    max_token_keys = ("max_completion_tokens", "max_tokens")
    stop_keys = ("stop",)

    def _register_routes(self, app):
        app.router.add_post("/v1/chat/completions", self._run_turn)
        app.router.add_post("/chat/completions", self._run_turn)

    def _translate(self, body):
        tools = [t for t in (body.get("tools") or []) if t.get("type", "function") == "function"] or None
        return _openai_messages(body.get("messages") or []), tools

    def _build_reply(self, parsed, raw_finish, translated, tools_schema) -> Reply:
        finish = "tool_calls" if parsed.tool_uses else ("length" if raw_finish == "length" else "stop")
        calls = [tool_call_dict(u["name"], u["arguments"], u["id"]) for u in parsed.tool_uses]
        stored = {"role": "assistant", "content": parsed.text}
        wire = {"role": "assistant", "content": parsed.text or None}
        if parsed.reasoning:
            stored["reasoning_content"] = wire["reasoning_content"] = parsed.reasoning
        if calls:
            stored["tool_calls"] = calls
            wire["tool_calls"] = [{**c, "function": {"name": c["function"]["name"],
                                                     "arguments": json.dumps(c["function"]["arguments"])}} for c in calls]  # fmt: skip
        return Reply(stored, wire, finish)

    async def _respond(self, request, body, reply, in_tok, out_tok, stream):
        usage = {"prompt_tokens": in_tok, "completion_tokens": out_tok, "total_tokens": in_tok + out_tok}
        base = {"id": f"chatcmpl-{uuid.uuid4().hex[:24]}", "created": int(time.time()), "model": body.get("model", "policy")}
        if not stream:
            return web.json_response({**base, "object": "chat.completion", "usage": usage,
                                      "choices": [{"index": 0, "message": reply.wire, "finish_reason": reply.finish}]})  # fmt: skip
        chunk = {**base, "object": "chat.completion.chunk"}
        delta = dict(reply.wire)
        if delta.get("tool_calls"):
            delta["tool_calls"] = [{**c, "index": i} for i, c in enumerate(delta["tool_calls"])]
        events = [(None, {**chunk, "choices": [{"index": 0, "delta": delta, "finish_reason": None}]}),
                  (None, {**chunk, "choices": [{"index": 0, "delta": {}, "finish_reason": reply.finish}], "usage": usage}),
                  (None, "[DONE]")]  # fmt: skip
        return await _sse(request, events)


# ---------------------------------------------------------------------------------- Anthropic
def _anthropic_messages(msgs: list[dict], system: Any) -> list[dict]:
    out = []
    sys_text = flatten_content(system)
    if sys_text:
        out.append({"role": "system", "content": sys_text})
    for m in msgs:
        content = m.get("content")
        if isinstance(content, str) or content is None:
            out.append({"role": m["role"], "content": content or ""})
            continue
        text, calls, results = [], [], []
        for b in content:
            t = b.get("type")
            if t == "text":
                text.append(b.get("text", ""))
            elif t == "tool_use":
                calls.append(tool_call_dict(b.get("name", ""), b.get("input") or {}, b.get("id")))
            elif t == "tool_result":
                results.append({"role": "tool", "tool_call_id": b.get("tool_use_id"), "content": flatten_content(b.get("content"))})
        if m["role"] == "assistant":
            msg = {"role": "assistant", "content": "\n".join(text)}
            if calls:
                msg["tool_calls"] = calls
            out.append(msg)
        else:
            out += results  # tool results come before any free text of the same user turn
            if text or not results:
                out.append({"role": "user", "content": "\n".join(text)})
    return out


class AnthropicAdapter(BaseAdapter):
    log_prefix = "anthropic"
    max_token_keys = ("max_tokens",)
    stop_keys = ("stop_sequences",)

    def _register_routes(self, app):
        app.router.add_post("/v1/messages", self._run_turn)
        app.router.add_post("/v1/messages/count_tokens", self._count_tokens)

    def _translate(self, body):
        tools = [{"type": "function", "function": {"name": t["name"], "description": t.get("description", ""),
                                                   "parameters": t.get("input_schema") or {"type": "object", "properties": {}}}}
                 for t in (body.get("tools") or []) if t.get("name")] or None  # fmt: skip
        return _anthropic_messages(body.get("messages") or [], body.get("system")), tools

    def _build_reply(self, parsed, raw_finish, translated, tools_schema) -> Reply:
        blocks = []
        if parsed.reasoning:
            blocks.append({"type": "thinking", "thinking": parsed.reasoning, "signature": ""})
        if parsed.text or not parsed.tool_uses:
            blocks.append({"type": "text", "text": parsed.text})
        for u in parsed.tool_uses:
            blocks.append({"type": "tool_use", "id": u["id"].replace("call_", "toolu_"), "name": u["name"], "input": u["arguments"]})
        stop = "tool_use" if parsed.tool_uses else ("max_tokens" if raw_finish == "length" else "end_turn")
        stored = {"role": "assistant", "content": parsed.text}
        if parsed.tool_uses:
            stored["tool_calls"] = [tool_call_dict(u["name"], u["arguments"], u["id"].replace("call_", "toolu_")) for u in parsed.tool_uses]
        return Reply(stored, blocks, stop)

    async def _respond(self, request, body, reply, in_tok, out_tok, stream):
        msg = {"id": f"msg_{uuid.uuid4().hex[:24]}", "type": "message", "role": "assistant", "model": body.get("model", "policy"),
               "content": reply.wire, "stop_reason": reply.finish, "stop_sequence": None,
               "usage": {"input_tokens": in_tok, "output_tokens": out_tok}}  # fmt: skip
        if not stream:
            return web.json_response(msg)
        ev = [("message_start", {"type": "message_start", "message": {**msg, "content": [], "stop_reason": None}})]
        for i, b in enumerate(reply.wire):
            if b["type"] == "text":
                start, delta = {"type": "text", "text": ""}, {"type": "text_delta", "text": b["text"]}
            elif b["type"] == "thinking":
                start, delta = {"type": "thinking", "thinking": ""}, {"type": "thinking_delta", "thinking": b["thinking"]}
            else:
                start = {"type": "tool_use", "id": b["id"], "name": b["name"], "input": {}}
                delta = {"type": "input_json_delta", "partial_json": json.dumps(b["input"])}
            ev += [("content_block_start", {"type": "content_block_start", "index": i, "content_block": start}),
                   ("content_block_delta", {"type": "content_block_delta", "index": i, "delta": delta}),
                   ("content_block_stop", {"type": "content_block_stop", "index": i})]  # fmt: skip
        ev += [("message_delta", {"type": "message_delta", "delta": {"stop_reason": reply.finish, "stop_sequence": None},
                                  "usage": {"output_tokens": out_tok}}),
               ("message_stop", {"type": "message_stop"})]  # fmt: skip
        return await _sse(request, ev)

    async def _count_tokens(self, request):
        body = await request.json()
        msgs, tools = self._translate(body)
        return web.json_response({"input_tokens": len(_render_token_ids(msgs, self.tokenizer, tools))})
