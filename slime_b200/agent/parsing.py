"""Split raw model text into reasoning, visible text and tool calls.

Supported conventions (the ones Qwen / Hermes style chat templates emit):
  reasoning   ``<think> ... </think>`` at the start of the output (an unterminated block means the model ran out of
              tokens while thinking: everything is reasoning, nothing is visible)
  tool calls  ``<tool_call>{"name": ..., "arguments": {...}}</tool_call>`` JSON blocks, or the XML form
              ``<tool_call><function=NAME><parameter=KEY>VALUE</parameter>...</function></tool_call>``
A block that cannot be parsed, or that names a tool absent from the schema, marks the output ``ill_formed``; the text of
the block stays in the visible text so nothing the model said is lost. Parity: slime/agent/parsing.py:16-114.
"""

from __future__ import annotations

import dataclasses
import json
import re
import uuid
from typing import Any

_THINK = re.compile(r"^\s*<think>(.*?)</think>\s*", re.S)
_CALL = re.compile(r"<tool_call>\s*(.*?)\s*</tool_call>", re.S)
_XML_FN = re.compile(r"<function=([^>\s]+)>\s*(.*?)\s*</function>", re.S)
_XML_PARAM = re.compile(r"<parameter=([^>\s]+)>\s*(.*?)\s*</parameter>", re.S)


@dataclasses.dataclass
class ParsedModelOutput:
    text: str = ""
    reasoning: str = ""
    tool_uses: list[dict[str, Any]] = dataclasses.field(default_factory=list)
    ill_formed: bool = False


def _known_tools(tools_schema) -> set[str] | None:
    if not tools_schema:
        return None
    names = set()
    for t in tools_schema:
        fn = t.get("function", t)
        if fn.get("name"):
            names.add(fn["name"])
    return names


def _coerce(value: str):
    try:
        return json.loads(value)
    except (ValueError, TypeError):
        return value


def parse_tool_uses(body: str, tools_schema=None) -> tuple[str, list[dict], bool]:
    """(text without well-formed call blocks, calls ``{"id", "name", "arguments": dict}``, ill_formed)."""
    known = _known_tools(tools_schema)
    calls, bad = [], False

    def take(m):
        nonlocal bad
        inner = m.group(1)
        name = args = None
        try:
            obj = json.loads(inner)
            name, args = obj.get("name"), obj.get("arguments", obj.get("parameters", {}))
            if isinstance(args, str):
                args = json.loads(args)
        except (ValueError, AttributeError):
            fn = _XML_FN.search(inner)
            if fn:
                name = fn.group(1)
                args = {k: _coerce(v) for k, v in _XML_PARAM.findall(fn.group(2))}
        if not name or not isinstance(args, dict) or (known is not None and name not in known):
            bad = True
            return m.group(0)
        calls.append({"id": f"call_{uuid.uuid4().hex[:24]}", "name": name, "arguments": args})
        return ""

    text = _CALL.sub(take, body)
    if "<tool_call>" in text and not bad:  # an opening tag whose block never closed
        bad = True
    return text.strip(), calls, bad


def parse_model_output(raw: str, tools_schema=None, tool_parser_name: str | None = None,
                       reasoning_parser_name: str | None = None) -> ParsedModelOutput:  # fmt: skip
    out = ParsedModelOutput()
    body = raw
    for tail in ("<|im_end|>", "<|endoftext|>", "</s>"):
        if body.endswith(tail):
            body = body[: -len(tail)]
    if reasoning_parser_name != "none":
        m = _THINK.match(body)
        if m:
            out.reasoning, body = m.group(1).strip(), body[m.end() :]
        elif body.lstrip().startswith("<think>"):
            out.reasoning, body = body.lstrip()[len("<think>") :].strip(), ""
        elif "</think>" in body:  # templates that open the think block in the prompt
            head, _, body = body.partition("</think>")
            out.reasoning = head.strip()
    if tool_parser_name != "none":
        out.text, out.tool_uses, out.ill_formed = parse_tool_uses(body, tools_schema)
    else:
        out.text = body.strip()
    return out
