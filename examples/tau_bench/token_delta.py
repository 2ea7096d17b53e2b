"""Tokens that the last message of a conversation adds to the training sequence, found on rendered text.

A chat template is not append-only: many templates drop the reasoning of earlier assistant turns once a new user turn
follows, so "render everything, subtract what was there before" cuts into the new message. The rules here:

* assistant message: the rendering of the history with a generation prompt must be a prefix of the rendering with the
  message (an assistant turn never rewrites history); the delta is what follows it, all trained on. With
  ``include_generation_prompt`` the prompt itself is part of the delta and masked out, and prompt and answer are tokenised
  together so that a token may span their boundary.
* any other message: the delta is what follows the rendering of the history; if the template rewrote the history, a user
  message rendered on its own must close the new rendering and is the delta. Never trained on.

``get_context_delta`` is the variant a rollout needs after an environment / user message: that message plus the
generation prompt of the assistant turn that follows, as context tokens.
Same contract as examples/tau-bench/token_delta.py in the reference (checked with its history-rewriting and
boundary-merging tokenizers in the tests).
"""

from __future__ import annotations


def _render(tokenizer, messages, generation_prompt: bool) -> str:
    return tokenizer.apply_chat_template(messages, add_generation_prompt=generation_prompt, tokenize=False)


def _ids(tokenizer, text: str) -> list[int]:
    return list(tokenizer.encode(text, add_special_tokens=False))


def _non_assistant_text(tokenizer, messages) -> str:
    now, before = _render(tokenizer, messages, False), _render(tokenizer, messages[:-1], False)
    if now.startswith(before):
        return now[len(before) :]
    if messages[-1]["role"] != "user":
        raise ValueError("the chat template rewrote the history while a non-user message was added")
    alone = _render(tokenizer, [messages[-1]], False)
    if not now.endswith(alone):
        raise ValueError("the new user message is not a standalone suffix of the rendered conversation")
    return alone


def get_token_delta(tokenizer, messages: list[dict], *, include_generation_prompt: bool = False) -> tuple[list[int], list[int]]:
    """``(token ids, loss mask)`` contributed by ``messages[-1]``."""
    if not messages:
        raise ValueError("an empty conversation has no last message")
    if messages[-1]["role"] != "assistant":
        ids = _ids(tokenizer, _non_assistant_text(tokenizer, messages))
        return ids, [0] * len(ids)
    before, prompted, now = (_render(tokenizer, messages[:-1], False), _render(tokenizer, messages[:-1], True), _render(tokenizer, messages, False))
    if not prompted.startswith(before):
        raise ValueError("adding the generation prompt rewrote the rendered conversation")
    if not now.startswith(prompted):
        raise ValueError("the assistant message does not extend its generation prompt")
    if not include_generation_prompt:
        ids = _ids(tokenizer, now[len(prompted) :])
        return ids, [1] * len(ids)
    ids = _ids(tokenizer, now[len(before) :])
    masked = min(len(_ids(tokenizer, prompted[len(before) :])), len(ids))
    return ids, [0] * masked + [1] * (len(ids) - masked)


def get_context_delta(tokenizer, messages: list[dict]) -> list[int]:
    """Token ids of ``messages[-1]`` (a user / tool message) followed by the next assistant turn's generation prompt."""
    text = _non_assistant_text(tokenizer, messages)
    prompted, plain = _render(tokenizer, messages, True), _render(tokenizer, messages, False)
    if not prompted.startswith(plain):
        raise ValueError("adding the generation prompt rewrote the rendered conversation")
    return _ids(tokenizer, text + prompted[len(plain) :])
