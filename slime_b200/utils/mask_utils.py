"""Loss masks for multi-turn conversations (SFT and multi-turn RL): 1 on assistant-generated tokens, 0 elsewhere.

``MultiTurnLossMaskGenerator(tokenizer, tokenizer_type).get_loss_mask(messages, tools)`` -> ``(token_ids, loss_mask)``.
A message with ``"step_loss_mask": 0`` is excluded from the loss whatever its role.

tokenizer_type:
  ``qwen``          each message is templated alone; the default system prompt the template injects in front of every
                    non-first message is measured once and cut off; the ``<|im_start|>assistant\\n`` header is not trained
  ``qwen3``         the template rewrites history (``<think>`` stripping), so a message is templated next to a fixed
                    dummy user turn whose tokens are then removed; consecutive tool messages are templated as one group
  ``qwen3_5``       the whole conversation is rendered once and assistant spans are located in the text; token masks come
                    from the tokenizer's offset mapping (needs a fast tokenizer); a leading ``<think>\\n`` is not trained
  ``distill_qwen``  prompt = first message + generation prompt, response = raw content of the last message
Parity: slime/utils/mask_utils.py:4-285.
"""

from __future__ import annotations

_PROBE = "FOR TESTING ONLY"
_DUMMY_TURN = {"role": "user", "content": "FOR CALCULATING LOSS MASK ONLY"}


def get_response_lengths(loss_masks: list[list[int]]) -> list[int]:
    """Tokens from the first trained token to the end (0 when nothing is trained)."""
    return [len(m) - m.index(1) if 1 in m else 0 for m in loss_masks]


def _find_all(haystack: list[int], needle: list[int]) -> list[int]:
    n = len(needle)
    return [i for i in range(len(haystack) - n + 1) if haystack[i : i + n] == needle]


class MultiTurnLossMaskGenerator:
    def __init__(self, tokenizer, tokenizer_type: str = "qwen"):
        self.tokenizer, self.tokenizer_type = tokenizer, tokenizer_type
        self.system_message_length = self.gen_token_length = 0
        if tokenizer_type in ("qwen", "qwen3"):
            self.system_message_length, self.gen_token_length = self.get_system_message_length()

    # ------------------------------------------------------------------ helpers
    def get_response_lengths(self, loss_masks):
        return get_response_lengths(loss_masks)

    def find_all_sublist_indices(self, main_list, sublist):
        return _find_all(main_list, sublist)

    def _template_ids(self, messages, **kw) -> list[int]:
        return list(self.tokenizer.apply_chat_template(messages, tokenize=True, return_dict=False, **kw))

    def get_system_message_length(self) -> tuple[int, int]:
        """Measure (tokens of the auto-injected system block, tokens of the generation header) with a probe: two equal
        user turns are templated; the spacing of the two probe occurrences gives the per-turn wrapper size and what
        precedes the first one beyond that wrapper is the injected system block."""
        tok = self.tokenizer
        probe_ids = tok(_PROBE, add_special_tokens=False)["input_ids"]
        turns = [{"role": "user", "content": _PROBE}] * 2
        text = tok.apply_chat_template(turns, add_special_tokens=False, tokenize=False)
        ids = tok(text, add_special_tokens=False)["input_ids"]
        first, second = _find_all(ids, probe_ids)
        tail = len(ids) - len(probe_ids) - second  # wrapper tokens after a turn's content
        head = (second - first) - tail - len(probe_ids)  # wrapper tokens before a turn's content
        with_gen = tok.apply_chat_template(turns, add_special_tokens=False, tokenize=True, add_generation_prompt=True,
                                           return_dict=False)  # fmt: skip
        return first - head, len(with_gen) - len(ids)

    def _mask_of(self, message: dict, ids: list[int]) -> list[int]:
        if message["role"] != "assistant" or message.get("step_loss_mask", 1) != 1:
            return [0] * len(ids)
        g = min(self.gen_token_length, len(ids))
        return [0] * g + [1] * (len(ids) - g)

    # --------------------------------------------------------------- per family
    def gen_multi_turn_loss_mask_qwen(self, messages, tools=None):
        ids_all, mask_all = [], []
        for i, msg in enumerate(messages):
            ids = self._template_ids([msg], tools=tools) if i == 0 else self._template_ids([msg])
            if i > 0 and msg["role"] != "system":
                ids = ids[self.system_message_length :]
            ids_all += ids
            mask_all += self._mask_of(msg, ids)
        return ids_all, mask_all

    def gen_multi_turn_loss_mask_qwen3(self, messages, tools=None):
        dummy_ids = self._template_ids([_DUMMY_TURN])
        ids_all, mask_all = [], []
        i = 0
        while i < len(messages):
            j = i + 1
            if messages[i]["role"] == "tool":  # a run of tool results shares one wrapper
                while j < len(messages) and messages[j]["role"] == "tool":
                    j += 1
            group = messages[i:j]
            if i == 0:
                ids = self._template_ids(group + [_DUMMY_TURN], tools=tools)[: -len(dummy_ids)]
            else:
                ids = self._template_ids([_DUMMY_TURN] + group)[len(dummy_ids) :]
                if messages[i]["role"] != "system":
                    ids = ids[self.system_message_length :]
            ids_all += ids
            mask_all += self._mask_of(messages[i], ids)
            i = j
        return ids_all, mask_all

    def gen_multi_turn_loss_mask_qwen3_5(self, messages, tools=None):
        tok = self.tokenizer
        text = tok.apply_chat_template(messages, tokenize=False, tools=tools, return_dict=False)
        enc = tok(text, add_special_tokens=False, return_offsets_mapping=True)
        ids, offsets = enc["input_ids"], enc.get("offset_mapping")
        if offsets is None:
            raise ValueError("qwen3_5 loss masks need a fast tokenizer (offset mapping)")
        if list(ids) != self._template_ids(messages, tools=tools):
            raise ValueError("tokenising the rendered chat text disagrees with apply_chat_template(tokenize=True)")
        header, think, end = "<|im_start|>assistant\n", "<think>\n", "<|im_end|>"
        trained = bytearray(len(text))  # per character
        cursor = 0
        for msg in messages:
            if msg["role"] != "assistant":
                continue
            at = text.find(header, cursor)
            if at < 0:
                raise ValueError("assistant turn not found in the rendered conversation")
            start = at + len(header)
            stop = text.find(end, start)
            if stop < 0:
                raise ValueError("assistant turn without <|im_end|> in the rendered conversation")
            stop += len(end)
            if stop < len(text) and text[stop] == "\n":
                stop += 1
            cursor = stop
            if msg.get("step_loss_mask", 1) != 1:
                continue
            if text.startswith(think, start):
                start += len(think)
            trained[start:stop] = b"\x01" * (stop - start)
        prefix = [0]
        for c in trained:
            prefix.append(prefix[-1] + c)
        mask = [1 if e > s and prefix[e] - prefix[s] > 0 else 0 for s, e in offsets]
        return list(ids), mask

    def gen_multi_turn_loss_mask_distill_qwen(self, messages, tools=None):
        tok = self.tokenizer
        prompt = tok.apply_chat_template(messages[:1], tokenize=False, add_generation_prompt=True, tools=tools)
        p_ids = tok(prompt, add_special_tokens=False)["input_ids"]
        r_ids = tok(messages[-1]["content"], add_special_tokens=False)["input_ids"]
        ids = list(p_ids) + list(r_ids)
        if messages[-1].get("step_loss_mask", 1) != 1:
            return ids, [0] * len(ids)
        return ids, [0] * len(p_ids) + [1] * len(r_ids)

    # ------------------------------------------------------------------- public
    def get_loss_mask(self, messages: list[dict], tools: list[dict] | None = None) -> tuple[list[int], list[int]]:
        kind = self.tokenizer_type
        if kind == "qwen":
            if "<｜Assistant｜>" in self.tokenizer.get_added_vocab():  # R1-distilled checkpoints keep the qwen type
                return self.gen_multi_turn_loss_mask_distill_qwen(messages, tools)
            return self.gen_multi_turn_loss_mask_qwen(messages, tools)
        if kind == "qwen3":
            return self.gen_multi_turn_loss_mask_qwen3(messages, tools)
        if kind == "qwen3_5":
            return self.gen_multi_turn_loss_mask_qwen3_5(messages, tools)
        if kind == "distill_qwen":
            return self.gen_multi_turn_loss_mask_distill_qwen(messages, tools)
        raise ValueError(f"unsupported tokenizer type {kind!r}")

    def get_loss_mask_with_multimodal_alignment(self, messages, input_ids, tools=None):
        """Multimodal prompts: the processor's ``input_ids`` contain extra image tokens in front; compute the mask on the
        text-only view and left-pad it with zeros to the processor's length."""
        flat = []
        for msg in messages:
            content = msg.get("content")
            if isinstance(content, list):
                parts = [c.get("text", "") if isinstance(c, dict) and c.get("type") == "text" else c
                         for c in content if isinstance(c, str) or (isinstance(c, dict) and c.get("type") == "text")]  # fmt: skip
                flat.append({"role": msg["role"], "content": " ".join(parts)})
            else:
                flat.append(msg)
        _, mask = self.get_loss_mask(flat, tools=tools)
        pad = len(input_ids) - len(mask)
        if pad < 0:
            raise ValueError(f"processor produced {len(input_ids)} tokens but the text alone needs {len(mask)}; "
                             "processor and tokenizer disagree")  # fmt: skip
        return input_ids, [0] * pad + mask

    def get_text_from_loss_mask(self, token_ids: list[int], loss_masks: list[int]) -> list[str]:
        """Decode each maximal run of trained tokens (debugging aid)."""
        out, run = [], []
        for t, m in zip(token_ids, loss_masks):
            if m == 1:
                run.append(t)
            elif run:
                out.append(self.tokenizer.decode(run))
                run = []
        if run:
            out.append(self.tokenizer.decode(run))
        return out
