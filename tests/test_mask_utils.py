"""Multi-turn loss masks against a small ChatML tokenizer whose behaviour is fully known."""

import re

import pytest

from slime_b200.utils.mask_utils import MultiTurnLossMaskGenerator, get_response_lengths

DEFAULT_SYSTEM = "You are a helpful assistant."


class ChatMLTokenizer:
    """Word-level tokenizer with a Qwen-style template: a default system block is injected when the conversation
    does not start with a system message; special markers are single tokens."""

    def __init__(self, inject_system=True):
        self.vocab: dict[str, int] = {}
        self.inject_system = inject_system  # Qwen2.5 injects a default system block, Qwen3 does not

    def _ids(self, text: str) -> list[int]:
        pieces = re.findall(r"<\|im_start\|>|<\|im_end\|>|\n|[^\s<]+|<", text)
        return [self.vocab.setdefault(p, len(self.vocab)) for p in pieces]

    def __call__(self, text, add_special_tokens=False, return_offsets_mapping=False):
        return {"input_ids": self._ids(text)}

    def get_added_vocab(self):
        return {"<|im_start|>": 0, "<|im_end|>": 1}

    def decode(self, ids):
        inv = {v: k for k, v in self.vocab.items()}
        return " ".join(inv[i] for i in ids)

    def apply_chat_template(self, messages, tokenize=True, add_generation_prompt=False, tools=None, return_dict=False,
                            add_special_tokens=False):  # fmt: skip
        text = ""
        if self.inject_system and messages and messages[0]["role"] != "system":
            text += f"<|im_start|>system\n{DEFAULT_SYSTEM}<|im_end|>\n"
        for m in messages:
            text += f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n"
        if add_generation_prompt:
            text += "<|im_start|>assistant\n"
        return self._ids(text) if tokenize else text


CONV = [
    {"role": "system", "content": "be brief"},
    {"role": "user", "content": "what is two plus two"},
    {"role": "assistant", "content": "four"},
    {"role": "user", "content": "and three plus three"},
    {"role": "assistant", "content": "six of course"},
]


def _trained_text(gen, messages):
    ids, mask = gen.get_loss_mask(messages)
    assert len(ids) == len(mask)
    return gen.get_text_from_loss_mask(ids, mask), ids, mask


@pytest.mark.parametrize("kind", ["qwen", "qwen3"])
def test_only_assistant_content_is_trained(kind):
    tok = ChatMLTokenizer(inject_system=kind == "qwen")
    gen = MultiTurnLossMaskGenerator(tok, kind)
    # injected system block: <|im_start|> system \n You are a helpful assistant. <|im_end|> \n = 3 + 5 + 2 tokens
    assert gen.system_message_length == (10 if kind == "qwen" else 0) and gen.gen_token_length == 3
    spans, ids, mask = _trained_text(gen, CONV)
    assert spans == ["four <|im_end|> \n", "six of course <|im_end|> \n"]
    # the concatenation of per-message pieces equals templating the whole conversation at once
    assert ids == tok.apply_chat_template(CONV, tokenize=True)
    assert get_response_lengths([mask]) == [len(mask) - mask.index(1)]


def test_step_loss_mask_zero_excludes_a_turn():
    gen = MultiTurnLossMaskGenerator(ChatMLTokenizer(), "qwen")
    conv = [dict(m) for m in CONV]
    conv[2]["step_loss_mask"] = 0
    spans, _, _ = _trained_text(gen, conv)
    assert spans == ["six of course <|im_end|> \n"]


def test_qwen3_groups_consecutive_tool_messages():
    tok = ChatMLTokenizer(inject_system=False)
    gen = MultiTurnLossMaskGenerator(tok, "qwen3")
    conv = [{"role": "user", "content": "weather in two cities"}, {"role": "assistant", "content": "calling tools"},
            {"role": "tool", "content": "sunny"}, {"role": "tool", "content": "rainy"},
            {"role": "assistant", "content": "sunny and rainy"}]  # fmt: skip
    spans, ids, _ = _trained_text(gen, conv)
    assert spans == ["calling tools <|im_end|> \n", "sunny and rainy <|im_end|> \n"]
    assert ids == tok.apply_chat_template(conv, tokenize=True)


def test_distill_qwen_trains_the_raw_last_message():
    tok = ChatMLTokenizer()
    gen = MultiTurnLossMaskGenerator(tok, "distill_qwen")
    conv = [{"role": "user", "content": "say hi"}, {"role": "assistant", "content": "hi there"}]
    ids, mask = gen.get_loss_mask(conv)
    assert gen.get_text_from_loss_mask(ids, mask) == ["hi there"]
    assert sum(mask) == 2 and mask[-2:] == [1, 1]


def test_multimodal_alignment_left_pads():
    gen = MultiTurnLossMaskGenerator(ChatMLTokenizer(), "qwen")
    conv = [{"role": "user", "content": [{"type": "image"}, {"type": "text", "text": "what is this"}]},
            {"role": "assistant", "content": "a cat"}]  # fmt: skip
    _, text_mask = gen.get_loss_mask([{"role": "user", "content": "what is this"}, conv[1]])
    ids = list(range(len(text_mask) + 7))  # the processor added 7 image tokens
    out_ids, mask = gen.get_loss_mask_with_multimodal_alignment(conv, ids)
    assert out_ids is ids and mask == [0] * 7 + text_mask
    with pytest.raises(ValueError):
        gen.get_loss_mask_with_multimodal_alignment(conv, ids[:3])


def test_unknown_type_is_rejected():
    with pytest.raises(ValueError):
        MultiTurnLossMaskGenerator(ChatMLTokenizer(), "llama").get_loss_mask(CONV)
