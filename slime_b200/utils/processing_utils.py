"""Tokenizer / processor loading and chat / vision helpers.

Parity: slime/utils/processing_utils.py:18-162. A ``DummyTokenizer`` (ids <-> space-separated
integers) lets the whole pipeline run without a model directory (synthetic workloads, tests)."""

from __future__ import annotations

import base64
import io
import logging
import os

logger = logging.getLogger(__name__)


class DummyTokenizer:
    """Text is a space-separated list of integer ids; no special tokens."""

    eos_token_id = None
    pad_token_id = 0
    chat_template = None

    def __init__(self, vocab_size: int = 1 << 20):
        self.vocab_size = vocab_size

    def encode(self, text, add_special_tokens=False):
        return [int(t) % self.vocab_size for t in str(text).split() if t.lstrip("-").isdigit()]

    def __call__(self, text, add_special_tokens=False, **kw):
        if isinstance(text, (list, tuple)):
            return {"input_ids": [self.encode(t) for t in text]}
        return {"input_ids": self.encode(text)}

    def decode(self, ids, skip_special_tokens=True, **kw):
        return " ".join(str(int(i)) for i in ids)

    def apply_chat_template(self, messages, tools=None, tokenize=False, add_generation_prompt=True, **kw):
        text = " ".join(str(m.get("content", "")) if isinstance(m, dict) else str(m) for m in messages)
        return self.encode(text) if tokenize else text


def load_tokenizer(name_or_path: str | None, **kwargs):
    if not name_or_path or not os.path.exists(name_or_path):
        logger.info("no tokenizer directory (%s): using the integer DummyTokenizer", name_or_path)
        return DummyTokenizer()
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(name_or_path, **kwargs)


def load_processor(name_or_path: str | None, **kwargs):
    """A multimodal processor if the checkpoint ships one, else None."""
    if not name_or_path or not os.path.exists(os.path.join(name_or_path, "preprocessor_config.json")):
        return None
    try:
        from transformers import AutoProcessor, PreTrainedTokenizerBase

        proc = AutoProcessor.from_pretrained(name_or_path, **kwargs)
        return None if isinstance(proc, PreTrainedTokenizerBase) else proc
    except Exception as e:  # noqa: BLE001
        logger.warning("failed to load processor from %s: %r", name_or_path, e)
        return None


def process_vision_info(prompt, processor) -> dict:
    """Collect images / videos referenced by a message list into processor kwargs."""
    images, videos = [], []
    if isinstance(prompt, list):
        for msg in prompt:
            content = msg.get("content") if isinstance(msg, dict) else None
            if isinstance(content, list):
                for part in content:
                    if part.get("type") == "image" and part.get("image") is not None:
                        images.append(_load_image(part["image"]))
                    elif part.get("type") == "video" and part.get("video") is not None:
                        videos.append(part["video"])
    out = {}
    if images:
        out["images"] = images
    if videos:
        out["videos"] = videos
    return out


def _load_image(src):
    try:
        from PIL import Image
    except ImportError:
        return src
    if isinstance(src, (bytes, bytearray)):
        return Image.open(io.BytesIO(src))
    if isinstance(src, str) and src.startswith("data:"):
        return Image.open(io.BytesIO(base64.b64decode(src.split(",", 1)[1])))
    if isinstance(src, str) and os.path.exists(src):
        return Image.open(src)
    return src


def encode_image_for_rollout_engine(image) -> str:
    """PIL image (or bytes / path) -> ``data:image/png;base64,...`` for the ``image_data`` request field."""
    if isinstance(image, str):
        return image
    buf = io.BytesIO()
    if hasattr(image, "save"):
        image.save(buf, format="PNG")
        raw = buf.getvalue()
    else:
        raw = bytes(image)
    return "data:image/png;base64," + base64.b64encode(raw).decode()
