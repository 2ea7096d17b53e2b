"""Multiple-choice (GPQA-style) reward: strip the chain of thought, extract the chosen letter and
compare with the label (letter, index or answer text). Parity: slime/rollout/rm_hub/gpqa.py:54-129."""

from __future__ import annotations

import re
import string

DEFAULT_LETTERS = list(string.ascii_uppercase[:8])
_PATTERNS = [
    r"(?i)(?:final\s+)?answer\s*(?:is|:)?\s*\(?\s*([A-H])\s*\)?(?![a-z])",
    r"(?i)(?:option|choice)\s*\(?\s*([A-H])\s*\)?(?![a-z])",
    r"\\boxed\{\s*\(?([A-H])\)?\s*\}",
    r"^\s*\(?([A-H])\)?\s*[.:)]?\s*$",
]


def _strip_cot(text: str) -> str:
    for marker in ("</think>", "###Response"):
        if marker in text:
            text = text.split(marker)[-1]
    return text.strip()


def extract_letter(response: str, letters=DEFAULT_LETTERS) -> str | None:
    text = _strip_cot(response or "")
    for pat in _PATTERNS:
        hits = re.findall(pat, text, flags=re.MULTILINE)
        hits = [h.upper() for h in hits if h.upper() in letters]
        if hits:
            return hits[-1]
    tail = re.findall(r"\b([A-H])\b", text[-64:])
    tail = [t for t in tail if t in letters]
    return tail[-1] if tail else None


# the reference's names for the same things (plug-ins import them)
DEFAULT_VALID_LETTERS = DEFAULT_LETTERS
_extract_letter_from_response = extract_letter


def compute_gpqa_reward(response: str, label, metadata: dict | None = None) -> float:
    md = metadata or {}
    choices = md.get("choices")
    letters = md.get("valid_letters") or (DEFAULT_LETTERS[: len(choices)] if choices else DEFAULT_LETTERS)
    correct = md.get("correct_letter")
    if isinstance(correct, str):
        correct = correct.strip().upper() or None
    if correct is None and label is not None:
        if isinstance(label, int):
            correct = letters[label] if 0 <= label < len(letters) else None
        elif isinstance(label, str) and label.strip().upper() in letters and len(label.strip()) == 1:
            correct = label.strip().upper()
        elif isinstance(label, str) and choices:
            norm = [str(c).strip().lower() for c in choices]
            if label.strip().lower() in norm:
                correct = letters[norm.index(label.strip().lower())]
    if correct is None:
        return 0.0
    picked = extract_letter(response, letters)
    if picked is None and choices:  # answered with the option text
        text = _strip_cot(response or "").lower()
        hits = [letters[i] for i, c in enumerate(choices) if str(c).strip().lower() in text]
        picked = hits[-1] if len(hits) == 1 else None
    return 1.0 if picked == correct else 0.0
