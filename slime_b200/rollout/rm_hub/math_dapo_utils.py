"""DAPO math reward (parity: slime/rollout/rm_hub/math_dapo_utils.py:262-292): look at the last 300
characters, take the final ``Answer: ...`` line (or the last boxed expression in strict mode), apply
Minerva-style normalisation and compare. Returns ``{"score": +-1.0, "acc": bool, "pred": str}`` so
recipes use ``--reward-key score``."""

from __future__ import annotations

import re

from slime_b200.rollout.rm_hub.math_utils import last_boxed_only_string
from slime_b200.rollout.rm_hub.math_utils import remove_boxed as _remove_boxed_or_none


def remove_boxed(s: str) -> str:
    """Content of ``\\boxed{...}``; unlike the lenient version of ``math_utils`` a string that is not a box is an error."""
    out = _remove_boxed_or_none(s)
    assert out is not None, f"box error: {s}"
    return out


_SUBS = [("an ", ""), ("a ", ""), (".$", "$"), ("\\$", ""), (r"\ ", ""), (" ", ""), ("mbox", "text"),
         (",\\text{and}", ","), ("\\text{and}", ","), ("\\text{m}", "\\text{}")]  # fmt: skip
_REMOVED = ["square", "ways", "integers", "dollars", "mph", "inches", "hours", "km", "units", "\\ldots", "sue", "points",
            "feet", "minutes", "digits", "cents", "degrees", "cm", "gm", "pounds", "meters", "meals", "edges", "students",
            "childrentickets", "multiples", "\\text{s}", "\\text{.}", "\\text{\ns}", "\\text{}^2", "\\text{}^3", "\\text{\n}",
            "\\text{}", r"\mathrm{th}", r"^\circ", r"^{\circ}", r"\;", r",\!", "{,}", '"', "\\dots", "<|im_end|>", "<|endoftext|>"]  # fmt: skip


def normalize_final_answer(final_answer: str) -> str:
    s = final_answer.split("=")[-1]
    for a, b in _SUBS:
        s = s.replace(a, b)
    for r in _REMOVED:
        s = s.replace(r, "")
    s = re.sub(r"(.*?)(\$)(.*?)(\$)(.*)", "$\\3$", s)
    s = re.sub(r"(\\text\{)(.*?)(\})", "\\2", s)
    s = re.sub(r"(\\textbf\{)(.*?)(\})", "\\2", s)
    s = re.sub(r"(\\overline\{)(.*?)(\})", "\\2", s)
    s = re.sub(r"(\\boxed\{)(.*)(\})", "\\2", s)
    s = re.sub(r"(frac)([^{])(.)", "frac{\\2}{\\3}", s)
    s = re.sub(r"(sqrt)([^{])", "sqrt{\\2}", s)
    s = s.replace("$", "")
    if s.replace(",", "").isdigit():
        s = s.replace(",", "")
    return s.strip()


def is_correct_minerva(solution_str: str, gt: str, gt_need_extract: bool = False,
                       answer_pattern: str = r"(?i)Answer\s*:\s*([^\n]+)") -> tuple[bool, str]:
    m = re.findall(answer_pattern, solution_str)
    pred = normalize_final_answer(m[-1]) if m else "[INVALID]"
    if gt_need_extract:
        gt = normalize_final_answer(_remove_boxed_or_none(last_boxed_only_string(gt)) or "")
    else:
        gt = normalize_final_answer(gt)
    return pred == gt, pred


def is_correct_strict_box(pred: str, gt: str, pause_tokens_index=None) -> tuple[int, str | None]:
    pred = pred[-100:]
    boxed = last_boxed_only_string(pred)
    ans = remove_boxed(boxed) if boxed is not None else None
    return (1 if ans == gt else -1), ans


def verify(solution_str: str, answer: str, strict_box_verify: bool = False, pause_tokens_index=None):
    if strict_box_verify:
        c, pred = is_correct_strict_box(solution_str, answer, pause_tokens_index)
        return c == 1, pred
    return is_correct_minerva(solution_str, answer)


def compute_score(solution_str: str, ground_truth: str, strict_box_verify: bool = False, pause_tokens_index=None) -> dict:
    solution_str = solution_str[-300:]
    correct, pred = verify(solution_str, str(ground_truth), strict_box_verify, pause_tokens_index)
    return {"score": 1.0 if correct else -1.0, "acc": bool(correct), "pred": pred}
