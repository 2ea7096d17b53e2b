"""SQuAD-style token F1 (parity: slime/rollout/rm_hub/f1.py:6-47). Returns (f1, precision, recall)."""

import re
import string
from collections import Counter


def normalize_answer(s: str) -> str:
    s = s.lower()
    s = "".join(ch for ch in s if ch not in set(string.punctuation))
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return " ".join(s.split())


def f1_score(prediction: str, ground_truth) -> tuple[float, float, float]:
    zero = (0.0, 0.0, 0.0)
    if ground_truth is None or prediction is None:
        return zero
    if isinstance(ground_truth, (list, tuple)):
        return max((f1_score(prediction, g) for g in ground_truth), key=lambda x: x[0], default=zero)
    pred, gt = normalize_answer(prediction), normalize_answer(str(ground_truth))
    if pred in ("yes", "no", "noanswer") and pred != gt:
        return zero
    if gt in ("yes", "no", "noanswer") and pred != gt:
        return zero
    p_tok, g_tok = pred.split(), gt.split()
    same = sum((Counter(p_tok) & Counter(g_tok)).values())
    if same == 0:
        return zero
    prec, rec = same / len(p_tok), same / len(g_tok)
    return 2 * prec * rec / (prec + rec), prec, rec
