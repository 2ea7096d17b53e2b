"""DeepScaleR rule-based reward (parity: slime/rollout/rm_hub/deepscaler.py:4-41): the answer must
come after the reasoning block (``</think>`` or ``###Response``), be ``\\boxed{}``, and match the label
by string normalisation or sympy equivalence. Returns 1 or 0."""

from slime_b200.rollout.rm_hub.math_utils import extract_boxed_answer, grade_answer_mathd, grade_answer_sympy


def get_deepscaler_rule_based_reward(response: str, label) -> int:
    if "</think>" in response:
        solution = response.split("</think>")[-1]
    elif "###Response" in response:
        solution = response.split("###Response")[1]
    else:
        return 0
    answer = extract_boxed_answer(solution)
    if answer is None or label is None or label == "":
        return 0
    labels = label if isinstance(label, (list, tuple)) else [label]
    truths = []
    for t in labels:
        t = str(t)
        if "\\boxed" in t:
            t = extract_boxed_answer(t)
        if t is not None and t.strip():
            truths.append(t.strip())
    if not truths:
        return 0
    return int(any(grade_answer_mathd(answer, t) or grade_answer_sympy(answer, t) for t in truths))
