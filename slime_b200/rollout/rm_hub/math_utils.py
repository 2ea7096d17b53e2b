"""Math answer extraction and equivalence (string normalisation first, sympy second).

Covers the graders the ``deepscaler`` / ``math`` reward types rely on (parity:
slime/rollout/rm_hub/math_utils.py:429-493): ``extract_boxed_answer``, ``grade_answer_mathd``
(MATH-dataset normalisation), ``grade_answer_sympy`` (symbolic difference == 0, tuples/intervals
element-wise), ``grade_answer_verl``.
"""

from __future__ import annotations

import re


def last_boxed_only_string(s: str) -> str | None:
    idx = s.rfind("\\boxed")
    if idx < 0:
        idx = s.rfind("\\fbox")
        if idx < 0:
            return None
    depth, i, start = 0, idx, None
    while i < len(s):
        if s[i] == "{":
            depth += 1
            if start is None:
                start = i
        elif s[i] == "}":
            depth -= 1
            if depth == 0 and start is not None:
                return s[idx : i + 1]
        i += 1
    return None


def remove_boxed(s: str) -> str | None:
    if not isinstance(s, str):
        return None
    for left in ("\\boxed{", "\\fbox{"):
        if s.startswith(left) and s.endswith("}"):
            return s[len(left) : -1]
    if s.startswith("\\boxed "):
        return s[len("\\boxed ") :]
    return None


def extract_boxed_answer(solution: str) -> str | None:
    b = last_boxed_only_string(solution or "")
    return remove_boxed(b) if b is not None else None


extract_answer = extract_boxed_answer

_UNITS = ["degree", "cm", "centimeter", "meter", "mile", "second", "minute", "hour", "day", "week", "month", "year",
          "foot", "feet", "inch", "yard", "unit", "point", "dollar", "cent"]  # fmt: skip


def _fix_fracs(s: str) -> str:
    # \frac12 -> \frac{1}{2}, \frac1{2} -> \frac{1}{2}
    s = re.sub(r"\\frac(\d)(\d)", r"\\frac{\1}{\2}", s)
    s = re.sub(r"\\frac(\d)\{", r"\\frac{\1}{", s)
    s = re.sub(r"\\frac\{([^{}]+)\}(\d)", r"\\frac{\1}{\2}", s)
    return s


def _fix_sqrt(s: str) -> str:
    return re.sub(r"\\sqrt(\w)", r"\\sqrt{\1}", s)


def _fix_a_slash_b(s: str) -> str:
    m = re.fullmatch(r"(-?\d+)/(\d+)", s)
    return f"\\frac{{{m.group(1)}}}{{{m.group(2)}}}" if m else s


def mathd_normalize_answer(answer: str | None) -> str | None:
    if answer is None:
        return None
    s = answer.strip()
    m = re.search(r"^\\text\{(?P<t>.+?)\}$", s)
    if m:
        s = m.group("t").strip()
    s = s.replace("\n", "").replace("\\!", "").replace("\\\\", "\\").replace("tfrac", "frac").replace("dfrac", "frac")
    s = s.replace("\\left", "").replace("\\right", "").replace("^{\\circ}", "").replace("^\\circ", "")
    s = s.replace("\\$", "").replace("$", "")
    s = re.sub(r"\\text\{\s*([^{}]*)\}", r"\1", s)
    for u in _UNITS:
        s = re.sub(rf"\s*{u}(es|s)?\b(\^\d+)?", "", s)
    s = s.replace("\\%", "").replace("%", "")
    s = s.replace(" .", " 0.").replace("{.", "{0.")
    if s.startswith("."):
        s = "0" + s
    if len(s.split("=")) == 2 and len(s.split("=")[0]) <= 2:
        s = s.split("=")[1]
    s = _fix_sqrt(s).replace(" ", "")
    s = _fix_fracs(s)
    if s == "0.5":
        s = "\\frac{1}{2}"
    return _fix_a_slash_b(s)


def grade_answer_mathd(given: str, truth: str) -> bool:
    return mathd_normalize_answer(given) == mathd_normalize_answer(truth)


def _strip_for_sympy(s: str) -> str:
    s = s.replace("\\left", "").replace("\\right", "").replace("\\!", "").replace("\\,", "").replace("\\ ", "")
    s = s.replace("\\dfrac", "\\frac").replace("\\tfrac", "\\frac").replace("\\cdot", "*").replace("\\times", "*")
    s = s.replace("\\pi", "pi").replace("^", "**").replace("\\%", "").replace("%", "").replace("$", "")
    s = re.sub(r"\\text\{[^{}]*\}", "", s)
    for _ in range(4):
        s = re.sub(r"\\frac\{([^{}]+)\}\{([^{}]+)\}", r"((\1)/(\2))", s)
        s = re.sub(r"\\sqrt\{([^{}]+)\}", r"sqrt(\1)", s)
    s = s.replace("{", "(").replace("}", ")")
    s = re.sub(r"(\d),(\d{3})\b", r"\1\2", s)
    s = re.sub(r"(\d)\s*([a-zA-Z(])", r"\1*\2", s)
    return s.strip()


def _sympy_equal(a: str, b: str) -> bool:
    try:
        import sympy
        from sympy.parsing.sympy_parser import parse_expr

        ea, eb = parse_expr(_strip_for_sympy(a)), parse_expr(_strip_for_sympy(b))
        return sympy.simplify(ea - eb) == 0
    except Exception:
        return False


def _split_tuple(s: str) -> list[str]:
    s = s.strip()
    if len(s) > 2 and s[0] in "([" and s[-1] in ")]" and "," in s:
        return [x.strip() for x in s[1:-1].split(",")]
    return [s]


def _plain_fraction(s: str) -> str | None:
    """``a/b`` for an answer that is nothing but a fraction of integer literals (``\frac{a}{b}`` or ``a/b``)."""
    s = re.sub(r"^\\[dt]?frac\{(-?\d+)\}\{(\d+)\}$", r"\1/\2", s.replace(" ", ""))
    return s if re.fullmatch(r"-?\d+/0*[1-9]\d*", s) else None


def _is_integer_literal(s: str) -> bool:
    try:
        x = float(re.sub(r"(\d),(\d{3})\b", r"\1\2", s.strip()))
        return abs(x - round(x)) <= 1e-7
    except ValueError:
        return False


def grade_answer_sympy(given: str, truth: str) -> bool:
    if given is None or truth is None:
        return False
    g, t = _split_tuple(given), _split_tuple(truth)
    if len(g) != len(t):
        return False
    if len(g) > 1 and (given.strip()[0] != truth.strip()[0] or given.strip()[-1] != truth.strip()[-1]):
        return False
    for x, y in zip(g, t):
        if x == y:
            continue
        if re.search(r"[a-zA-Z]{3,}", x) and not re.search(r"(sqrt|pi|frac)", x):
            return False  # free text never equals a different free text
        fx, fy = _plain_fraction(x), _plain_fraction(y)
        if fx is not None and fy is not None:
            if fx != fy:
                return False  # an unreduced fraction is not the reduced one: no simplification between two plain fractions
            continue
        if _is_integer_literal(x) != _is_integer_literal(y):
            return False  # an integer answer must be given as that integer, not as an expression that evaluates to it
        if not _sympy_equal(x, y):
            return False
    return True


def grade_answer_verl(solution_str: str, ground_truth: str) -> bool:
    if not ground_truth:
        return False
    truth = extract_boxed_answer(ground_truth) if "\\boxed" in ground_truth else ground_truth
    given = extract_boxed_answer(solution_str)
    if given is None or truth is None:
        return False
    return grade_answer_mathd(given, truth) or grade_answer_sympy(given, truth)
