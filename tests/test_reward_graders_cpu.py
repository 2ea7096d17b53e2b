"""Rule-based reward graders on fixed cases: a wrong brace count or one bad substitution silently turns rewards 1 -> 0.
The expected values are those of the reference's grader tests (tests/test_rm_math.py, test_rm_math_dapo.py,
test_rm_deepscaler.py, test_rm_f1.py, test_rm_gpqa.py), restated as tables."""

import pytest

from slime_b200.rollout.rm_hub import gpqa, math_dapo_utils as dapo, math_utils as mu
from slime_b200.rollout.rm_hub.deepscaler import get_deepscaler_rule_based_reward as deepscaler
from slime_b200.rollout.rm_hub.f1 import f1_score, normalize_answer


@pytest.mark.parametrize("text,want", [
    (r"first attempt \boxed{wrong}, final \boxed{42}", r"\boxed{42}"),  # the last box wins
    (r"answer: \boxed{\frac{1}{2}}", r"\boxed{\frac{1}{2}}"),  # nested braces are balanced
    (r"answer: \fbox{7}", r"\fbox{7}"),
    ("plain text, no box", None),
    (r"start \boxed{never closes", None),
])  # fmt: skip
def test_last_boxed_expression(text, want):
    assert mu.last_boxed_only_string(text) == want == dapo.last_boxed_only_string(text)


def test_box_removal_lenient_and_strict():
    assert mu.remove_boxed(r"\boxed{x+1}") == "x+1" and mu.remove_boxed(r"\boxed{\frac{1}{2}}") == r"\frac{1}{2}"
    assert mu.remove_boxed("not boxed at all") is None and mu.remove_boxed(None) is None
    assert mu.extract_boxed_answer(r"Solution: \boxed{42}") == "42" and mu.extract_answer("just 42") is None
    assert dapo.remove_boxed(r"\boxed{42}") == "42"
    with pytest.raises(AssertionError, match="box error"):
        dapo.remove_boxed("not boxed")


@pytest.mark.parametrize("raw,want", [
    (r"\frac12", r"\frac{1}{2}"), (r"\tfrac{1}{2}", r"\frac{1}{2}"), (r"\left(1\right)", "(1)"), (r"45^{\circ}", "45"),
    (r"45^\circ", "45"), (".7", "0.7"), ("0.5", r"\frac{1}{2}"), (".5", r"\frac{1}{2}"), ("3/4", r"\frac{3}{4}"), ("1 + 1", "1+1"),
    (r"\text{42}", "42"), (None, None),
])  # fmt: skip
def test_hendrycks_normalisation(raw, want):
    assert mu.mathd_normalize_answer(raw) == want


def test_math_grading_paths():
    for given, truth in [(r"\frac{1}{2}", "0.5"), (r"\frac12", r"\frac{1}{2}"), (r"45^\circ", "45"), ("3/4", r"\frac{3}{4}")]:
        assert mu.grade_answer_mathd(given, truth)
    assert not mu.grade_answer_mathd("42", "43")
    assert mu.grade_answer_sympy("x+1", "1+x") and mu.grade_answer_sympy("2x+2", "2(x+1)")
    assert not mu.grade_answer_sympy(r"\frac{2}{4}", r"\frac{1}{2}")  # an unreduced fraction is not the reduced one
    assert not mu.grade_answer_sympy("4/2", "2")  # an integer answer must be given as that integer
    assert mu.grade_answer_sympy("1/2", "0.5") and mu.grade_answer_sympy("2.0", "2")
    assert mu.grade_answer_verl(r"answer: \boxed{42}", r"\boxed{42}")
    assert not mu.grade_answer_verl("just 42", "42") and not mu.grade_answer_verl(r"\boxed{42}", "")


@pytest.mark.parametrize("raw,want", [
    ("x = 42", "42"), ("an answer", "answer"), ("42 square", "42"), ("100 dollars", "100"), (r"\text{hello}", "hello"),
    (r"\boxed{42}", "42"), ("1,234,567", "1234567"), ("a b c", "bc"), ("42<|endoftext|>", "42"), ("42<|im_end|>", "42"),
])  # fmt: skip
def test_minerva_normalisation(raw, want):
    assert dapo.normalize_final_answer(raw) == want


def test_dapo_scoring():
    assert dapo.is_correct_strict_box(r"long preamble … \boxed{42}", "42") == (1, "42")
    assert dapo.is_correct_strict_box(r"\boxed{43}", "42") == (-1, "43") and dapo.is_correct_strict_box("plain 42", "42") == (-1, None)
    assert dapo.is_correct_minerva("Long solution. Answer: 42", "42") == (True, "42")
    assert dapo.is_correct_minerva("Answer: 41 was a wrong guess.\nAnswer: 42", "42")[0]  # the last "Answer:" line counts
    assert not dapo.is_correct_minerva("just a number 42", "42")[0]
    assert dapo.verify(r"\boxed{42}", "42", strict_box_verify=True) == (True, "42") and dapo.verify("Answer: 42", "42")[0]
    assert dapo.compute_score(r"\boxed{42}", "42", strict_box_verify=True) == {"score": 1.0, "acc": True, "pred": "42"}
    out = dapo.compute_score(r"\boxed{43}", "42", strict_box_verify=True)
    assert out["score"] == -1.0 and out["acc"] is False
    assert dapo.compute_score(r"\boxed{42}" + " filler" * 60, "42", strict_box_verify=True)["score"] == -1.0  # only the last 300 characters count


@pytest.mark.parametrize("response,label,want", [
    (r"scratch \boxed{wrong}</think>\boxed{42}", "42", 1), (r"Scratch work \boxed{wrong}###Response\boxed{42}", "42", 1),
    (r"\boxed{42}", "42", 0),  # neither marker: nothing is graded
    ("plain</think>no box here", "42", 0), (r"</think>\boxed{42}", "", 0), (r"</think>\boxed{42}", 42, 1),
    (r"</think>\boxed{42}", r"\boxed{42}", 1), (r"</think>\boxed{43}", "42", 0), (r"</think>\boxed{\frac{1}{2}}", "0.5", 1),
])  # fmt: skip
def test_deepscaler_reward(response, label, want):
    assert deepscaler(response, label) == want


def test_f1_reward():
    for raw, want in [("The Quick Brown Fox.", "quick brown fox"), ("An apple, a day", "apple day"), ("HELLO   WORLD", "hello world"),
                      ("a.b,c!", "abc"), ("", ""), ("the", "")]:  # fmt: skip
        assert normalize_answer(raw) == want
    assert f1_score("Paris is the capital", "Paris is the capital") == (1.0, 1.0, 1.0)
    f1, p, r = f1_score("the brown fox", "a quick brown fox")  # 2 of 2 predicted, 2 of 3 wanted
    assert p == pytest.approx(1.0) and r == pytest.approx(2 / 3) and f1 == pytest.approx(0.8)
    assert f1_score("apple banana", "carrot date") == (0, 0, 0) and f1_score(None, "anything") == (0, 0, 0)
    for special in ("yes", "no", "noanswer"):  # these only ever match themselves
        assert f1_score(special, "some other phrase") == (0, 0, 0) and f1_score("some other phrase", special) == (0, 0, 0)
    assert f1_score("yes", "yes") == (1.0, 1.0, 1.0)


def test_gpqa_reward():
    letters = gpqa.DEFAULT_VALID_LETTERS
    for response, want in [("The answer is B.", "B"), ("Answer: C", "C"), ("My choice is D", "D"), ("A is correct here", "A"),
                           ("E is the correct option", "E"), ("Final answer: B", "B"), ("the final option is C", "C"),
                           ("we ruled out A, then B, settled on C", "C"), ("no idea, sorry", None), ("", None), (None, None),
                           ("Let me think… Answer: A is wrong.</think>The answer is B.", "B")]:  # fmt: skip
        assert gpqa._extract_letter_from_response(response, letters) == want, response
    assert gpqa._extract_letter_from_response("Answer: C, but actually A was right, no wait B.", ["A", "B"]) == "B"
    R = gpqa.compute_gpqa_reward
    assert R("The answer is C.", label="C") == 1.0 and R("The answer is C.", label="D") == 0.0
    assert R("Answer: C", label=2, metadata={"choices": ["alpha", "beta", "gamma", "delta"]}) == 1.0
    assert R("Answer: B", label=1, metadata={"choices": {"a": "first", "b": "second", "c": "third"}}) == 1.0
    assert R("I think the answer is B.", label="capital of france", metadata={"choices": ["London", "Capital of France", "Berlin"]}) == 1.0
    assert R("Definitely paris.", label="Paris", metadata={"choices": ["London", "Paris", "Berlin"]}) == 1.0  # answer text, no letter
    assert R("Answer: A", label="anything", metadata={"correct_letter": "a"}) == 1.0
    assert R(None, label="A") == 0.0 and R("random text", label="some answer") == 0.0
