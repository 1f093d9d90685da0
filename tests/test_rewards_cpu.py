"""Exact rational final-answer reward: the accepted grammar, the extraction rules and the resource limits
(golden vectors of the reference's tests/test_rl_rewards.py)."""
import pytest

from archlab_b200.services.rewards import (MAX_ANSWER_CHARACTERS, REWARD_BACKEND, canonical_math_answer,
                                           extract_final_answer, verify_math_answer)

EQUIVALENT = {
    "42": "42", "−42": "-42", " 1,234,567 ": "1234567", ".125": "1/8", "1.25e-2": "1/80", "2/4": "1/2",
    r"\frac{2}{4}": "1/2", r"-\dfrac{3}{\frac{9}{2}}": "-2/3", r"$\tfrac{ 1 }{ 2 }$": "1/2",
    r"\left(\frac{1}{2}+\frac{1}{3}\right)": "5/6", r"\frac{2^{3}}{4}": "2", "-2^2": "-4", "(-2)^2": "4", "25%": "1/4",
    r"25\%": "1/4", r"2\times3\div4": "3/2", "2^-2": "1/4", "2^3^2": "512", "1-2-3": "-4", "8/4/2": "1", "2*-3": "-6",
}


@pytest.mark.parametrize("answer,expected", EQUIVALENT.items())
def test_exact_scalar_equivalence(answer, expected):
    assert canonical_math_answer(answer) == expected


@pytest.mark.parametrize("completion", [
    r"After combining the terms, we obtain \boxed{\frac{2}{4}}.", r"Final answer: $\frac{2}{4}$.",
    r"The answer is: \frac{2}{4}.", "#### 0.5", "0.5", r"Final answer: \boxed{0.5}",
    r"<think>An intermediate \boxed{99} is not final.</think>\boxed{0.5}",
    r"reasoning from an open template</think>\boxed{0.5}",
])
def test_final_answer_formats(completion):
    r = verify_math_answer(completion, "1/2")
    assert r.correct and r.reward == 1.0 and r.reason == "correct" and r.backend == REWARD_BACKEND


@pytest.mark.parametrize("completion", [
    "I considered 42 but the answer is unknown.", r"\boxed{42} or \boxed{43}", r"\boxed{42} actually the answer is 43",
    "Final answer: 42\nFinal answer: 43", "42 dollars", r"\boxed{42\text{ or 43}}", r"\boxed{42", r"\boxed42",
    r"\boxed{42}/0", r"Final answer: 43, but \boxed{42}", "4 2", r"4\,2", "1,2", "nan", "inf", "1/0", "0^0",
    r"<think>\boxed{42}", r"</think><think>\boxed{42}", "__import__('os').system('echo 42')", "42; 0",
    r"\boxed{42}\text{ meters}", "50%%", "50%^2",
])
def test_no_reward_for_unsupported_or_adversarial_answers(completion):
    assert extract_final_answer(completion) is None
    assert verify_math_answer(completion, "42").reward == 0.0


@pytest.mark.parametrize("answer", [r"\sqrt{2}", "x+1", "x=2", "2 cm", "{1,2}", r"\pi"])
def test_symbolic_answers_and_units_are_never_rewarded(answer):
    r = verify_math_answer(answer, answer)
    assert r.reward == 0.0 and r.reason == "unsupported_reference"


def test_incorrect_differs_from_unparseable_and_decimals_are_exact():
    wrong = verify_math_answer(r"\boxed{41}", "42")
    assert (wrong.reason, wrong.canonical_answer, wrong.canonical_reference) == ("incorrect", "41", "42")
    missing = verify_math_answer("I do not know", "42")
    assert missing.reason == "missing_or_unsupported_final_answer" and missing.answer is None
    assert verify_math_answer("0.33333333333333", "1/3").reward == 0.0
    assert verify_math_answer("42.000000001", "42").reward == 0.0


@pytest.mark.parametrize("answer", ["9" * (MAX_ANSWER_CHARACTERS + 1), "1e999999", "9^999", "(" * 40 + "1" + ")" * 40,
                                    "+".join(["1"] * 70), "2^32^32"])
def test_resource_limits(answer):
    assert canonical_math_answer(answer) is None


def test_overlong_completion_is_not_scanned():
    assert extract_final_answer("x" * 70000 + r"\boxed{42}") is None
