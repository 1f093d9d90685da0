"""Verifiable math rewards: exact rational comparison of one unambiguous final answer
(src/archlab/rl/rewards.py:32-260).  No tolerance: a rounded decimal is wrong unless mathematically equal."""
from __future__ import annotations

import re
from dataclasses import dataclass
from fractions import Fraction

MAX_ANSWER = 256
MAX_COMPLETION = 200_000
_BOX = re.compile(r"\\(?:boxed|fbox)\b")
_FINAL = re.compile(r"(?i)final answer\s*(?:is|:)?")
_TOKEN = re.compile(r"\s*(\d+\.\d*|\.\d+|\d+|\\frac|\\dfrac|\*\*|[-+*/^(){}%])")


class _Parser:
    def __init__(self, text: str):
        self.toks, pos = [], 0
        text = text.strip()
        while pos < len(text):
            m = _TOKEN.match(text, pos)
            if not m:
                raise ValueError("unsupported character")
            self.toks.append(m.group(1))
            pos = m.end()
        self.i = 0

    def peek(self):
        return self.toks[self.i] if self.i < len(self.toks) else None

    def take(self, tok=None):
        t = self.peek()
        if t is None or (tok is not None and t != tok):
            raise ValueError("unexpected token")
        self.i += 1
        return t

    def expression(self) -> Fraction:
        v = self.product()
        while self.peek() in ("+", "-"):
            v = v + self.product() if self.take() == "+" else v - self.product()
        return v

    def product(self) -> Fraction:
        v = self.unary()
        while self.peek() in ("*", "/"):
            v = v * self.unary() if self.take() == "*" else v / self.unary()
        return v

    def unary(self) -> Fraction:
        if self.peek() in ("+", "-"):
            return self.unary() if self.take() == "+" else -self.unary()
        return self.power()

    def power(self) -> Fraction:
        base = self.primary()
        if self.peek() in ("^", "**"):
            self.take()
            e = self.unary()
            if e.denominator != 1 or abs(e.numerator) > 64:
                raise ValueError("unsupported exponent")
            base = base ** e.numerator
        if abs(base.numerator).bit_length() > 4096 or base.denominator.bit_length() > 4096:
            raise OverflowError("result too large")
        return base

    def primary(self) -> Fraction:
        t = self.take()
        if t in ("\\frac", "\\dfrac"):
            self.take("{"); a = self.expression(); self.take("}")
            self.take("{"); b = self.expression(); self.take("}")
            return a / b
        if t in ("(", "{"):
            v = self.expression()
            self.take(")" if t == "(" else "}")
            return v
        if re.fullmatch(r"\d+\.\d*|\.\d+|\d+", t):
            v = Fraction(t)
            if self.peek() == "%":
                self.take()
                v /= 100
            return v
        raise ValueError("unsupported token")


def _unwrap(text: str) -> str:
    t = text.strip()
    for a, b in (("$$", "$$"), ("$", "$"), (r"\(", r"\)"), (r"\[", r"\]")):
        if t.startswith(a) and t.endswith(b) and len(t) >= len(a) + len(b):
            t = t[len(a):len(t) - len(b)].strip()
    return t


def canonical_math_answer(answer: str) -> str | None:
    if not isinstance(answer, str) or not answer or len(answer) > MAX_ANSWER:
        return None
    t = _unwrap(answer).replace("−", "-")
    t = re.sub(r"\\(?:left|right)\b", "", t)
    t = re.sub(r"\\(?:,|!|;|:)|\\(?:quad|qquad)\b", " ", t)
    t = t.replace(r"\times", "*").replace(r"\cdot", "*").replace(r"\div", "/").replace(r"\%", "%")
    t = re.sub(r"(?<![\d.,])\d{1,3}(?:,\d{3})+(?![\d,])", lambda m: m.group().replace(",", ""), t)
    try:
        p = _Parser(t)
        v = p.expression()
        return None if p.peek() is not None else str(v)
    except (ValueError, ZeroDivisionError, OverflowError, RecursionError):
        return None


def extract_final_answer(completion: str) -> str | None:
    """One boxed expression at the end, or one explicit final-answer marker, or a bare scalar; an open
    think block, several boxes / markers or trailing text are rejected."""
    if not isinstance(completion, str) or len(completion) > MAX_COMPLETION:
        return None
    text = completion.strip()
    if "<think>" in text and "</think>" not in text:
        return None
    if "</think>" in text:
        text = text.rsplit("</think>", 1)[-1].strip()
    if "<think>" in text or "</think>" in text:
        return None
    boxes = list(_BOX.finditer(text))
    if boxes:
        if len(boxes) != 1:
            return None
        start = boxes[0].end()
        while start < len(text) and text[start].isspace():
            start += 1
        if start == len(text) or text[start] != "{":
            return None
        depth, end = 1, start + 1
        while end < len(text) and depth:
            depth += (text[end] == "{") - (text[end] == "}")
            end += 1
        if depth or text[end:].replace(r"\]", "").replace(r"\)", "").strip(" \t\r\n.$"):
            return None
        answer = text[start + 1:end - 1].strip()
    else:
        marks = list(_FINAL.finditer(text))
        if len(marks) > 1:
            return None
        answer = text[marks[0].end():].strip() if marks else text
        answer = _unwrap(answer[:-1].rstrip() if answer.endswith(".") else answer)
    return answer if canonical_math_answer(answer) is not None else None


@dataclass(frozen=True)
class MathReward:
    answer: str | None
    canonical_answer: str | None
    canonical_reference: str | None
    correct: bool
    reason: str

    @property
    def reward(self) -> float:
        return float(self.correct)


def verify_math_answer(completion: str, reference: str) -> MathReward:
    want = canonical_math_answer(reference)
    if want is None:
        return MathReward(None, None, None, False, "unsupported_reference")
    ans = extract_final_answer(completion)
    if ans is None:
        return MathReward(None, None, want, False, "missing_or_unsupported_final_answer")
    got = canonical_math_answer(ans)
    return MathReward(ans, got, want, got == want, "correct" if got == want else "incorrect")
