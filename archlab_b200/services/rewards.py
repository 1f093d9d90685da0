"""Exact final-answer reward for unitless rational-valued mathematics.

Contract (the reference's `exact-rational-scalar-v1` backend, src/archlab/rl/rewards.py:1-262, vectors in its
tests/test_rl_rewards.py): an answer is accepted only if it is bounded numeric arithmetic over integers, finite
decimals / scientific notation, fractions (also ``\\frac{..}{..}``) and percentages; it is compared as an exact
rational, never with a tolerance; a completion is rewarded only for one unambiguous final answer (a single
``\\boxed{}``, one "final answer" marker, or a bare scalar), and nothing generated is ever evaluated as code.
Variables, units, sets, roots and equations are unsupported even when answer and reference are the same string.

Implementation: a tokenizer producing typed tokens, a precedence-climbing evaluator over ``fractions.Fraction``
with explicit resource limits, and an extractor built from three small scanners (reasoning block, box, marker).
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from fractions import Fraction

REWARD_BACKEND = "exact-rational-scalar-v1"
MAX_ANSWER_CHARACTERS = 512
MAX_COMPLETION_CHARACTERS = 65536
LIMITS = {"tokens": 128, "nesting": 16, "integer_bits": 4096, "literal_chars": 128, "sci_exponent": 128, "power": 32}

_LEX = re.compile(r"\s*(?:(?P<num>(?:\d+(?:\.\d*)?|\.\d+)(?:[eE][+-]?\d+)?)|(?P<frac>\\[dt]?frac)|(?P<op>[-+*/^(){}%]))")
_BINARY = {"+": (1, Fraction.__add__), "-": (1, Fraction.__sub__), "*": (2, Fraction.__mul__), "/": (2, Fraction.__truediv__)}
_CLOSER = {"(": ")", "{": "}"}
# LaTeX spellings rewritten before lexing: (pattern, replacement)
_REWRITES = ((re.compile(r"\\(?:left|right)\b"), ""), (re.compile(r"\\[,!;:]|\\q?quad\b"), " "),
             (re.compile(r"\\times|\\cdot"), "*"), (re.compile(r"\\div"), "/"), (re.compile(r"\\%"), "%"), (re.compile("\u2212"), "-"))
_THOUSANDS = re.compile(r"(?<![\d.,])\d{1,3}(?:,\d{3})+(?![\d,])")
_MATH_DELIMITERS = (("$$", "$$"), (r"\[", r"\]"), (r"\(", r"\)"), ("$", "$"))
_BOX = re.compile(r"\\f?box(?:ed)?\b")
_MARKER = re.compile(r"(?:^|\n)\s*(?:final\s+answer|answer)\s*:|\bthe\s+answer\s+is\s*:?|(?:^|\n)\s*####\s*", re.IGNORECASE)


class _Rejected(Exception):
    """The text is outside the supported grammar or over a resource limit."""


def _bounded(x: Fraction) -> Fraction:
    if max(x.numerator.bit_length(), x.denominator.bit_length()) > LIMITS["integer_bits"]:
        raise _Rejected
    return x


def _lex(text: str) -> list[tuple[str, object]]:
    out, pos = [], 0
    text = text.rstrip()
    while pos < len(text):
        m = _LEX.match(text, pos)
        if m is None:
            raise _Rejected
        if m.group("num") is not None:
            lit = m.group("num")
            mantissa, _, exponent = lit.lower().partition("e")
            if len(lit) > LIMITS["literal_chars"] or (exponent and abs(int(exponent)) > LIMITS["sci_exponent"]):
                raise _Rejected
            out.append(("num", _bounded(Fraction(lit))))
        elif m.group("frac") is not None:
            out.append(("frac", None))
        else:
            out.append(("op", m.group("op")))
        if len(out) > LIMITS["tokens"]:
            raise _Rejected
        pos = m.end()
    return out


class _Evaluator:
    """value := term (binary term)* by precedence climbing; term := sign* atom ['^' term-of-signs] ['%']."""

    def __init__(self, tokens):
        self.toks, self.i, self.nesting = tokens, 0, 0

    def _peek_op(self):
        return self.toks[self.i][1] if self.i < len(self.toks) and self.toks[self.i][0] == "op" else None

    def _expect(self, op: str) -> None:
        if self._peek_op() != op:
            raise _Rejected
        self.i += 1

    def value(self, floor: int = 1) -> Fraction:
        left = self.signed()
        while (op := self._peek_op()) in _BINARY and _BINARY[op][0] >= floor:
            level, fn = _BINARY[op]
            self.i += 1
            right = self.value(level + 1)
            if op == "/" and right == 0:
                raise _Rejected
            left = _bounded(fn(left, right))
        return left

    def signed(self) -> Fraction:
        self.nesting += 1
        if self.nesting > LIMITS["nesting"]:
            raise _Rejected
        try:
            if (op := self._peek_op()) in ("+", "-"):
                self.i += 1
                inner = self.signed()
                return -inner if op == "-" else inner
            return self.powered()
        finally:
            self.nesting -= 1

    def powered(self) -> Fraction:
        base = self.atom()
        if self._peek_op() == "^":
            self.i += 1
            e = self.signed()
            if e.denominator != 1 or abs(e.numerator) > LIMITS["power"] or (base == 0 and e <= 0):
                raise _Rejected
            base = _bounded(base ** e.numerator)
        if self._peek_op() == "%":
            self.i += 1
            base = _bounded(base / 100)
        return base

    def group(self, opener: str) -> Fraction:
        self._expect(opener)
        inner = self.value()
        self._expect(_CLOSER[opener])
        return inner

    def atom(self) -> Fraction:
        if self.i >= len(self.toks):
            raise _Rejected
        kind, payload = self.toks[self.i]
        if kind == "num":
            self.i += 1
            return payload
        if kind == "frac":
            self.i += 1
            top, bottom = self.group("{"), self.group("{")
            if bottom == 0:
                raise _Rejected
            return _bounded(top / bottom)
        if payload in _CLOSER:
            return self.group(payload)
        raise _Rejected


def _strip_math_delimiters(text: str) -> str:
    text = text.strip()
    for left, right in _MATH_DELIMITERS:
        if len(text) >= len(left) + len(right) and text.startswith(left) and text.endswith(right):
            return text[len(left):len(text) - len(right)].strip()
    return text


def canonical_math_answer(answer: str) -> str | None:
    """``numerator`` or ``numerator/denominator`` in lowest terms for an answer of the supported subset, else None.
    The input is an answer, not a solution trace; decimals are compared exactly, so a rounded approximation of an
    exact fraction is a different number."""
    if not isinstance(answer, str) or not 0 < len(answer) <= MAX_ANSWER_CHARACTERS:
        return None
    text = _strip_math_delimiters(answer)
    for pattern, replacement in _REWRITES:
        text = pattern.sub(replacement, text)
    text = _THOUSANDS.sub(lambda m: m.group().replace(",", ""), text)     # 1,234 yes; the list "1,2" stays invalid
    try:
        ev = _Evaluator(_lex(text))
        result = ev.value()
        return str(result) if ev.i == len(ev.toks) else None
    except (_Rejected, ValueError, ZeroDivisionError, OverflowError, RecursionError):
        return None


def _after_reasoning(text: str) -> str | None:
    """The part of a completion after its (closed) think block; None while the block is still open."""
    opened, closed = "<think>" in text, "</think>" in text
    if opened and not closed:
        return None
    if closed:
        text = text.rsplit("</think>", 1)[1].strip()
    return None if ("<think>" in text or "</think>" in text) else text


def _brace_body(text: str, start: int) -> tuple[str, int] | None:
    """Body of the ``{...}`` group that opens at or after ``start`` (whitespace skipped) and the index after it."""
    while start < len(text) and text[start].isspace():
        start += 1
    if start >= len(text) or text[start] != "{":
        return None
    level = 0
    for end in range(start, len(text)):
        level += {"{": 1, "}": -1}.get(text[end], 0)
        if level > LIMITS["nesting"]:
            return None
        if level == 0:
            return text[start + 1:end].strip(), end + 1
    return None


def _boxed_answer(text: str, box: re.Match) -> str | None:
    before = list(_MARKER.finditer(text[:box.start()]))
    if len(before) > 1:
        return None
    if before:        # "Final answer: \boxed{..}" - nothing but math openers may sit between marker and box
        gap = text[before[0].end():box.start()].replace(r"\[", "").replace(r"\(", "")
        if gap.strip(" \t\r\n$"):
            return None
    found = _brace_body(text, box.end())
    if found is None:
        return None
    body, end = found
    tail = text[end:].replace(r"\]", "").replace(r"\)", "")
    return None if tail.strip(" \t\r\n.$") else body


def extract_final_answer(completion: str) -> str | None:
    """The one unambiguous final answer of a completion, or None.  Numbers are never mined from prose: the answer is
    a single box at the end, what follows a single final-answer marker, or the whole text."""
    if not isinstance(completion, str) or len(completion) > MAX_COMPLETION_CHARACTERS:
        return None
    text = _after_reasoning(completion.strip())
    if text is None:
        return None
    boxes = list(_BOX.finditer(text))
    if len(boxes) > 1:
        return None
    if boxes:
        answer = _boxed_answer(text, boxes[0])
    else:
        markers = list(_MARKER.finditer(text))
        if len(markers) > 1:
            return None
        answer = (text[markers[0].end():] if markers else text).strip()
        answer = _strip_math_delimiters(answer[:-1].rstrip() if answer.endswith(".") else answer)
    return answer if answer is not None and canonical_math_answer(answer) is not None else None


@dataclass(frozen=True)
class MathReward:
    answer: str | None
    canonical_answer: str | None
    canonical_reference: str | None
    correct: bool
    reason: str
    backend: str = REWARD_BACKEND

    @property
    def reward(self) -> float:
        return 1.0 if self.correct else 0.0


def verify_math_answer(completion: str, reference: str) -> MathReward:
    """Binary outcome reward against a reference answer (never against a reference solution trace)."""
    want = canonical_math_answer(reference)
    if want is None:
        return MathReward(None, None, None, False, "unsupported_reference")
    answer = extract_final_answer(completion)
    if answer is None:
        return MathReward(None, None, want, False, "missing_or_unsupported_final_answer")
    got = canonical_math_answer(answer)
    return MathReward(answer, got, want, got == want, "correct" if got == want else "incorrect")
