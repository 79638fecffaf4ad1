"""Verifiable math reward: 1.0 when the last number of the completion equals the reference answer.

The completion's answer is taken after ``####`` or inside ``\\boxed{}`` when present, else the last
number in the text; numbers compare as exact rationals so ``0.50`` equals ``1/2``.
"""

from __future__ import annotations

import re
from fractions import Fraction

_NUM = re.compile(r"-?\d+(?:\.\d+)?(?:/\d+)?")


def _candidate(text: str) -> str | None:
    boxed = re.findall(r"\\boxed\{([^{}]*)\}", text)
    if boxed:
        text = boxed[-1]
    elif "####" in text:
        text = text.rsplit("####", 1)[-1]
    nums = _NUM.findall(text.replace(",", "").replace("$", ""))
    return nums[-1] if nums else None


def _value(text: str | None) -> Fraction | None:
    if text is None:
        return None
    try:
        return Fraction(text)
    except (ValueError, ZeroDivisionError):
        return None


def reward_fn(record) -> float:
    completion = getattr(record, "final_answer", None) or getattr(record, "completion", "") or ""
    got = _value(_candidate(str(completion)))
    want = _value(_candidate(str(getattr(record, "answer", "") or "")))
    return 1.0 if got is not None and want is not None and got == want else 0.0
