"""Self-contained coding tasks: a tiny repository (one module with a seeded bug, one test file) per task,
generated from templates so that no network, checkout or package installation is needed.  Fields follow the
familiar SWE-bench names (``instance_id``, ``problem_statement``, ``FAIL_TO_PASS``) plus ``files`` and
``test_command`` so that a task can be materialised locally."""

from __future__ import annotations

import random

_TEMPLATES = [
    ("sum_range", "def sum_range(a, b):\n    \"\"\"Sum of the integers a..b inclusive.\"\"\"\n    return sum(range(a, b))\n",
     "def sum_range(a, b):\n    \"\"\"Sum of the integers a..b inclusive.\"\"\"\n    return sum(range(a, b + 1))\n",
     "from mod import sum_range\n\ndef test_inclusive():\n    assert sum_range(1, 4) == 10\n\ndef test_single():\n    assert sum_range(3, 3) == 3\n",
     "sum_range(a, b) must include b."),
    ("clamp", "def clamp(x, lo, hi):\n    if x < lo:\n        return lo\n    if x > hi:\n        return lo\n    return x\n",
     "def clamp(x, lo, hi):\n    if x < lo:\n        return lo\n    if x > hi:\n        return hi\n    return x\n",
     "from mod import clamp\n\ndef test_high():\n    assert clamp(9, 0, 5) == 5\n\ndef test_inside():\n    assert clamp(3, 0, 5) == 3\n",
     "clamp returns the lower bound for values above the upper bound."),
    ("is_palindrome", "def is_palindrome(s):\n    t = [c for c in s if c.isalnum()]\n    return t == t[::-1]\n",
     "def is_palindrome(s):\n    t = [c.lower() for c in s if c.isalnum()]\n    return t == t[::-1]\n",
     "from mod import is_palindrome\n\ndef test_case():\n    assert is_palindrome('Never odd or even')\n\ndef test_no():\n    assert not is_palindrome('abc')\n",
     "is_palindrome should ignore letter case."),
    ("chunks", "def chunks(xs, n):\n    return [xs[i:i + n] for i in range(0, len(xs) - 1, n)]\n",
     "def chunks(xs, n):\n    return [xs[i:i + n] for i in range(0, len(xs), n)]\n",
     "from mod import chunks\n\ndef test_tail():\n    assert chunks([1, 2, 3, 4, 5], 2) == [[1, 2], [3, 4], [5]]\n\ndef test_exact():\n    assert chunks([1, 2], 2) == [[1, 2]]\n",
     "chunks drops the last element when the length is 1 modulo n."),
    ("mean", "def mean(xs):\n    return sum(xs) / (len(xs) - 1)\n",
     "def mean(xs):\n    return sum(xs) / len(xs)\n",
     "from mod import mean\n\ndef test_mean():\n    assert mean([2, 4, 6]) == 4\n",
     "mean divides by the wrong count."),
    ("dedupe", "def dedupe(xs):\n    return list(set(xs))\n",
     "def dedupe(xs):\n    seen, out = set(), []\n    for x in xs:\n        if x not in seen:\n            seen.add(x)\n            out.append(x)\n    return out\n",
     "from mod import dedupe\n\ndef test_order():\n    assert dedupe([3, 1, 3, 2, 1]) == [3, 1, 2]\n",
     "dedupe must keep the first occurrence order."),
]


def make_task(index: int) -> dict:
    name, buggy, fixed, test, statement = _TEMPLATES[index % len(_TEMPLATES)]
    rng = random.Random(index)
    return {
        "instance_id": f"local__{name}-{index}", "repo": "local/snippets", "base_commit": "0" * 8,
        "problem_statement": statement, "files": {"mod.py": buggy, "test_mod.py": test},
        "FAIL_TO_PASS": [f"test_mod.py::{t.split('(')[0].replace('def ', '')}" for t in test.splitlines() if t.startswith("def test")],
        "PASS_TO_PASS": [], "test_command": "python -m pytest -q test_mod.py", "reference_fix": {"mod.py": fixed},
        "difficulty": rng.choice(["easy", "medium"]),
    }
