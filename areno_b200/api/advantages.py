"""Generalised advantage estimation for PPO.

``A_t = sum_l (gamma lam)^l delta_{t+l}``, ``delta_t = r_t + gamma V_{t+1} - V_t`` with
``V_{T} = 0``; returns are ``A + V``.  An installed ``cugae`` module is used when present
(``areno/api/advantages.py:15-74`` in the reference); otherwise a backward recurrence.
"""

from __future__ import annotations

from collections.abc import Callable


def compute_gae(rewards, values, *, gamma: float, lam: float):
    fn = _resolve_cugae()
    if fn is not None:
        return fn(rewards, values, gamma=gamma, lam=lam)
    return _compute_gae_python(list(rewards), list(values), gamma=gamma, lam=lam)


def _resolve_cugae() -> Callable | None:
    try:
        import cugae
    except ImportError:
        return None
    for name in ("compute_gae", "gae", "generalized_advantage_estimation"):
        fn = getattr(cugae, name, None)
        if callable(fn):
            return fn
    return None


def _compute_gae_python(rewards: list[float], values: list[float], *, gamma: float, lam: float):
    if len(values) != len(rewards):
        raise ValueError(f"GAE requires one value per reward, got {len(values)} and {len(rewards)}")
    n = len(rewards)
    adv = [0.0] * n
    carry, nxt = 0.0, 0.0
    for t in reversed(range(n)):
        delta = rewards[t] + gamma * nxt - values[t]
        carry = delta + gamma * lam * carry
        adv[t] = carry
        nxt = values[t]
    return adv, [a + v for a, v in zip(adv, values)]
