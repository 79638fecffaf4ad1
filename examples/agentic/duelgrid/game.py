"""DuelGrid: a small turn-based grid duel.  The policy controls ``A``, a scripted opponent controls ``U``.
Each side has health and energy; tiles may hold a health pickup (+), an energy pickup (e) or a trap (x).
Actions are JSON objects from a strict legal list: move (n / s / e / w), attack (adjacent), wait."""

from __future__ import annotations

import copy
import random

SIZE = 6
DIRS = {"n": (-1, 0), "s": (1, 0), "w": (0, -1), "e": (0, 1)}


def new_state(seed: int) -> dict:
    rng = random.Random(seed)
    cells = [(r, c) for r in range(SIZE) for c in range(SIZE)]
    rng.shuffle(cells)
    a, u = cells[0], cells[1]
    extras = cells[2:11]
    tiles = {}
    for i, rc in enumerate(extras):
        tiles[f"{rc[0]},{rc[1]}"] = "+ex"[i % 3]
    return {"seed": seed, "turn": 0, "max_turns": 16, "A": {"pos": list(a), "hp": 6, "en": 3},
            "U": {"pos": list(u), "hp": 6, "en": 3}, "tiles": tiles}


def render(s: dict) -> str:
    rows = []
    for r in range(SIZE):
        row = []
        for c in range(SIZE):
            if s["A"]["pos"] == [r, c]:
                row.append("A")
            elif s["U"]["pos"] == [r, c]:
                row.append("U")
            else:
                row.append(s["tiles"].get(f"{r},{c}", "."))
        rows.append(" ".join(row))
    return "\n".join(rows) + f"\nA hp={s['A']['hp']} en={s['A']['en']} | U hp={s['U']['hp']} en={s['U']['en']} | turn {s['turn']}/{s['max_turns']}"


def _adjacent(p, q) -> bool:
    return abs(p[0] - q[0]) + abs(p[1] - q[1]) == 1


def legal_actions(s: dict, who: str) -> list[dict]:
    me, other = s[who], s["U" if who == "A" else "A"]
    acts = [{"action": "wait"}]
    for d, (dr, dc) in DIRS.items():
        r, c = me["pos"][0] + dr, me["pos"][1] + dc
        if 0 <= r < SIZE and 0 <= c < SIZE and [r, c] != other["pos"]:
            acts.append({"action": "move", "dir": d})
    if me["en"] >= 1 and _adjacent(me["pos"], other["pos"]):
        acts.append({"action": "attack"})
    return acts


def apply(s: dict, who: str, act: dict) -> dict:
    s = copy.deepcopy(s)
    me, other = s[who], s["U" if who == "A" else "A"]
    kind = act.get("action")
    if kind == "move" and act in legal_actions(s, who):
        dr, dc = DIRS[act["dir"]]
        me["pos"] = [me["pos"][0] + dr, me["pos"][1] + dc]
        key = f"{me['pos'][0]},{me['pos'][1]}"
        tile = s["tiles"].pop(key, None)
        if tile == "+":
            me["hp"] = min(8, me["hp"] + 2)
        elif tile == "e":
            me["en"] = min(5, me["en"] + 2)
        elif tile == "x":
            me["hp"] -= 1
    elif kind == "attack" and act in legal_actions(s, who):
        me["en"] -= 1
        other["hp"] -= 2
    else:   # wait (or an illegal action, which costs the turn)
        me["en"] = min(5, me["en"] + 1)
    return s


def opponent_policy(s: dict) -> dict:
    """Scripted ``U``: attack when possible, otherwise step toward ``A`` (avoiding traps when it can)."""
    acts = legal_actions(s, "U")
    if {"action": "attack"} in acts:
        return {"action": "attack"}
    best, best_d = {"action": "wait"}, 99
    for a in acts:
        if a["action"] != "move":
            continue
        dr, dc = DIRS[a["dir"]]
        r, c = s["U"]["pos"][0] + dr, s["U"]["pos"][1] + dc
        d = abs(r - s["A"]["pos"][0]) + abs(c - s["A"]["pos"][1]) + (2 if s["tiles"].get(f"{r},{c}") == "x" else 0)
        if d < best_d:
            best, best_d = a, d
    return best


def outcome(s: dict) -> str | None:
    if s["U"]["hp"] <= 0:
        return "win"
    if s["A"]["hp"] <= 0:
        return "loss"
    if s["turn"] >= s["max_turns"]:
        return "win" if s["A"]["hp"] > s["U"]["hp"] else ("draw" if s["A"]["hp"] == s["U"]["hp"] else "loss")
    return None


def parse_action(text: str) -> dict:
    import json
    import re

    m = re.search(r"\{[^{}]*\}", text or "")
    if not m:
        return {"action": "invalid"}
    try:
        act = json.loads(m.group(0))
    except ValueError:
        return {"action": "invalid"}
    return act if isinstance(act, dict) else {"action": "invalid"}


def step(s: dict, answer: str) -> tuple[dict, bool]:
    """One full turn: the policy's answer (an illegal one becomes ``wait``), then the scripted opponent.
    Returns the new state and whether the answer was legal."""
    act = parse_action(answer)
    legal = act in legal_actions(s, "A")
    s = apply(s, "A", act if legal else {"action": "wait"})
    if outcome(s) is None:
        s = apply(s, "U", opponent_policy(s))
    s["turn"] += 1
    return s, legal


def replay(start: dict, answers: list[str]) -> dict:
    """Deterministic replay of a finished episode from the policy's answers (used by the reward)."""
    s, illegal = copy.deepcopy(start), 0
    for a in answers:
        if outcome(s) is not None:
            break
        s, ok = step(s, a)
        illegal += 0 if ok else 1
    return {"outcome": outcome(s), "hp": s["A"]["hp"], "enemy_hp": s["U"]["hp"], "illegal": illegal, "turns": s["turn"]}
