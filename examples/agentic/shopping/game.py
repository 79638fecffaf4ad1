"""Shopping-kit task: pick one catalogue item per required category, honour feature constraints and a
budget.  Pure rule engine shared by the dataset generator, the agent loop and the reward."""

from __future__ import annotations

import random

CATEGORIES = ("tent", "stove", "lamp", "bag", "bottle", "mat")
FEATURES = ("light", "waterproof", "compact", "durable", "cheap")


def make_task(seed: int) -> dict:
    rng = random.Random(seed)
    cats = rng.sample(CATEGORIES, 3)
    catalog = []
    for c in CATEGORIES:
        for i in range(4):
            catalog.append({"id": f"{c}-{i}", "category": c, "price": rng.randrange(8, 60),
                            "features": sorted(rng.sample(FEATURES, rng.randrange(1, 4)))})
    # build the constraints around one feasible bundle so every task has a solution
    pick = {c: rng.choice([it for it in catalog if it["category"] == c]) for c in cats}
    needs = {c: rng.choice(pick[c]["features"]) for c in cats}
    budget = sum(it["price"] for it in pick.values()) + rng.randrange(0, 10)
    return {"seed": seed, "categories": cats, "needs": needs, "budget": budget, "catalog": catalog}


def search(task: dict, category: str) -> list[dict]:
    return [{"id": it["id"], "price": it["price"]} for it in task["catalog"] if it["category"] == category]


def inspect(task: dict, ids: list[str]) -> list[dict]:
    wanted = set(ids)
    return [it for it in task["catalog"] if it["id"] in wanted]


def check(task: dict, ids: list[str]) -> dict:
    items = inspect(task, ids)
    by_cat = {it["category"]: it for it in items}
    missing = [c for c in task["categories"] if c not in by_cat]
    unmet = [c for c in task["categories"] if c in by_cat and task["needs"][c] not in by_cat[c]["features"]]
    total = sum(it["price"] for it in items)
    ok = not missing and not unmet and total <= task["budget"] and len(items) == len(task["categories"])
    return {"ok": ok, "missing": missing, "unmet": unmet, "total": total, "budget": task["budget"]}


def describe(task: dict) -> str:
    needs = ", ".join(f"{c} must be {task['needs'][c]}" for c in task["categories"])
    return (f"Build a kit with one item from each of: {', '.join(task['categories'])}. Constraints: {needs}. "
            f"Total budget {task['budget']}. Use search_catalog, inspect_items, check_kit, then submit_bundle.")
