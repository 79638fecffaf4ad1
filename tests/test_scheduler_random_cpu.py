"""Randomised walks over the C++ scheduler, driven the way the engine drives it (admit, prefill in chunks, reserve pages
for a decode step, advance, finish, re-queue under page pressure), with the bookkeeping invariants checked after every
operation: no page belongs to two sequences, pages are conserved, a sequence always has the pages its length needs,
requests are admitted in arrival order and every request eventually completes."""

from __future__ import annotations

import random

import pytest

from areno_b200.engine._runtime import Scheduler


def _check(s: Scheduler, live: dict[int, dict], num_pages: int, page: int) -> None:
    seen: set[int] = set()
    for slot in live:
        pages = s.slot_pages(slot)
        assert len(pages) == len(set(pages)) and not (seen & set(pages)), "a page is owned twice"
        seen |= set(pages)
        assert all(0 <= p < num_pages for p in pages)
        assert len(pages) * page >= s.slot_seq_len(slot), "a sequence outgrew its pages"
    assert s.num_free_pages + len(seen) == num_pages, "pages leaked or were invented"
    assert s.num_running == len(live) and s.num_decoding == sum(1 for v in live.values() if v["decoding"])


@pytest.mark.parametrize("seed", range(24))
def test_random_walk_keeps_pages_consistent_and_finishes_every_request(seed):
    rng = random.Random(seed)
    page = 16
    max_slots = rng.choice([1, 2, 3, 5])
    per_seq = rng.choice([3, 4, 6])
    num_pages = rng.randint(per_seq, per_seq * max_slots)                  # often less than every slot's worst case
    budget = rng.choice([8, 24, 64])
    s = Scheduler(max_slots, num_pages, page, per_seq, budget)
    live: dict[int, dict] = {}                   # slot -> {"req", "left" (decode steps still wanted), "decoding"}
    want: dict[int, int] = {}                    # request -> decode steps it still needs in total
    arrival: list[int] = []
    admitted: list[int] = []
    finished: set[int] = set()
    next_id, total = 0, rng.randint(4, 14)
    for _ in range(4000):
        # arrivals
        while next_id < total and rng.random() < 0.4:
            prompt = rng.randint(1, page * per_seq - 2)
            new = rng.randint(1, page * per_seq - prompt)
            s.add(next_id, prompt, new)
            want[next_id] = new
            arrival.append(next_id)
            next_id += 1
        # prefill: chunks of the prompts admitted so far, first come first served
        for slot, req, start, length, last in s.plan_prefill():
            assert length > 0 and length <= budget
            if slot not in live:
                if req not in admitted:
                    admitted.append(req)
                live[slot] = {"req": req, "left": want[req], "decoding": False}
                assert start == 0
            assert live[slot]["req"] == req
            if last:
                live[slot]["decoding"] = True
                live[slot]["left"] -= 1            # the prefill's last position samples the first new token
        _check(s, live, num_pages, page)
        # sequences whose budget is spent leave before the next step
        for slot in [k for k, v in live.items() if v["decoding"] and v["left"] <= 0]:
            finished.add(live[slot]["req"])
            s.finish(slot)
            del live[slot]
        # one decode step for everybody that decodes
        if any(v["decoding"] for v in live.values()):
            before = {slot: s.slot_pages(slot) for slot in live}
            try:
                s.reserve_decode(1)
            except MemoryError as err:
                assert before == {slot: s.slot_pages(slot) for slot in live}          # all or nothing: nothing moved
                victim = s.preempt_victim()
                if victim < 0:
                    victim = int(err.args[0])
                    assert sum(1 for v in live.values() if v["decoding"]) <= 1 or victim in live
                v = live.pop(victim)
                if s.num_decoding >= 2 or v["left"] <= 0 or rng.random() < 0.2:
                    # give up on it (the engine finishes a lone sequence with reason "length")
                    finished.add(v["req"])
                    s.finish(victim)
                else:
                    # back to the head of the queue with what it has so far as its new prompt
                    s.requeue(victim, s.slot_seq_len(victim), v["left"])
                    want[v["req"]] = v["left"]
                _check(s, live, num_pages, page)
                continue
            s.advance(1)
            for v in live.values():
                if v["decoding"]:
                    v["left"] -= 1
            _check(s, live, num_pages, page)
        # some sequences stop early (EOS)
        for slot in [k for k, v in live.items() if v["decoding"] and rng.random() < 0.05]:
            finished.add(live[slot]["req"])
            s.finish(slot)
            del live[slot]
        _check(s, live, num_pages, page)
        if next_id == total and not live and s.num_waiting == 0:
            break
    assert finished == set(range(total)), "a request was lost or never completed"
    assert s.num_free_pages == num_pages and s.num_running == 0 and s.num_waiting == 0
    # first admissions follow arrival order (re-queued requests return to the head of the queue)
    firsts = [r for i, r in enumerate(admitted) if r not in admitted[:i]]
    assert firsts == sorted(firsts)
