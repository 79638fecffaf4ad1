"""Native (C++) request scheduler and sequence packer."""

from __future__ import annotations

import numpy as np
import pytest

from areno_b200.engine._runtime import Scheduler, pack_indices


def test_fifo_admission_chunked_prefill_and_page_accounting():
    s = Scheduler(max_slots=2, num_pages=16, page_size=64, max_pages_per_seq=8, max_prefill_tokens=100)
    s.add(10, 150, 100)  # needs two prefill chunks (100 + 50)
    s.add(11, 30, 60)
    s.add(12, 40, 10)    # waits: only two slots
    assert (s.num_waiting, s.num_running) == (3, 0)
    plan = s.plan_prefill()
    assert plan == [(0, 10, 0, 100, False)]          # budget spent on the first request
    assert (s.num_running, s.num_waiting) == (1, 2)
    plan = s.plan_prefill()
    assert plan[0] == (0, 10, 100, 50, True)
    assert plan[1] == (1, 11, 0, 30, True)           # FIFO: next request fills the rest of the budget
    assert s.num_decoding == 2 and s.num_waiting == 1
    assert len(s.slot_pages(0)) == 3 and len(s.slot_pages(1)) == 1   # ceil(150/64), ceil(30/64)
    free_before = s.num_free_pages
    assert s.slot_seq_len(0) == 150 and s.slot_request(1) == 11
    # decoding past a page boundary allocates exactly one page for that slot
    updates = []
    for _ in range(45):
        updates += s.reserve_decode(1)
        s.advance(1)
    # slot 1 crosses 64 tokens after 34 steps, slot 0 crosses 192 after 42
    assert sorted((u[0], u[1]) for u in updates) == [(0, 3), (1, 1)]
    assert s.num_free_pages == free_before - len(updates)
    # finishing a slot returns its pages and admits the waiting request into the freed slot
    s.finish(1)
    assert s.num_running == 1
    plan = s.plan_prefill()
    assert plan == [(1, 12, 0, 40, True)]
    assert s.active_extent == 2
    s.finish(0)
    s.finish(1)
    assert s.num_free_pages == 16 and s.num_running == 0


def test_rejects_requests_that_cannot_fit_and_reports_memory_pressure():
    s = Scheduler(max_slots=4, num_pages=4, page_size=64, max_pages_per_seq=2, max_prefill_tokens=512)
    with pytest.raises(ValueError, match="page limit"):
        s.add(1, 100, 100)          # 200 tokens > 2 pages
    with pytest.raises(ValueError, match="empty prompt"):
        s.add(2, 0, 4)
    for rid in (3, 4, 5, 6):
        s.add(rid, 60, 60)          # each may grow to two pages; four pages in total
    assert len(s.plan_prefill()) == 4 and s.num_free_pages == 0
    for _ in range(4):
        s.reserve_decode(1)
        s.advance(1)
    with pytest.raises(MemoryError) as err:   # the fifth token of each sequence needs a second page
        s.reserve_decode(1)
    victim = int(err.value.args[0])
    assert 0 <= victim < 4
    assert s.clear_waiting() == 0


def test_pack_indices_maps_padded_rows_to_packed_tokens():
    lens = np.array([3, 1, 2, 9], dtype=np.int64)
    rows, cols, aidx, arows = pack_indices(lens, 4)          # the last row is clipped to the padded width
    assert rows.tolist() == [0, 0, 0, 1, 2, 2, 3, 3, 3, 3]
    assert cols.tolist() == [0, 1, 2, 0, 0, 1, 0, 1, 2, 3]
    # actions: every packed position whose successor belongs to the same row
    assert aidx.tolist() == [0, 1, 4, 6, 7, 8]
    assert arows.tolist() == [0, 0, 2, 3, 3, 3]


def test_longest_sequence_waiting_queue_and_slot_reuse():
    s = Scheduler(max_slots=3, num_pages=32, page_size=64, max_pages_per_seq=8, max_prefill_tokens=512)
    assert s.max_seq_len == 0 and s.active_extent == 0
    for rid, n in ((1, 20), (2, 200), (3, 70), (4, 10), (5, 10)):
        s.add(rid, n, 32)
    plan = s.plan_prefill()
    assert [(p[0], p[1]) for p in plan] == [(0, 1), (1, 2), (2, 3)] and s.num_waiting == 2
    assert s.max_seq_len == 200                              # the decode graph's context bucket follows the longest row
    s.reserve_decode(1)
    s.advance(1)
    assert s.max_seq_len == 201 and s.slot_seq_len(0) == 21
    s.finish(1)                                              # the longest leaves: the bound drops to the next one
    assert s.max_seq_len == 71 and s.active_extent == 3      # slot 2 is still the highest active slot
    plan = s.plan_prefill()
    assert plan == [(1, 4, 0, 10, True)]                     # the freed slot is reused by the next waiting request
    assert s.clear_waiting() == 1 and s.num_waiting == 0     # request 5 never started
    for slot in (0, 1, 2):
        s.finish(slot)
    assert s.num_running == 0 and s.num_free_pages == 32 and s.max_seq_len == 0


def test_multi_step_reservation_allocates_all_pages_up_front():
    s = Scheduler(max_slots=1, num_pages=8, page_size=64, max_pages_per_seq=8, max_prefill_tokens=512)
    s.add(7, 60, 300)
    s.plan_prefill()
    updates = s.reserve_decode(100)                          # 60 -> 160 tokens: pages 2 and 3 at once
    assert [(u[0], u[1]) for u in updates] == [(0, 1), (0, 2)]
    s.advance(100)
    assert s.slot_seq_len(0) == 160 and len(s.slot_pages(0)) == 3
    assert s.reserve_decode(1) == []                         # still inside the third page


def test_reserve_decode_is_all_or_nothing_when_pages_run_out():
    # two sequences cross a page boundary on the same step and only one page is free: neither may be served,
    # and after room is made the retry reports the new pages of both
    s = Scheduler(max_slots=2, num_pages=3, page_size=4, max_pages_per_seq=4, max_prefill_tokens=64)
    s.add(1, 3, 8)
    s.add(2, 3, 8)
    assert len(s.plan_prefill()) == 2 and s.num_free_pages == 1      # one page each (prompt + first token)
    assert s.reserve_decode(1) == []                                 # token 4 still fits the first page
    s.advance(1)
    before = [s.slot_pages(0), s.slot_pages(1)]
    with pytest.raises(MemoryError) as err:
        s.reserve_decode(1)                                          # both need a second page, one is free
    assert int(err.value.args[0]) == 1                               # the slot whose share did not fit
    assert [s.slot_pages(0), s.slot_pages(1)] == before and s.num_free_pages == 1
    assert s.preempt_victim() == 1                                   # admitted last
    s.requeue(1, 3 + 2, 8 - 2)
    assert s.num_waiting == 1 and s.num_running == 1 and s.num_free_pages == 2
    ups = s.reserve_decode(1)
    assert [(u[0], u[1]) for u in ups] == [(0, 1)] and s.slot_pages(0)[1] == ups[0][2]
    s.finish(0)
    plan = s.plan_prefill()                                          # the evicted request comes back first
    assert [(p[1], p[3]) for p in plan] == [(2, 5)]


def test_preempt_victim_needs_two_decoding_sequences():
    s = Scheduler(max_slots=2, num_pages=2, page_size=4, max_pages_per_seq=2, max_prefill_tokens=64)
    s.add(7, 3, 5)
    s.plan_prefill()
    assert s.preempt_victim() == -1


def test_chunked_prompt_keeps_its_pages_between_chunks():
    # prefill budget below the prompt length: the first prompt is admitted and reserves all of its pages, so the
    # second long prompt has to wait instead of being admitted against pages the first still needs
    s = Scheduler(max_slots=4, num_pages=6, page_size=8, max_pages_per_seq=6, max_prefill_tokens=8)
    s.add(1, 30, 4)      # 31 tokens -> 4 pages
    s.add(2, 30, 4)
    plan = s.plan_prefill()
    assert [(p[1], p[2], p[3], p[4]) for p in plan] == [(1, 0, 8, False)]
    assert s.num_free_pages == 2 and s.num_running == 1 and s.num_waiting == 1
    admitted_second_at = None
    for step in range(40):
        plan = s.plan_prefill()
        if any(p[1] == 2 for p in plan) and admitted_second_at is None:
            admitted_second_at = step
            assert s.slot_request(0) != 1          # only after the first sequence had left
        if s.num_decoding:
            s.reserve_decode(1)                    # never raises: a mid-prompt sequence cannot be stranded
            s.advance(1)
        if s.slot_request(0) == 1 and s.slot_seq_len(0) >= 34:
            s.finish(0)
    assert admitted_second_at is not None
