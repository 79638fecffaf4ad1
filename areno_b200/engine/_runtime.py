"""ctypes bindings of ``libareno_runtime.so`` (C++ scheduler, block allocator, batch packer)."""

from __future__ import annotations

import ctypes
import threading

import numpy as np

_lock = threading.Lock()
_lib = None

_I, _L, _P = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p


def lib():
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            from areno_b200 import build

            path = build.runtime_lib_path()
            try:
                build.build_runtime()
            except Exception:
                if not path.exists():
                    raise
            l = ctypes.CDLL(str(path))
            l.areno_sched_create.restype = _P
            l.areno_sched_create.argtypes = [_I] * 5
            l.areno_sched_destroy.argtypes = [_P]
            l.areno_sched_add.argtypes = [_P, _L, _I, _I]
            l.areno_sched_plan_prefill.argtypes = [_P, _I, _P, _P, _P, _P, _P]
            l.areno_sched_reserve_decode.argtypes = [_P, _I, _I, _P, _P, _P]
            l.areno_sched_advance.argtypes = [_P, _I]
            l.areno_sched_advance.restype = None
            l.areno_sched_finish.argtypes = [_P, _I]
            l.areno_sched_preempt_victim.argtypes = [_P]
            l.areno_sched_requeue.argtypes = [_P, _I, _I, _I]
            l.areno_sched_slot_pages.argtypes = [_P, _I, _P, _I]
            l.areno_sched_slot_seq_len.argtypes = [_P, _I]
            l.areno_sched_slot_request.argtypes = [_P, _I]
            l.areno_sched_slot_request.restype = _L
            for name in ("num_running", "num_waiting", "num_free_pages", "active_extent", "num_decoding",
                         "clear_waiting", "max_seq_len"):
                getattr(l, f"areno_sched_{name}").argtypes = [_P]
            l.areno_pack_indices.argtypes = [_P, _I, _I, _P, _P, _P, _P, _P]
            l.areno_pack_indices.restype = _L
            _lib = l
    return _lib


def _np_ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


class Scheduler:
    """Thin object wrapper over the C++ scheduler."""

    def __init__(self, max_slots: int, num_pages: int, page_size: int, max_pages_per_seq: int,
                 max_prefill_tokens: int):
        self._l = lib()
        self._h = self._l.areno_sched_create(max_slots, num_pages, page_size, max_pages_per_seq, max_prefill_tokens)
        if not self._h:
            raise ValueError("invalid scheduler configuration")
        self.max_slots = max_slots
        self.max_pages_per_seq = max_pages_per_seq
        n = max(max_slots, 1)
        self._slot = np.zeros(n, np.int32)
        self._req = np.zeros(n, np.int64)
        self._start = np.zeros(n, np.int32)
        self._len = np.zeros(n, np.int32)
        self._last = np.zeros(n, np.int32)
        cap = max_slots * 8 + 64
        self._us, self._ui, self._up = (np.zeros(cap, np.int32) for _ in range(3))
        self._pages = np.zeros(max_pages_per_seq, np.int32)

    def close(self):
        if self._h:
            self._l.areno_sched_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def add(self, req_id: int, prompt_len: int, max_new: int) -> None:
        rc = self._l.areno_sched_add(self._h, req_id, prompt_len, max_new)
        if rc == -2:
            raise ValueError(f"request {req_id}: prompt_len + max_new_tokens exceeds the per-sequence page limit")
        if rc != 0:
            raise ValueError(f"request {req_id}: empty prompt")

    def plan_prefill(self):
        """-> list of (slot, req_id, start, length, is_last_chunk)."""
        n = self._l.areno_sched_plan_prefill(self._h, len(self._slot), _np_ptr(self._slot), _np_ptr(self._req),
                                             _np_ptr(self._start), _np_ptr(self._len), _np_ptr(self._last))
        return [(int(self._slot[i]), int(self._req[i]), int(self._start[i]), int(self._len[i]), bool(self._last[i]))
                for i in range(n)]

    def reserve_decode(self, steps: int):
        """-> list of (slot, page_index, page_id) newly allocated.  All or nothing: when the free pages do not
        cover every decoding slot's demand it raises ``MemoryError(slot)`` and no page has moved."""
        n = self._l.areno_sched_reserve_decode(self._h, steps, len(self._us), _np_ptr(self._us), _np_ptr(self._ui),
                                               _np_ptr(self._up))
        if n == -(self.max_slots + 1):
            raise RuntimeError("scheduler: page-update buffer too small for one decode step")
        if n < 0:
            raise MemoryError(-n - 1)
        return [(int(self._us[i]), int(self._ui[i]), int(self._up[i])) for i in range(n)]

    def advance(self, steps: int = 1) -> None:
        self._l.areno_sched_advance(self._h, steps)

    def finish(self, slot: int) -> None:
        self._l.areno_sched_finish(self._h, slot)

    def preempt_victim(self) -> int:
        """The decoding slot admitted last, or -1 when fewer than two sequences decode."""
        return int(self._l.areno_sched_preempt_victim(self._h))

    def requeue(self, slot: int, prompt_len: int, max_new: int) -> None:
        """Free the slot's pages and put its request back at the head of the waiting queue."""
        if self._l.areno_sched_requeue(self._h, slot, prompt_len, max_new) != 0:
            raise ValueError(f"slot {slot} cannot be re-queued")

    def slot_pages(self, slot: int) -> list[int]:
        n = self._l.areno_sched_slot_pages(self._h, slot, _np_ptr(self._pages), len(self._pages))
        return [int(x) for x in self._pages[: max(n, 0)]]

    def slot_seq_len(self, slot: int) -> int:
        return self._l.areno_sched_slot_seq_len(self._h, slot)

    def slot_request(self, slot: int) -> int:
        return int(self._l.areno_sched_slot_request(self._h, slot))

    @property
    def num_running(self) -> int:
        return self._l.areno_sched_num_running(self._h)

    @property
    def num_waiting(self) -> int:
        return self._l.areno_sched_num_waiting(self._h)

    @property
    def num_free_pages(self) -> int:
        return self._l.areno_sched_num_free_pages(self._h)

    @property
    def active_extent(self) -> int:
        return self._l.areno_sched_active_extent(self._h)

    @property
    def num_decoding(self) -> int:
        return self._l.areno_sched_num_decoding(self._h)

    @property
    def max_seq_len(self) -> int:
        """Longest context among the decoding slots, counting the token of the step being planned."""
        return self._l.areno_sched_max_seq_len(self._h)

    def clear_waiting(self) -> int:
        return self._l.areno_sched_clear_waiting(self._h)


def pack_indices(lengths: np.ndarray, max_len: int):
    """Padded [B, T] -> (token_rows, token_cols, action_idx, action_rows) index arrays (int64)."""
    l = lib()
    lengths = np.ascontiguousarray(lengths, dtype=np.int64)
    total = int(np.clip(lengths, 1, max_len).sum())
    rows, cols = np.empty(total, np.int64), np.empty(total, np.int64)
    aidx, arows = np.empty(total, np.int64), np.empty(total, np.int64)
    na = ctypes.c_longlong(0)
    l.areno_pack_indices(_np_ptr(lengths), len(lengths), int(max_len), _np_ptr(rows), _np_ptr(cols), _np_ptr(aidx),
                         _np_ptr(arows), ctypes.byref(na))
    return rows, cols, aidx[: na.value], arows[: na.value]
