"""Named ranges around the engine's phases: NVTX for timeline tools, CUDA events for device-side phase times.

The reference has no tracing beyond wall-clock step timers (areno/api/trainer.py:340-348,
areno/api/backend/areno/backend.py:342-400).  Here every named path of a step (prefill, decode, sampling,
micro-batch forward / backward, optimizer, weight sync, ...) sits inside ``trace_range(name)``:

* ``ARENO_NVTX=1``          each range is pushed / popped as an NVTX range (visible in any NVTX-aware timeline).
* ``ARENO_PHASE_TIMERS=1``  each range is bracketed by CUDA events on the current stream; ``phase_report()``
                            turns them into milliseconds per name, ``phase_report_max(group)`` takes the max
                            over the ranks of a process group, which is the figure to quote for a multi-GPU run.

With neither variable set ``trace_range`` returns one shared no-op context manager: no allocation, no CUDA call.
Both switches can also be flipped at run time with ``configure``.
"""

from __future__ import annotations

import contextlib
import os
import threading
from collections import defaultdict

import torch

_lock = threading.Lock()
_nvtx = os.environ.get("ARENO_NVTX", "0") not in ("", "0")
_timers = os.environ.get("ARENO_PHASE_TIMERS", "0") not in ("", "0")
_pending: dict[str, list] = defaultdict(list)     # name -> [(start event, end event)]
_host_ms: dict[str, float] = defaultdict(float)   # ranges timed without a GPU (CPU runs)
_counts: dict[str, int] = defaultdict(int)
_NULL = contextlib.nullcontext()
# events are kept until phase_report(); cap them so a long run with timers left on cannot grow without bound
_MAX_PENDING = 1 << 16


def configure(nvtx: bool | None = None, timers: bool | None = None) -> None:
    """Switch NVTX ranges and / or event timers on or off at run time."""
    global _nvtx, _timers
    if nvtx is not None:
        _nvtx = bool(nvtx)
    if timers is not None:
        _timers = bool(timers)


def enabled() -> bool:
    return _nvtx or _timers


class _Range:
    __slots__ = ("name", "start", "t0", "pushed")

    def __init__(self, name: str):
        self.name = name
        self.start = None
        self.t0 = 0.0
        self.pushed = False

    def __enter__(self):
        cuda = torch.cuda.is_available()
        if _nvtx and cuda:
            torch.cuda.nvtx.range_push(self.name)
            self.pushed = True
        if _timers:
            if cuda:
                self.start = torch.cuda.Event(enable_timing=True)
                self.start.record()
            else:
                import time

                self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if _timers:
            if self.start is not None:
                end = torch.cuda.Event(enable_timing=True)
                end.record()
                with _lock:
                    lst = _pending[self.name]
                    if len(lst) < _MAX_PENDING:
                        lst.append((self.start, end))
                    _counts[self.name] += 1
            else:
                import time

                with _lock:
                    _host_ms[self.name] += (time.perf_counter() - self.t0) * 1e3
                    _counts[self.name] += 1
        if self.pushed:
            torch.cuda.nvtx.range_pop()
        return False


def trace_range(name: str):
    """Context manager for one named phase; a shared no-op when tracing is off."""
    if not (_nvtx or _timers):
        return _NULL
    return _Range(name)


def traced(name: str):
    """Decorator form of ``trace_range``."""

    def deco(fn):
        def wrapper(*args, **kwargs):
            with trace_range(name):
                return fn(*args, **kwargs)

        wrapper.__name__ = getattr(fn, "__name__", name)
        wrapper.__doc__ = fn.__doc__
        wrapper.__wrapped__ = fn
        return wrapper

    return deco


def phase_report(reset: bool = True) -> dict[str, dict[str, float]]:
    """``{name: {"ms": total device milliseconds, "count": ranges}}`` since the last reset.

    Synchronises the device once (the events must have completed to be read)."""
    with _lock:
        pending = {k: list(v) for k, v in _pending.items()}
        host = dict(_host_ms)
        counts = dict(_counts)
        if reset:
            _pending.clear()
            _host_ms.clear()
            _counts.clear()
    out: dict[str, dict[str, float]] = {}
    if pending and torch.cuda.is_available():
        torch.cuda.synchronize()
    for name, pairs in pending.items():
        out[name] = {"ms": float(sum(s.elapsed_time(e) for s, e in pairs)), "count": float(counts.get(name, len(pairs)))}
    for name, ms in host.items():
        cur = out.setdefault(name, {"ms": 0.0, "count": float(counts.get(name, 0))})
        cur["ms"] += ms
    return out


def phase_report_max(group=None, reset: bool = True) -> dict[str, dict[str, float]]:
    """``phase_report`` with each phase's time replaced by the maximum over the ranks of ``group``.

    Every rank must call it (it is a collective when ``torch.distributed`` is initialised).  Names are merged over
    ranks, so a phase that only some ranks ran is still reported."""
    local = phase_report(reset=reset)
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return local
    world = dist.get_world_size(group)
    gathered: list = [None] * world
    dist.all_gather_object(gathered, local, group=group)
    out: dict[str, dict[str, float]] = {}
    for rep in gathered:
        for name, rec in (rep or {}).items():
            cur = out.setdefault(name, {"ms": 0.0, "count": 0.0})
            cur["ms"] = max(cur["ms"], rec["ms"])
            cur["count"] = max(cur["count"], rec["count"])
    return out


def format_report(report: dict[str, dict[str, float]]) -> str:
    """One line per phase, longest first."""
    rows = sorted(report.items(), key=lambda kv: -kv[1]["ms"])
    width = max((len(k) for k, _ in rows), default=4)
    return "\n".join(f"{k:<{width}}  {v['ms']:10.2f} ms  x{int(v['count'])}" for k, v in rows)
