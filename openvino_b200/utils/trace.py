"""Phase tracing: named scopes around the API entry points, passes, request stages and serving steps.

``scope(domain, name)`` is a context manager. When tracing is on (``enable()`` or ``OVB_TRACE=1``) it records
(domain, name, start, duration, thread) in a bounded in-process buffer and, on a CUDA machine, pushes an NVTX range of
the same name so that the scopes line up with the kernels in a timeline. ``dump_chrome_trace(path)`` writes the buffer
in the Chrome / Perfetto trace-event format; ``summary()`` aggregates per (domain, name). Domains mirror the
reference's ITT domains (src/inference/src/itt.hpp:17-23: ov, ov::ReadTime, ov::LoadTime, ov::phases; src/core/src/
itt.hpp:20-24: ov::core, ov::pass, ov::Op::exec). Off, a scope costs one attribute check.
"""
from __future__ import annotations

import collections
import json
import os
import sys
import threading
import time
from contextlib import contextmanager
from typing import Dict, List, Tuple

_enabled = os.environ.get("OVB_TRACE", "") not in ("", "0")
_events: "collections.deque" = collections.deque(maxlen=int(os.environ.get("OVB_TRACE_CAPACITY", "200000")))
_lock = threading.Lock()


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled


def clear() -> None:
    with _lock:
        _events.clear()


def _nvtx():
    torch = sys.modules.get("torch")
    if torch is None or not torch.cuda.is_available():
        return None
    return torch.cuda.nvtx


@contextmanager
def scope(domain: str, name: str):
    if not _enabled:
        yield
        return
    nv = _nvtx()
    if nv is not None:
        nv.range_push("%s/%s" % (domain, name))
    t0 = time.perf_counter_ns()
    try:
        yield
    finally:
        dur = time.perf_counter_ns() - t0
        if nv is not None:
            nv.range_pop()
        with _lock:
            _events.append((domain, name, t0, dur, threading.get_ident()))


def events() -> List[Tuple[str, str, int, int, int]]:
    with _lock:
        return list(_events)


def summary() -> Dict[Tuple[str, str], Dict[str, float]]:
    """(domain, name) -> {count, total_ms, max_ms}."""
    out: Dict[Tuple[str, str], Dict[str, float]] = {}
    for d, n, _, dur, _ in events():
        s = out.setdefault((d, n), {"count": 0, "total_ms": 0.0, "max_ms": 0.0})
        s["count"] += 1
        s["total_ms"] += dur / 1e6
        s["max_ms"] = max(s["max_ms"], dur / 1e6)
    return out


def dump_chrome_trace(path: str) -> int:
    """Write the recorded scopes as complete ("X") trace events; returns the number of events."""
    evs = events()
    data = [{"name": n, "cat": d, "ph": "X", "ts": t0 / 1e3, "dur": dur / 1e3, "pid": os.getpid(), "tid": tid} for d, n, t0, dur, tid in evs]
    with open(path, "w") as f:
        json.dump({"traceEvents": data, "displayTimeUnit": "ms"}, f)
    return len(data)
