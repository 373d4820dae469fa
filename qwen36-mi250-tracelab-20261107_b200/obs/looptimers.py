"""Per-iteration stage timers of the engine loop, reported on ``/health``.

Enabled with ``ENGINE_LOOP_TIMERS=1``. Each worker-loop iteration opens a record with ``begin()``;
code under measurement wraps itself in ``with stage("name")`` (or calls ``add``); ``end(batch)``
files the record under a key ``(kind, batch)`` where kind is ``pure`` (decode only) or ``mixed``
(the iteration also ran prefill). ``summary()`` gives count, mean, p50 and p90 per stage in
milliseconds. GPU spans are measured with CUDA events by ``gpu_span`` (reference:
``engine/looptimers.py:40-155``).
"""

from __future__ import annotations

import os
import time
from collections import defaultdict
from contextlib import contextmanager

ENABLED = os.environ.get("ENGINE_LOOP_TIMERS") == "1"
MAX_SAMPLES = 4096

_cur: dict[str, float] | None = None
_records: dict[tuple, dict[str, list[float]]] = defaultdict(lambda: defaultdict(list))
_gpu_pending: list[tuple[str, object, object]] = []


def now() -> float:
    return time.perf_counter()


def begin() -> None:
    global _cur
    if ENABLED:
        _cur = {"_t0": now()}


def add(name: str, seconds: float) -> None:
    if ENABLED and _cur is not None:
        _cur[name] = _cur.get(name, 0.0) + seconds


NVTX = os.environ.get("ENGINE_NVTX") == "1"  # also open an NVTX range per stage (visible to nsys / ncu --nvtx)


@contextmanager
def stage(name: str):
    if not (ENABLED or NVTX):
        yield
        return
    if NVTX:
        import torch

        torch.cuda.nvtx.range_push(name)
    t = now()
    try:
        yield
    finally:
        add(name, now() - t)
        if NVTX:
            torch.cuda.nvtx.range_pop()


def gpu_span(name: str):
    """Returns ``(start, stop)`` callables that bracket GPU work with CUDA events."""
    if not ENABLED:
        return (lambda: None), (lambda: None)
    import torch

    if not torch.cuda.is_available():  # the graph schedulers also run without a device (kernel by kernel on the CPU)
        return (lambda: None), (lambda: None)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def start() -> None:
        a.record()

    def stop() -> None:
        b.record()
        _gpu_pending.append((name, a, b))

    return start, stop


def _drain_gpu() -> None:
    keep = []
    for name, a, b in _gpu_pending:
        if b.query():
            add(name, a.elapsed_time(b) / 1e3)
        else:
            keep.append((name, a, b))
    _gpu_pending[:] = keep


def end(batch: int) -> None:
    global _cur
    if not ENABLED or _cur is None:
        return
    _drain_gpu()
    rec, _cur = _cur, None
    total = now() - rec.pop("_t0")
    if len(rec) == 0:
        return  # idle iteration
    rec["total"] = total
    key = ("mixed" if "prefill" in rec else "pure", batch)
    store = _records[key]
    for k, v in rec.items():
        lst = store[k]
        lst.append(v)
        if len(lst) > MAX_SAMPLES:
            del lst[: len(lst) - MAX_SAMPLES]


def _pct(sorted_vals: list[float], p: float) -> float:
    return sorted_vals[min(len(sorted_vals) - 1, int(p * len(sorted_vals)))]


def summary() -> dict:
    out = {}
    for (kind, batch), stages in sorted(_records.items()):
        entry = {}
        for name, vals in stages.items():
            s = sorted(vals)
            entry[name] = {"n": len(s), "mean_ms": 1e3 * sum(s) / len(s), "p50_ms": 1e3 * _pct(s, 0.5),
                           "p90_ms": 1e3 * _pct(s, 0.9)}
        out[f"{kind}:b{batch}"] = entry
    return out


def reset() -> None:
    _records.clear()
