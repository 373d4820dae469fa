"""Time stamps along a request's path to its first byte, summarised on ``/health``.

Enabled with ``ENGINE_REQ_STAMPS=1``. The router adds an ``X-Engine-Sent`` header (its send time,
seconds since the epoch) so that the replica can attribute the hop; the handler marks ``parsed``,
``tokenized``, ``first_event`` and ``first_byte``. ``summary()`` reports mean/p50/p90 of each
stage's offset from the start in milliseconds (reference: ``engine/reqstamps.py:32-92``).
"""

from __future__ import annotations

import os
import threading
import time
from collections import defaultdict

ENABLED = os.environ.get("ENGINE_REQ_STAMPS") == "1"
MAX_SAMPLES = 4096
_lock = threading.Lock()
_samples: dict[str, list[float]] = defaultdict(list)


def start(sent_header: str | None = None) -> dict | None:
    if not ENABLED:
        return None
    t = time.time()
    stamp = {"_t0": t}
    if sent_header:
        try:
            stamp["router_hop"] = max(0.0, t - float(sent_header))
        except ValueError:
            pass
    return stamp


def mark(stamp: dict | None, name: str) -> None:
    if stamp is not None:
        stamp[name] = time.time() - stamp["_t0"]


def finish(stamp: dict | None) -> None:
    if stamp is None:
        return
    stamp.setdefault("done", time.time() - stamp["_t0"])
    with _lock:
        for k, v in stamp.items():
            if k.startswith("_"):
                continue
            lst = _samples[k]
            lst.append(v)
            if len(lst) > MAX_SAMPLES:
                del lst[: len(lst) - MAX_SAMPLES]


def summary() -> dict:
    out = {}
    with _lock:
        for k, vals in _samples.items():
            s = sorted(vals)
            out[k] = {"n": len(s), "mean_ms": 1e3 * sum(s) / len(s), "p50_ms": 1e3 * s[len(s) // 2],
                      "p90_ms": 1e3 * s[min(len(s) - 1, int(0.9 * len(s)))]}
    return out


def reset() -> None:
    with _lock:
        _samples.clear()
