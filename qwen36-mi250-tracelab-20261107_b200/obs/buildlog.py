"""Record of native-code builds and loads, with a ``serving`` flag.

The reference logs every Triton JIT compile and whether it happened while serving
(``engine/fast/jit_log.py:33-77``), because a compile after ``/health`` stalls requests. This
engine compiles nothing at run time; the equivalent guarantee is that the kernel library is built
ahead of time and loaded once. ``ENGINE_LOG_JIT=1`` prints each load; ``events()`` lets a test or
``/health`` assert that no load happened after the server reported ready.
"""

from __future__ import annotations

import os
import time

ENABLED = os.environ.get("ENGINE_LOG_JIT") == "1"
_events: list[dict] = []
_serving = False


def mark_serving() -> None:
    global _serving
    _serving = True


def record(kind: str, what: str, seconds: float = 0.0) -> None:
    ev = {"t": time.time(), "kind": kind, "what": what, "seconds": seconds, "serving": _serving}
    _events.append(ev)
    if ENABLED:
        print(f"engine: native {kind} {what} ({seconds * 1e3:.1f} ms) serving={_serving}", flush=True)


def events(serving_only: bool = False) -> list[dict]:
    return [e for e in _events if e["serving"] or not serving_only]
