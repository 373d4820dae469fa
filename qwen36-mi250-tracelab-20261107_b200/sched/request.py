"""Request state: sampling parameters and the per-request generation record.

``Sampling`` carries the OpenAI-style knobs the wire protocol accepts (reference:
``engine/protocol.py:33-44``); ``Generation`` is what the scheduler tracks for one request
from admission to retirement (reference: ``engine/generator.py:433-543``).
"""

from __future__ import annotations

import itertools
import threading
from dataclasses import dataclass, field
from typing import Any, Callable


@dataclass
class Sampling:
    max_tokens: int | None = 16
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    seed: int | None = None
    stop: list[str] = field(default_factory=list)
    ignore_eos: bool = False
    min_tokens: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0


class EngineError(Exception):
    """A request-level failure with an HTTP status (400 bad request, 503 busy, ...)."""

    def __init__(self, message: str, status: int = 400, kind: str = "invalid_request_error") -> None:
        super().__init__(message)
        self.status, self.kind = status, kind


_ids = itertools.count(1)


@dataclass
class TokenEvent:
    token: int | None  # None: the request ended without a further token (EOS hit, cancelled, failed)
    finish_reason: str | None  # None while running; "length" | "stop" | "error" | "cancelled"
    error: EngineError | None = None


class Generation:
    """One request inside the engine."""

    def __init__(self, prompt: list[int], sampling: Sampling, on_event: Callable[["Generation", TokenEvent], None] | None = None) -> None:
        self.id = next(_ids)
        self.prompt = list(prompt)
        self.sampling = sampling
        self.on_event = on_event
        self.output: list[int] = []
        self.finish_reason: str | None = None
        self.cancelled = threading.Event()  # set by any thread; the engine latches it into cancel_now
        self.cancel_now = False
        # engine-owned
        self.slot: int = 0
        self.pages: list[int] = []
        self.computed = 0  # tokens whose KV / state are in the cache
        self.cached_tokens = 0  # of those, how many came from the prefix cache
        self.spans: list[tuple[int, int]] = []  # pending prefill spans [a, b)
        self.snapshot_at = 0  # boundary to snapshot during prefill (0 = none)
        self.next_token: int | None = None  # sampled, not yet fed back
        self.draft: list[int] = []  # MTP draft tokens following next_token
        self.mtp_computed = 0  # tokens covered by the MTP block's KV
        self.rng: Any = None
        self.user: Any = None  # opaque handle of the API layer
        self.spec_proposed = 0
        self.spec_accepted = 0

    @property
    def done(self) -> bool:
        return self.finish_reason is not None

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.output

    @property
    def remaining(self) -> int | None:
        if self.sampling.max_tokens is None:
            return None
        return self.sampling.max_tokens - len(self.output)

    def emit(self, event: TokenEvent) -> None:
        if self.on_event is not None:
            self.on_event(self, event)
