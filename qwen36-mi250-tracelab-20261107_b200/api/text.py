"""Streaming text assembly: incremental detokenisation and stop-string matching.

``Detokenizer`` turns a growing id sequence into text deltas without ever emitting half of a
multi-byte character (it waits while the decoded tail ends in U+FFFD). ``StopMatcher`` releases
only text that can no longer become part of a stop string and cuts the output right before the
first match (reference behaviour: ``engine/text.py:20-79``).
"""

from __future__ import annotations

REPLACEMENT = "�"
CONTEXT_TOKENS = 6  # already-emitted ids kept as left context so that joins decode as in the full text


class Detokenizer:
    def __init__(self, tokenizer) -> None:
        self.tok = tokenizer
        self.context: list[int] = []  # emitted ids that still influence how the next ones decode
        self.pending: list[int] = []  # ids not yet turned into text

    def _text(self, ids: list[int]) -> str:
        return self.tok.decode(ids, skip_special_tokens=True) if ids else ""

    def _delta(self) -> str:
        base = self._text(self.context)
        full = self._text(self.context + self.pending)
        return full[len(base):] if full.startswith(base) else full

    def push(self, token: int) -> str:
        self.pending.append(token)
        delta = self._delta()
        if not delta or delta.endswith(REPLACEMENT):
            return ""
        self.context = (self.context + self.pending)[-CONTEXT_TOKENS:]
        self.pending = []
        return delta

    def flush(self) -> str:
        delta = self._delta() if self.pending else ""
        self.context, self.pending = (self.context + self.pending)[-CONTEXT_TOKENS:], []
        return delta


class StopMatcher:
    def __init__(self, stops: list[str] | tuple[str, ...]) -> None:
        self.stops = [s for s in stops if s]
        self.keep = max((len(s) for s in self.stops), default=1) - 1
        self.held = ""
        self.stopped = False

    def push(self, text: str) -> str:
        if self.stopped:
            return ""
        if not self.stops:
            return text
        buf = self.held + text
        hits = [i for i in (buf.find(s) for s in self.stops) if i >= 0]
        if hits:
            self.stopped, self.held = True, ""
            return buf[: min(hits)]
        n_out = max(len(buf) - self.keep, 0)
        self.held = buf[n_out:]
        return buf[:n_out]

    def flush(self) -> str:
        out, self.held = ("" if self.stopped else self.held), ""
        return out
