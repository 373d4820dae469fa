"""Streaming text assembly: incremental detokenisation and stop-string matching.

``Detokenizer`` turns a growing id sequence into text deltas without ever emitting half of a
multi-byte character (it waits while the decoded tail ends in U+FFFD). ``StopMatcher`` releases
only text that can no longer become part of a stop string and cuts the output right before the
first match (reference behaviour: ``engine/text.py:20-79``).
"""

from __future__ import annotations

REPLACEMENT = "�"
CONTEXT_TOKENS = 6  # already-emitted ids kept as left context so that joins decode as in the full text


def decoder_of(tokenizer):
    """``ids -> text`` (special tokens skipped) of a Hugging Face tokenizer. Its ``decode`` spends most of its time
    in Python-side argument handling (about 50 us a call, twice per streamed token); when the tokenizer is a fast one
    that does no clean-up of spaces, the Rust backend's ``decode`` gives the same text in a few microseconds. The
    shortcut is taken only after it has reproduced the wrapper's output on a sample of ids, once per tokenizer."""
    cached = getattr(tokenizer, "_direct_decode", None)
    if cached is not None:
        return cached

    def slow(ids: list[int]) -> str:
        return tokenizer.decode(ids, skip_special_tokens=True)

    chosen = slow
    backend = getattr(tokenizer, "backend_tokenizer", None)
    if backend is not None and not getattr(tokenizer, "clean_up_tokenization_spaces", False):
        def fast(ids: list[int]) -> str:
            return backend.decode(ids, skip_special_tokens=True)

        try:
            n = len(tokenizer)
            step = max(1, n // 256)
            sample = list(range(0, n, step))[:256] + list(getattr(tokenizer, "all_special_ids", []))
            windows = [sample[i : i + 7] for i in range(0, len(sample), 3)]
            if all(fast(w) == slow(w) for w in windows):
                chosen = fast
        except Exception:  # noqa: BLE001 - any surprise: keep the wrapper
            chosen = slow
    try:
        tokenizer._direct_decode = chosen
    except Exception:  # noqa: BLE001 - a tokenizer object that takes no attributes
        pass
    return chosen


class Detokenizer:
    def __init__(self, tokenizer) -> None:
        self.tok = tokenizer
        self._decode = decoder_of(tokenizer)
        self.context: list[int] = []  # emitted ids that still influence how the next ones decode
        self.pending: list[int] = []  # ids not yet turned into text

    def _text(self, ids: list[int]) -> str:
        return self._decode(ids) if ids else ""

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
        # the stop string that is complete first wins (of two that end together, the one that starts earlier), which
        # is what arrives first when the text comes in one character at a time: the cut does not depend on how the
        # text was chunked, even for stop strings that overlap
        hits = [(i + len(s), i) for s, i in ((s, buf.find(s)) for s in self.stops) if i >= 0]
        if hits:
            self.stopped, self.held = True, ""
            return buf[: min(hits)[1]]
        n_out = max(len(buf) - self.keep, 0)
        self.held = buf[n_out:]
        return buf[:n_out]

    def flush(self) -> str:
        out, self.held = ("" if self.stopped else self.held), ""
        return out
