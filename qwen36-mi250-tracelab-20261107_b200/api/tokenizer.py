"""Tokenizer access: encode/decode, chat template rendering, exact incremental encoding.

``PromptEncoder`` makes tokenising a growing session prompt cost O(new text): it remembers recent
prompts with their token offsets and, when a new prompt shares a prefix with one of them, reuses
the ids up to a *safe cut* and encodes only the remainder. A cut is safe where the byte-level BPE
pre-tokenizer is certain to split whatever follows: right after a line break that is followed by
a non-space character, or right before a single space that follows a non-space character and
precedes one. The tokenizer's JSON is checked first; any other tokenizer kind just encodes in
full (reference: ``engine/inctok.py:58-214``). ``ENGINE_TOKENIZE_CHECK=1`` verifies every
incremental result against a full encode.
"""

from __future__ import annotations

import json
import os
import threading
from collections import OrderedDict
from pathlib import Path
from typing import Any


def safe_config(tokenizer_json: dict[str, Any]) -> bool:
    """Whether the tokenizers pipeline is the byte-level BPE kind the cut rule was derived for."""
    try:
        if tokenizer_json["model"]["type"] != "BPE":
            return False
        if tokenizer_json.get("normalizer") not in (None, {"type": "NFC"}):
            return False
        pre = tokenizer_json.get("pre_tokenizer") or {}
        kinds = [p.get("type") for p in pre.get("pretokenizers", [pre])]
        if "ByteLevel" not in kinds or not set(kinds) <= {"ByteLevel", "Split"}:
            return False
        for p in pre.get("pretokenizers", [pre]):
            if p.get("type") == "ByteLevel" and p.get("add_prefix_space"):
                return False
        return True
    except (KeyError, TypeError, AttributeError):
        return False


def _safe_cut(text: str, limit: int) -> int:
    """Largest safe cut position ``<= limit`` (0 when there is none)."""
    i = min(limit, len(text) - 1)
    while i > 0:
        prev, cur = text[i - 1], text[i]
        if prev == "\n" and not cur.isspace():
            return i
        if cur == " " and not prev.isspace() and i + 1 < len(text) and not text[i + 1].isspace() and i < limit:
            return i
        i -= 1
    return 0


class PromptEncoder:
    def __init__(self, backend, capacity: int = 256, enabled: bool = True) -> None:
        """``backend``: a ``tokenizers.Tokenizer`` (gives offsets). Disabled -> plain full encodes."""
        self.backend = backend
        self.enabled = enabled and backend is not None
        self.capacity = capacity
        self._lru: "OrderedDict[str, tuple[list[int], list[int]]]" = OrderedDict()
        self._lock = threading.Lock()
        self.check = os.environ.get("ENGINE_TOKENIZE_CHECK") == "1"
        self.stats = {"tokenize_calls": 0, "tokenize_reused_chars": 0, "tokenize_encoded_chars": 0}

    def _full(self, text: str) -> tuple[list[int], list[int]]:
        enc = self.backend.encode(text, add_special_tokens=False)
        return list(enc.ids), [e for _, e in enc.offsets]

    def encode(self, text: str) -> list[int]:
        if not self.enabled:
            raise RuntimeError("incremental encoder is disabled")
        with self._lock:
            self.stats["tokenize_calls"] += 1
            best, best_len = None, 0
            for old in reversed(self._lru):
                n = _common_prefix(old, text)
                if n > best_len:
                    best, best_len = old, n
                    if n == len(old):
                        break
            ids: list[int] | None = None
            if best is not None and best_len > 64:
                cut = _safe_cut(text, min(best_len, len(text) - 1)) if best_len < len(text) else 0
                if best_len == len(text) == len(best):
                    ids, ends = self._lru[best]
                    ids, ends = list(ids), list(ends)
                elif cut > 0:
                    old_ids, old_ends = self._lru[best]
                    k = _count_upto(old_ends, cut)
                    if k > 0 and old_ends[k - 1] == cut:
                        tail_ids, tail_ends = self._full(text[cut:])
                        ids = old_ids[:k] + tail_ids
                        ends = old_ends[:k] + [e + cut for e in tail_ends]
                        self.stats["tokenize_reused_chars"] += cut
                        self.stats["tokenize_encoded_chars"] += len(text) - cut
            if ids is None:
                ids, ends = self._full(text)
                self.stats["tokenize_encoded_chars"] += len(text)
            elif self.check:
                full, _ = self._full(text)
                if full != ids:
                    raise AssertionError("incremental tokenisation differs from a full encode")
            self._lru[text] = (ids, ends)
            self._lru.move_to_end(text)
            while len(self._lru) > self.capacity:
                self._lru.popitem(last=False)
            return list(ids)


def _common_prefix(a: str, b: str) -> int:
    n = min(len(a), len(b))
    if a[:n] == b[:n]:
        return n
    lo, hi = 0, n
    while lo < hi:  # binary search on the first differing position
        mid = (lo + hi + 1) // 2
        if a[:mid] == b[:mid]:
            lo = mid
        else:
            hi = mid - 1
    return lo


def _count_upto(ends: list[int], cut: int) -> int:
    import bisect

    return bisect.bisect_right(ends, cut)


class TextCodec:
    """The checkpoint's tokenizer and chat template behind a small interface."""

    def __init__(self, model_dir: str | os.PathLike) -> None:
        from transformers import AutoTokenizer

        self.tok = AutoTokenizer.from_pretrained(str(model_dir))
        self.vocab_size = len(self.tok)
        tid = self.tok.convert_tokens_to_ids("</think>")
        self.think_end_id = tid if isinstance(tid, int) and tid != self.tok.unk_token_id and tid >= 0 else None
        backend = getattr(self.tok, "backend_tokenizer", None)
        ok = False
        tj = Path(model_dir) / "tokenizer.json"
        if backend is not None and tj.exists():
            try:
                ok = safe_config(json.loads(tj.read_text()))
            except (OSError, json.JSONDecodeError):
                ok = False
        self.encoder = PromptEncoder(backend, enabled=ok and os.environ.get("ENGINE_REQ_FAST", "1") == "1")

    def encode(self, text: str) -> list[int]:
        if self.encoder.enabled:
            return self.encoder.encode(text)
        return list(self.tok.encode(text, add_special_tokens=False))

    def decode(self, ids: list[int], skip_special_tokens: bool = True) -> str:
        return self.tok.decode(ids, skip_special_tokens=skip_special_tokens)

    def render_chat(self, messages, tools=None, **kwargs: Any) -> str:
        """Chat template with thinking off unless the request turns it on (reference: generator.py:738-750)."""
        return self.tok.apply_chat_template(
            list(messages), tools=list(tools) if tools else None, add_generation_prompt=True, tokenize=False,
            **{"enable_thinking": False, **kwargs},
        )

    def encode_chat(self, messages, tools=None, **kwargs: Any) -> list[int]:
        return self.encode(self.render_chat(messages, tools, **kwargs))
