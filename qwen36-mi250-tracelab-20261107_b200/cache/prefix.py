"""Block-granular prefix cache with session tails.

Two kinds of entry, both keyed by a token prefix and both referring to device state
without copying KV:

* **snapshot** — taken at a chunk boundary (a multiple of the 64-token page) while a
  prompt is prefilled. It shares the sequence's full KV pages by reference count and owns
  one state slot holding a *copy* of the GDN state at that boundary. Any later prompt that
  starts with the same tokens resumes there; because page, GDN-chunk and prefill-chunk
  boundaries coincide, the resumed computation is the one a cold run would do, so cached
  and cold outputs are identical.
* **tail** — left behind by a finished request: key = prompt + all generated tokens but
  the last, at any length. The request's pages and state slot simply stay with the entry
  ("parking": nothing moves), and the next round of the session adopts them.

A GDN state cannot be rewound, so an entry is reusable only at exactly its own length
(reference rules: ``engine/generator.py:10-16, 134-233, 244-430``). Lookup walks the
prompt once, hashing 64-token blocks in a chain; eviction is LRU under entry, token and
byte budgets and is also driven by page / slot pressure.
"""

from __future__ import annotations

import hashlib
from array import array
from collections import OrderedDict
from dataclasses import dataclass

from ..config import PAGE_SIZE
from .pools import PagePool, SlotPool


def _block_hash(prev: bytes, tokens) -> bytes:
    return hashlib.blake2b(array("q", tokens).tobytes(), key=prev, digest_size=16).digest()


@dataclass
class Entry:
    kind: str  # "snapshot" | "tail"
    tokens: array  # the key (token ids)
    pages: list[int]
    slot: int
    key: tuple  # index key
    nbytes: int = 0
    hits: int = 0

    @property
    def length(self) -> int:
        return len(self.tokens)


@dataclass
class CacheStats:
    tail_hits: int = 0
    snapshot_hits: int = 0
    evictions: int = 0
    stored: int = 0


class PrefixCache:
    def __init__(
        self,
        pages: PagePool,
        slots: SlotPool,
        page_bytes: int,
        slot_bytes: int,
        max_entries: int = 128,
        max_tokens: int = 4194304,
        max_bytes: int = 16 << 30,
        block: int = PAGE_SIZE,
    ) -> None:
        self.pages, self.slots = pages, slots
        self.page_bytes, self.slot_bytes = page_bytes, slot_bytes
        self.max_entries, self.max_tokens, self.max_bytes = max_entries, max_tokens, max_bytes
        self.block = block
        self._lru: "OrderedDict[tuple, Entry]" = OrderedDict()
        self._tails_at: dict[tuple, list[Entry]] = {}  # (n_blocks, chain hash) -> tails starting in that block
        self.stats = CacheStats()
        self.tokens = 0
        self.bytes = 0

    # ------------------------------------------------------------------ keys
    def _chain(self, tokens, upto_blocks: int) -> list[bytes]:
        """Chain hashes after 0, 1, ..., ``upto_blocks`` full blocks."""
        out = [b"\0" * 16]
        if upto_blocks <= 0:
            return out
        # one conversion of the covered tokens to bytes, then a digest per block over slices of it (the per-block
        # list slice + array conversion was most of a lookup's time on long prompts)
        src = tokens if isinstance(tokens, array) and tokens.typecode == "q" else array("q", tokens[: upto_blocks * self.block])
        raw = memoryview(src).cast("B")
        step = self.block * 8
        for i in range(upto_blocks):
            out.append(hashlib.blake2b(raw[i * step : (i + 1) * step], key=out[-1], digest_size=16).digest())
        return out

    def __len__(self) -> int:
        return len(self._lru)

    # ------------------------------------------------------------------ store
    def _insert(self, e: Entry) -> None:
        old = self._lru.pop(e.key, None)
        if old is not None:
            self._drop(old)
        self._lru[e.key] = e
        if e.kind == "tail":
            self._tails_at.setdefault(e.key[:2], []).append(e)
        self.tokens += e.length
        self.bytes += e.nbytes
        self.stats.stored += 1
        self._enforce()

    def store_snapshot(self, tokens, length: int, pages: list[int], slot: int) -> bool:
        """Keep the state at ``length`` (a block multiple). ``pages`` are shared (ref count raised);
        ``slot`` must already hold a private copy of the GDN state and is owned by the cache."""
        assert length % self.block == 0 and length > 0
        nb = length // self.block
        chain = self._chain(tokens, nb)
        key = (nb, chain[nb], "s")
        if key in self._lru:
            self._lru.move_to_end(key)
            return False
        self.pages.incref(pages[:nb])
        e = Entry("snapshot", array("q", tokens[:length]), list(pages[:nb]), slot, key,
                  nbytes=self.slot_bytes)  # pages are shared: charge the state copy only
        self._insert(e)
        return True

    def has_snapshot(self, tokens, length: int) -> bool:
        nb = length // self.block
        return (nb, self._chain(tokens, nb)[nb], "s") in self._lru

    def store_tail(self, tokens, pages: list[int], slot: int) -> None:
        """Park a finished sequence: ``tokens`` are what its KV and state cover; ownership moves here."""
        n = len(tokens)
        nb = n // self.block
        chain = self._chain(tokens, nb)
        key = (nb, chain[nb], "t", bytes(array("q", tokens[nb * self.block :]).tobytes()))
        e = Entry("tail", array("q", tokens), list(pages), slot, key,
                  nbytes=self.slot_bytes + len(pages) * self.page_bytes)
        self._insert(e)

    # ------------------------------------------------------------------ lookup
    def lookup(self, prompt) -> Entry | None:
        """Longest entry that covers a proper prefix of ``prompt`` (at most ``len(prompt) - 1`` tokens,
        so that at least one row is left to produce logits). A tail is removed from the cache and
        handed to the caller; a snapshot stays and the caller copies its state."""
        limit = len(prompt) - 1
        if limit <= 0 or not self._lru:
            return None
        nb_max = limit // self.block
        chain = self._chain(prompt, nb_max)
        best: Entry | None = None
        for nb in range(nb_max, -1, -1):
            for e in self._tails_at.get((nb, chain[nb]), ()):
                n = e.length
                if n <= limit and (best is None or n > best.length) and list(prompt[nb * self.block : n]) == list(
                    e.tokens[nb * self.block :]
                ):
                    best = e
            if best is not None:
                break
            if nb > 0:
                s = self._lru.get((nb, chain[nb], "s"))
                if s is not None and list(s.tokens) == list(prompt[: s.length]):
                    best = s
                    break
        if best is None:
            return None
        best.hits += 1
        if best.kind == "tail":
            self.stats.tail_hits += 1
            self._unlink(best)
        else:
            self.stats.snapshot_hits += 1
            self._lru.move_to_end(best.key)
        return best

    # ------------------------------------------------------------------ eviction
    def _unlink(self, e: Entry) -> None:
        self._lru.pop(e.key, None)
        if e.kind == "tail":
            lst = self._tails_at.get(e.key[:2])
            if lst is not None:
                lst.remove(e)
                if not lst:
                    del self._tails_at[e.key[:2]]
        self.tokens -= e.length
        self.bytes -= e.nbytes

    def _drop(self, e: Entry) -> None:
        self._unlink(e)
        self.pages.release(e.pages)
        self.slots.release(e.slot)

    def evict_one(self) -> bool:
        if not self._lru:
            return False
        e = next(iter(self._lru.values()))
        self._drop(e)
        self.stats.evictions += 1
        return True

    def _enforce(self) -> None:
        while self._lru and (
            len(self._lru) > self.max_entries or self.tokens > self.max_tokens or self.bytes > self.max_bytes
        ):
            self.evict_one()

    def clear(self) -> None:
        while self.evict_one():
            pass
