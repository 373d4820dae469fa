"""Host-side allocators: ref-counted KV pages and GDN state slots.

Both pools hand out small integers that index device tensors owned by the model
(``Model.kv[:, page]``, ``Model.conv_state[:, slot]`` / ``Model.rec_state[:, slot]``).
Index 0 of each pool is never handed out: it is the scratch target of padding rows
in fixed-size CUDA-graph buckets. When a pool runs dry it calls ``on_pressure`` (the
prefix cache's eviction hook) until enough entries are free or nothing is left to
evict (reference: ``PagePool`` with ``on_pressure``, ``engine/fast/model.py:121-148``).
"""

from __future__ import annotations

from typing import Callable


class OutOfCapacity(RuntimeError):
    """No free page / slot even after evicting every cache entry."""


class PagePool:
    def __init__(self, num_pages: int, on_pressure: Callable[[], bool] | None = None) -> None:
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, 0, -1))  # pop() hands out low ids first
        self._ref = [0] * num_pages
        self.on_pressure = on_pressure

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def used(self) -> int:
        return self.num_pages - 1 - len(self._free)

    def alloc(self, n: int) -> list[int]:
        while len(self._free) < n:
            if self.on_pressure is None or not self.on_pressure():
                raise OutOfCapacity(f"need {n} KV pages, {len(self._free)} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._ref[p] = 1
        return out

    def incref(self, pages: list[int]) -> None:
        for p in pages:
            assert self._ref[p] > 0, p
            self._ref[p] += 1

    def release(self, pages: list[int]) -> None:
        for p in pages:
            assert self._ref[p] > 0, p
            self._ref[p] -= 1
            if self._ref[p] == 0:
                self._free.append(p)

    def refcount(self, page: int) -> int:
        return self._ref[page]


class SlotPool:
    def __init__(self, num_slots: int, on_pressure: Callable[[], bool] | None = None) -> None:
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, 0, -1))
        self.on_pressure = on_pressure

    @property
    def free(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        while not self._free:
            if self.on_pressure is None or not self.on_pressure():
                raise OutOfCapacity("all sequence slots are busy")
        return self._free.pop()

    def release(self, slot: int) -> None:
        assert slot > 0 and slot not in self._free
        self._free.append(slot)
