"""CUDA-graph runners for the decode step.

One graph per batch bucket: fixed-shape device buffers (tokens, positions, slots, page
tables) are refreshed from pinned host memory with one copy each, the graph replays the
whole layer stack plus the fused LM-head argmax, and the picks come back with one
device-to-host copy. Rows beyond the live batch point at scratch slot 0 / page 0
(reference: per-bucket decode graphs, ``engine/fast/model.py:2009-2120``).
"""

from __future__ import annotations

import torch

from ..config import PAGE_SIZE
from ..models.qwen36 import PackedBatch


class _Bucket:
    def __init__(self, engine, size: int, width: int) -> None:
        dev = engine.device
        self.size, self.width = size, width
        self.tokens = torch.zeros(size, dtype=torch.int64, device=dev)
        self.positions = torch.zeros(size, dtype=torch.int64, device=dev)
        self.slots = torch.zeros(size, dtype=torch.int32, device=dev)
        self.tables = torch.zeros(size, width, dtype=torch.int32, device=dev)
        self.seq = torch.arange(size, dtype=torch.int32, device=dev)
        self.h_tokens = torch.zeros(size, dtype=torch.int64).pin_memory()
        self.h_positions = torch.zeros(size, dtype=torch.int64).pin_memory()
        self.h_slots = torch.zeros(size, dtype=torch.int32).pin_memory()
        self.h_tables = torch.zeros(size, width, dtype=torch.int32).pin_memory()
        self.h_picks = torch.zeros(size, dtype=torch.int64).pin_memory()
        self.batch = PackedBatch(self.tokens, self.positions, self.seq, self.slots, self.tables, 1)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.hidden = None
        self.picks = None

    def capture(self, engine) -> None:
        model = engine.model

        def body():
            h = model.forward(self.batch)
            return h, model.greedy(h)

        s = torch.cuda.Stream(device=engine.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            body()
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.hidden, self.picks = body()
        self.graph = g


class DecodeGraphs:
    def __init__(self, engine) -> None:
        self.engine = engine
        self.sizes = sorted(b for b in engine.cfg.decode_buckets if b <= max(engine.cfg.max_seqs, 1)) or [engine.cfg.max_seqs]
        if self.sizes[-1] < engine.cfg.max_seqs:
            self.sizes.append(engine.cfg.max_seqs)
        # page-table widths of the graphs (context classes of 4k / 32k / 256k tokens): the decode attention
        # launches one CTA per 8 pages of table width, so short contexts should not pay for long tables
        cap = engine.max_pages_per_seq
        self.widths = sorted({min(w, cap) for w in (64, 512, 4096)} | ({cap} if cap <= 4096 else set()))
        self.width = self.widths[-1]
        self.buckets: dict = {}
        self.errors: dict = {}

    def usable(self, gens) -> bool:
        if len(gens) > self.sizes[-1]:
            return False
        return all(len(g.pages) <= self.width for g in gens)

    def _bucket(self, n: int, pages: int = 0) -> _Bucket | None:
        size = next(s for s in self.sizes if s >= n)
        width = next(w for w in self.widths if w >= pages)
        key = (size, width)
        b = self.buckets.get(key)
        if b is None and key not in self.errors:
            b = _Bucket(self.engine, size, width)
            try:
                b.capture(self.engine)
            except Exception as e:  # capture failure: remember it, run eagerly (reference: model.py:2009-2029)
                self.errors[key] = repr(e)
                return None
            self.buckets[key] = b
        return b

    def warm(self) -> None:
        for s in self.sizes:
            self._bucket(s)

    def run(self, gens, tokens, positions):
        n = len(gens)
        b = self._bucket(n, max(len(g.pages) for g in gens))
        if b is None:
            eng = self.engine
            batch = PackedBatch.uniform(tokens, positions, [g.slot for g in gens], eng._table(gens), 1, eng.device)
            return eng.model.forward(batch), None
        b.h_tokens.zero_(); b.h_positions.zero_(); b.h_slots.zero_(); b.h_tables.zero_()
        b.h_tokens[:n] = torch.tensor(tokens, dtype=torch.int64)
        b.h_positions[:n] = torch.tensor(positions, dtype=torch.int64)
        b.h_slots[:n] = torch.tensor([g.slot for g in gens], dtype=torch.int32)
        for i, g in enumerate(gens):
            b.h_tables[i, : len(g.pages)] = torch.tensor(g.pages, dtype=torch.int32)
        b.tokens.copy_(b.h_tokens, non_blocking=True)
        b.positions.copy_(b.h_positions, non_blocking=True)
        b.slots.copy_(b.h_slots, non_blocking=True)
        b.tables.copy_(b.h_tables, non_blocking=True)
        b.graph.replay()
        b.h_picks.copy_(b.picks, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return b.hidden[:n], b.h_picks[:n]
