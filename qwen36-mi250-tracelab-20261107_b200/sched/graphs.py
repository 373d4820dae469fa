"""CUDA-graph runners for the decode step.

One graph per batch bucket: fixed-shape device buffers (tokens, positions, slots, page
tables) are refreshed from pinned host memory with one copy each, the graph replays the
whole layer stack plus the fused LM-head argmax, and the picks come back with one
device-to-host copy. Rows beyond the live batch point at scratch slot 0 / page 0
(reference: per-bucket decode graphs, ``engine/fast/model.py:2009-2120``).
"""

from __future__ import annotations

import torch

from ..models.qwen36 import PackedBatch
from ..obs import looptimers


class _Bucket:
    """Fixed-shape inputs of one graph. Tokens, positions, slots and page tables live in ONE device buffer mirrored
    by ONE pinned host buffer, so a step costs a single host-to-device copy; the host side is written through
    numpy views, and a page-table row is rewritten only when its request or its page count changed."""

    def __init__(self, engine, size: int, width: int) -> None:
        dev = engine.device
        self.size, self.width = size, width
        n_tok, n_pos, n_slot, n_tab = size * 8, size * 8, size * 4, size * width * 4
        offs = [0, n_tok, n_tok + n_pos, n_tok + n_pos + ((n_slot + 15) // 16) * 16]
        total = offs[3] + n_tab
        self.tab_off = offs[3]
        self.dev_buf = torch.zeros(total, dtype=torch.uint8, device=dev)
        self.host_buf = torch.zeros(total, dtype=torch.uint8)
        if dev.type == "cuda":
            self.host_buf = self.host_buf.pin_memory()

        def views(buf):
            return (buf[offs[0] : offs[0] + n_tok].view(torch.int64), buf[offs[1] : offs[1] + n_pos].view(torch.int64),
                    buf[offs[2] : offs[2] + n_slot].view(torch.int32), buf[offs[3] : offs[3] + n_tab].view(torch.int32).view(size, width))

        self.tokens, self.positions, self.slots, self.tables = views(self.dev_buf)
        h = views(self.host_buf)
        self.np_tokens, self.np_positions, self.np_slots, self.np_tables = (t.numpy() for t in h)
        self.seq = torch.arange(size, dtype=torch.int32, device=dev)
        # results come back into one of two pinned buffers: a step launched ahead must not overwrite what the host
        # has not read yet
        self.h_picks2 = [torch.zeros(size, dtype=torch.int64) for _ in range(2)]
        self.h_err2 = [torch.zeros(1, dtype=torch.int32) for _ in range(2)]
        if dev.type == "cuda":
            self.h_picks2 = [t.pin_memory() for t in self.h_picks2]
            self.h_err2 = [t.pin_memory() for t in self.h_err2]
        self.h_picks, self.h_err = self.h_picks2[0], self.h_err2[0]
        self.parity = 0
        self.rows: list = [None] * size  # (request id, page count, last page) whose table each row currently holds
        self.live = 0
        self.batch = PackedBatch(self.tokens, self.positions, self.seq, self.slots, self.tables, 1)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.hidden = None
        self.picks = None

    def fill(self, gens, tokens, positions) -> None:
        n = len(gens)
        self.np_tokens[:n] = tokens
        self.np_positions[:n] = positions
        self.np_slots[:n] = [g.slot for g in gens]
        if n < self.live:  # rows that fell out of the batch go back to the scratch slot and page
            self.np_tokens[n : self.live] = 0
            self.np_positions[n : self.live] = 0
            self.np_slots[n : self.live] = 0
            self.np_tables[n : self.live] = 0
            for i in range(n, self.live):
                self.rows[i] = None
        self.live = n
        rows, tab = self.rows, self.np_tables
        for i, g in enumerate(gens):
            sig = (g.id, len(g.pages), g.pages[-1] if g.pages else 0)
            if rows[i] != sig:
                rows[i] = sig
                k = len(g.pages)
                tab[i, :k] = g.pages
                tab[i, k:] = 0
        self.dev_buf.copy_(self.host_buf, non_blocking=True)

    def refresh_tables(self, gens) -> None:
        """Before a step whose tokens and positions are built on the device: only page-table rows that grew are sent."""
        changed = False
        rows, tab = self.rows, self.np_tables
        for i, g in enumerate(gens):
            sig = (g.id, len(g.pages), g.pages[-1] if g.pages else 0)
            if rows[i] != sig:
                rows[i] = sig
                k = len(g.pages)
                tab[i, :k] = g.pages
                tab[i, k:] = 0
                changed = True
        if changed:
            self.dev_buf[self.tab_off :].copy_(self.host_buf[self.tab_off :], non_blocking=True)

    def replay(self) -> None:
        if self.graph is not None:
            self.graph.replay()
        else:  # no CUDA device: the same body, run kernel by kernel into the same static buffers
            h, p = self._body()
            self.hidden.copy_(h)
            self.picks.copy_(p)

    def capture(self, engine) -> None:
        model = engine.model

        def body():
            h = model.forward(self.batch)
            return h, model.greedy(h)

        self._body = body
        if engine.device.type != "cuda":
            self.hidden, self.picks = body()
            self.hidden, self.picks = self.hidden.clone(), self.picks.clone()
            self.launches = 0
            return
        s = torch.cuda.Stream(device=engine.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            body()
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        count = getattr(engine.ops, "launch_count", None)
        n0 = count() if count else 0
        with torch.cuda.graph(g):
            self.hidden, self.picks = body()
        self.launches = (count() - n0) if count else 0  # kernels of this library in one replay
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
        # Replicas that share expert-parallel MoE blocks must launch the same passes: capturing a graph runs the pass
        # once for real, so every shape is captured at start-up (``warm``), on all replicas in the same order, and
        # never later; a shape without a graph runs kernel by kernel.
        self.frozen = False

    def usable(self, gens) -> bool:
        if len(gens) > self.sizes[-1]:
            return False
        return all(len(g.pages) <= self.width for g in gens)

    def _bucket(self, n: int, pages: int = 0) -> _Bucket | None:
        size = next(s for s in self.sizes if s >= n)
        width = next(w for w in self.widths if w >= pages)
        key = (size, width)
        b = self.buckets.get(key)
        if b is None and key not in self.errors and not self.frozen:
            b = _Bucket(self.engine, size, width)
            try:
                b.capture(self.engine)
            except Exception as e:  # capture failure: remember it, run eagerly (reference: model.py:2009-2029)
                self.errors[key] = repr(e)
                return None
            self.buckets[key] = b
        return b

    def warm(self) -> None:
        every_width = self.engine.tick is not None
        for w in (self.widths if every_width else self.widths[:1]):
            for s in self.sizes:
                if every_width:
                    self.engine.tick.rendezvous(self.engine)  # replicas capture in step: their eager runs pair up
                self._bucket(s, w)
        self.frozen = every_width

    def run(self, gens, tokens, positions):
        """One decode step from host inputs, launched and collected."""
        h = self.launch(gens, tokens, positions)
        if h is None:
            eng = self.engine
            batch = PackedBatch.uniform(tokens, positions, [g.slot for g in gens], eng._table(gens), 1, eng.device)
            hidden = eng.model.forward(batch)
            eng.check_device()
            return hidden, None
        return self.collect(h)

    # A step in flight: launched, results not read yet. ``launch_next`` starts the step after it from inputs built on
    # the device (tokens = this step's picks, positions + 1) before the host has read this step's result, so the
    # GPU never waits for the host's bookkeeping (reference: run-ahead, engine/speculative.py:266-274, 427-451;
    # input builder engine/fast/tp.py:296-318).
    def launch(self, gens, tokens, positions):
        n = len(gens)
        b = self._bucket(n, max(len(g.pages) for g in gens))
        if b is None:
            return None
        with looptimers.stage("build"):
            b.fill(gens, tokens, positions)
        return self._start(b, gens)

    def launch_next(self, handle):
        b, gens = handle["bucket"], handle["gens"]
        b.refresh_tables(gens)
        n = len(gens)
        b.tokens[:n].copy_(b.picks[:n])  # stream-ordered after the step that produced the picks
        b.positions[:n].add_(1)
        return self._start(b, gens)

    def _start(self, b, gens):
        start, stop = looptimers.gpu_span("gpu_graph")
        start()
        b.replay()
        stop()
        self.engine.flush_events()  # the previous step's tokens go out while the GPU runs this one
        par = b.parity
        b.parity ^= 1
        b.h_picks2[par].copy_(b.picks, non_blocking=True)
        err = getattr(self.engine.ops, "err_word", None)
        if err is not None:  # the device error word travels with the picks: one more 4-byte copy, no extra sync
            b.h_err2[par].copy_(err(self.engine.device), non_blocking=True)
        ev = None
        if self.engine.device.type == "cuda":
            ev = torch.cuda.Event()
            ev.record()
        return {"bucket": b, "gens": list(gens), "parity": par, "event": ev, "err": err is not None}

    def collect(self, handle):
        b, n, par = handle["bucket"], len(handle["gens"]), handle["parity"]
        with looptimers.stage("wait"):
            if handle["event"] is not None:
                handle["event"].synchronize()
        if handle["err"]:
            self.engine.check_device(int(b.h_err2[par][0]))
        return b.hidden[:n], b.h_picks2[par][:n]


class _VerifyBucket:
    """One captured speculative step: verify pass over ``G = k + 1`` rows per sequence, greedy picks, the accepted
    prefix length of every sequence, the MTP block over all rows and the ``kmax`` draft links that start at each
    sequence's last accepted row, all on the device; the host reads one ``[picks | accepted | drafts]`` vector back
    (the reference captures verify + accept + draft chain the same way and reads one packed row,
    ``engine/fast/kernels.py:544-571``, ``engine/fast/model.py:2009-2120``)."""

    def __init__(self, engine, size: int, width: int, k: int, kmax: int, ring) -> None:
        dev = engine.device
        G = k + 1
        self.size, self.width, self.k, self.G, self.kmax = size, width, k, G, kmax
        n_tok, n_slot, n_tab = size * G * 8, size * 4, size * width * 4
        offs = [0, n_tok, 2 * n_tok, 2 * n_tok + ((n_slot + 15) // 16) * 16, 2 * n_tok + 2 * (((n_slot + 15) // 16) * 16)]
        total = offs[4] + n_tab
        self.dev_buf = torch.zeros(total, dtype=torch.uint8, device=dev)
        self.host_buf = torch.zeros(total, dtype=torch.uint8).pin_memory()

        def views(buf):
            return (buf[offs[0] : offs[0] + n_tok].view(torch.int64), buf[offs[1] : offs[1] + n_tok].view(torch.int64),
                    buf[offs[2] : offs[2] + n_slot].view(torch.int32), buf[offs[3] : offs[3] + n_slot].view(torch.int32),
                    buf[offs[4] : offs[4] + n_tab].view(torch.int32).view(size, width))

        self.tokens, self.positions, self.slots, self.n_valid, self.tables = views(self.dev_buf)
        self.np_tokens, self.np_positions, self.np_slots, self.np_valid, self.np_tables = (t.numpy() for t in views(self.host_buf))
        self.seq = torch.repeat_interleave(torch.arange(size, dtype=torch.int32, device=dev), G)
        self.seq1 = torch.arange(size, dtype=torch.int32, device=dev)
        self.batch = PackedBatch(self.tokens, self.positions, self.seq, self.slots, self.tables, G)
        self.ring = ring
        self.h_out = torch.zeros(size * G + size + size * kmax, dtype=torch.int64).pin_memory()
        self.h_err = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.rows: list = [None] * size
        self.live = 0
        self.graph: torch.cuda.CUDAGraph | None = None
        self.out = None

    def _body(self, model):
        """Verify pass, greedy picks, chain acceptance, MTP block and draft chain; returns the int64 vector
        ``[picks (size * G) | accepted (size) | drafts (kmax links x size)]`` the host reads back. The acceptance
        arithmetic and the gathers around it are one kernel (``chain_accept``), and every argmax writes its picks
        straight into the result vector."""
        size, G, kmax = self.size, self.G, self.kmax
        dev = self.tokens.device
        ops = model.ops
        out = torch.empty(size * G + size + size * kmax, dtype=torch.int64, device=dev)
        picks, acc_out = out[: size * G], out[size * G : size * G + size]
        dr0 = size * G + size
        hidden = model.forward(self.batch, ring=self.ring)
        model.greedy(hidden, out=picks)
        y = model.mtp_forward(hidden, picks, self.batch)
        _acc, h, link_pos = ops.chain_accept(self.tokens, picks, self.n_valid, self.positions, y, G, kmax - 1, acc_out=acc_out)
        d = model.draft_pick(h, out=out[dr0 : dr0 + size])
        for j in range(1, kmax):
            link = PackedBatch(d, link_pos[j - 1], self.seq1, self.slots, self.tables, 1)
            h = model.mtp_forward(h, d, link)
            d = model.draft_pick(h, out=out[dr0 + j * size : dr0 + (j + 1) * size])
        return out

    def capture(self, engine, pool) -> None:
        s = torch.cuda.Stream(device=engine.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._body(engine.model)
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, pool=pool):
            self.out = self._body(engine.model)
        self.graph = g

    def fill(self, gens, tokens, positions, n_valid) -> None:
        n, G = len(gens), self.G
        self.np_tokens[: n * G] = tokens
        self.np_positions[: n * G] = positions
        self.np_slots[:n] = [g.slot for g in gens]
        self.np_valid[:n] = n_valid
        if n < self.live:
            self.np_tokens[n * G : self.live * G] = 0
            self.np_positions[n * G : self.live * G] = 0
            self.np_slots[n : self.live] = 0
            self.np_valid[n : self.live] = 0
            self.np_tables[n : self.live] = 0
            for i in range(n, self.live):
                self.rows[i] = None
        self.live = n
        rows, tab = self.rows, self.np_tables
        for i, g in enumerate(gens):
            sig = (g.id, len(g.pages), g.pages[-1] if g.pages else 0)
            if rows[i] != sig:
                rows[i] = sig
                m = len(g.pages)
                tab[i, :m] = g.pages
                tab[i, m:] = 0
        self.dev_buf.copy_(self.host_buf, non_blocking=True)


class VerifyGraphs:
    """Captured speculative steps per (batch bucket, context class, draft depth); shares the decode graphs' buckets'
    sizes and memory pool. ``run`` returns None when a capture failed (the caller runs the step eagerly)."""

    def __init__(self, engine, decode: DecodeGraphs, kmax: int, ring_of) -> None:
        self.engine, self.decode, self.kmax, self.ring_of = engine, decode, kmax, ring_of
        self.pool = torch.cuda.graph_pool_handle()
        self.buckets: dict = {}
        self.errors: dict = {}
        # Replicas that share expert-parallel MoE blocks must launch the same passes: capturing a graph runs the pass
        # once for real, so every shape is captured at start-up (``warm``), on all replicas in the same order, and
        # never later; a shape without a graph runs kernel by kernel.
        self.frozen = False

    def usable(self, gens) -> bool:
        return self.decode.usable(gens)

    def _bucket(self, n: int, pages: int, k: int):
        size = next(s for s in self.decode.sizes if s >= n)
        width = next(w for w in self.decode.widths if w >= pages)
        key = (size, width, k)
        b = self.buckets.get(key)
        if b is None and key not in self.errors:
            try:
                b = _VerifyBucket(self.engine, size, width, k, self.kmax, self.ring_of(size, k + 1))
                b.capture(self.engine, self.pool)
            except Exception as e:  # noqa: BLE001 - remember the failure, run eagerly
                self.errors[key] = repr(e)
                return None
            self.buckets[key] = b
        return b

    def run(self, gens, tokens, positions, n_valid, k: int):
        n = len(gens)
        b = self._bucket(n, max(len(g.pages) for g in gens), k)
        if b is None:
            return None
        b.fill(gens, tokens, positions, n_valid)
        b.graph.replay()
        self.engine.flush_events()
        b.h_out.copy_(b.out, non_blocking=True)
        b.h_err.copy_(self.engine.ops.err_word(self.engine.device), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.engine.check_device(int(b.h_err[0]))
        G, size = b.G, b.size
        out = b.h_out
        picks = out[: size * G].view(size, G)[:n].tolist()
        acc = out[size * G : size * G + size][:n].tolist()
        drafts = out[size * G + size :].view(self.kmax, size)[:, :n].t().tolist()
        return picks, acc, drafts, b.ring, b.slots[:n]


# --------------------------------------------------------------------------- captured prefill passes
GDN_CHUNK_ROWS = 64  # rows per chunk of the gated-delta-rule prefill kernels


def prefill_layout(n: int, rows: int) -> list[int]:
    """Span starts ``[0, n, n + a, rows]`` of a padded prefill pass: the real span of ``n`` tokens, then two filler
    spans (scratch slot, scratch page) of ``a`` and ``rows - n - a`` rows. ``a`` completes the real span's last
    64-row chunk (32 when there is nothing to complete), so the three spans always split into ``rows / 64 + 1``
    chunks: the chunk count, like every other launch parameter of the pass, does not depend on ``n``."""
    if rows % GDN_CHUNK_ROWS or not 1 <= n <= rows - GDN_CHUNK_ROWS:
        raise ValueError(f"a padded pass of {rows} rows takes 1..{rows - GDN_CHUNK_ROWS} tokens, not {n}")
    r = n % GDN_CHUNK_ROWS
    a = GDN_CHUNK_ROWS - r if r else GDN_CHUNK_ROWS // 2
    return [0, n, n + a, rows]


def span_chunks(starts: list[int]) -> tuple[list[tuple[int, int, int, int]], list[tuple[int, int]]]:
    """``(span, first row, rows, is the span's first chunk)`` per 64-row chunk, span by span, and ``(first chunk,
    chunk count)`` per span: the tables of the gated-delta-rule prefill kernels."""
    chunks, per_span = [], []
    for i in range(len(starts) - 1):
        a, b = starts[i], starts[i + 1]
        first = len(chunks)
        for r0 in range(a, b, GDN_CHUNK_ROWS):
            chunks.append((i, r0, min(GDN_CHUNK_ROWS, b - r0), int(r0 == a)))
        per_span.append((first, len(chunks) - first))
    return chunks, per_span


def span_tiles(starts: list[int], r_tile: int, n_tiles: int) -> list[tuple[int, int, int, int]]:
    """``(span, offset in the span, the span's first row, the span's rows)`` per query tile of the flash kernel,
    filled up to ``n_tiles`` entries with fillers of a zero-row span, which their CTAs skip."""
    tiles = []
    for i in range(len(starts) - 1):
        n = starts[i + 1] - starts[i]
        tiles.extend((i, p0, starts[i], n) for p0 in range(0, n, r_tile))
    if len(tiles) > n_tiles:
        raise ValueError("more query tiles than the table holds")
    return tiles + [(0, 0, 0, 0)] * (n_tiles - len(tiles))


class PrefillTables:
    """Span tables of a ragged prefill pass as fixed-shape device tensors that the owner rewrites before each run
    (what ``cuda_ops.gdn_prefill`` / ``flash_prefill`` otherwise build from host lists, pass by pass)."""

    __slots__ = ("gdn", "flash")

    def __init__(self, gdn, flash) -> None:
        self.gdn, self.flash = gdn, flash


class _PrefillBucket:
    """One captured prefill pass of ``rows`` packed rows: ONE request's span of up to ``rows - 64`` tokens plus filler
    rows that run on the scratch slot and the scratch page (``prefill_layout``). Tokens, positions, the MTP block's
    shifted tokens, the span tables and the page table live in one device buffer mirrored by one pinned host
    buffer: a pass costs one host-to-device copy and one graph replay instead of some twenty launches per layer
    (reference: prefill graphs per padded size with device-side counts, ``engine/fast/tp.py:1088-1200``)."""

    N_SPANS = 3

    def __init__(self, engine, rows: int, width: int, r_tile: int) -> None:
        dev = engine.device
        self.rows, self.width, self.r_tile = rows, width, r_tile
        self.cap = rows - GDN_CHUNK_ROWS
        self.n_chunks = rows // GDN_CHUNK_ROWS + 1
        self.n_tiles = rows // r_tile + self.N_SPANS
        sizes = [("tokens", rows * 8), ("positions", rows * 8), ("nxt", rows * 8), ("seq", rows * 4),
                 ("chunks", self.n_chunks * 16), ("per_span", self.N_SPANS * 8), ("starts", (self.N_SPANS + 1) * 4),
                 ("slots", self.N_SPANS * 4), ("tiles", self.n_tiles * 16), ("pos0", self.N_SPANS * 4),
                 ("tables", self.N_SPANS * width * 4)]
        offs, o = {}, 0
        for name, nbytes in sizes:  # every table starts on a 16-byte boundary (the kernels read some as int4)
            offs[name] = (o, nbytes)
            o += (nbytes + 15) // 16 * 16
        self.dev_buf = torch.zeros(o, dtype=torch.uint8, device=dev)
        self.host_buf = torch.zeros(o, dtype=torch.uint8)
        if dev.type == "cuda":
            self.host_buf = self.host_buf.pin_memory()

        def views(buf):
            v = {}
            for name, (a, nbytes) in offs.items():
                dt = torch.int64 if name in ("tokens", "positions", "nxt") else torch.int32
                v[name] = buf[a : a + nbytes].view(dt)
            v["tables"] = v["tables"].view(self.N_SPANS, width)
            return v

        d = views(self.dev_buf)
        self.np = {k: t.numpy() for k, t in views(self.host_buf).items()}
        self.tokens, self.positions, self.nxt = d["tokens"], d["positions"], d["nxt"]
        meta = None
        if dev.type == "cuda":
            meta = PrefillTables(
                (self.N_SPANS, self.n_chunks, d["chunks"], d["per_span"], d["seq"], d["starts"], d["slots"]),
                (r_tile, self.n_tiles, d["tiles"].view(-1, 4), d["pos0"]),
            )
        self.batch = PackedBatch(self.tokens, self.positions, d["seq"], d["slots"], d["tables"], 0,
                                 [0, 0, 0, 0], [0, 0, 0], [0, 0, 0], meta)
        self.with_mtp = engine.spec is not None
        self.graph: torch.cuda.CUDAGraph | None = None
        self.hidden = None
        self.launches = 0

    def fill(self, tokens, nxt, pos0: int, slot: int, pages) -> None:
        """Write one request's span (``tokens`` at positions ``pos0...``, state slot, page list) and its filler rows."""
        import numpy as np

        n, rows, v = len(tokens), self.rows, self.np
        starts = prefill_layout(n, rows)
        v["tokens"][:n] = tokens
        v["tokens"][n:] = 0
        v["nxt"][:n] = nxt
        v["nxt"][n:] = 0
        v["positions"][:n] = np.arange(pos0, pos0 + n)
        for i in (1, 2):  # filler spans start at position 0 of the scratch page
            v["positions"][starts[i] : starts[i + 1]] = np.arange(starts[i + 1] - starts[i])
            v["seq"][starts[i] : starts[i + 1]] = i
        v["seq"][:n] = 0
        chunks, per_span = span_chunks(starts)
        assert len(chunks) == self.n_chunks
        v["chunks"][:] = np.asarray(chunks, dtype=np.int32).reshape(-1)
        v["per_span"][:] = np.asarray(per_span, dtype=np.int32).reshape(-1)
        v["starts"][:] = starts
        v["slots"][:] = (slot, 0, 0)
        v["tiles"][:] = np.asarray(span_tiles(starts, self.r_tile, self.n_tiles), dtype=np.int32).reshape(-1)
        v["pos0"][:] = (pos0, 0, 0)
        k = len(pages)
        v["tables"][0, :k] = pages
        v["tables"][0, k:] = 0
        # the kernel-by-kernel form of the same pass (no CUDA device) reads the spans from these host lists
        self.batch.seg_starts, self.batch.seg_slots, self.batch.seg_pos0 = starts, [slot, 0, 0], [pos0, 0, 0]
        self.dev_buf.copy_(self.host_buf, non_blocking=True)

    def _body(self, model):
        h = model.forward(self.batch)
        if self.with_mtp:  # the MTP block sees the prompt rows too: (token t + 1, hidden t) fills its own KV pages
            model.mtp_forward(h, self.nxt, self.batch)
        return h

    def capture(self, engine) -> None:
        """Capture with every row on the scratch slot and page, so that the two runs a capture needs touch no request."""
        n = min(self.cap, GDN_CHUNK_ROWS)
        self.fill([0] * n, [0] * n, 0, 0, [])
        model = engine.model
        if engine.device.type != "cuda":
            return
        s = torch.cuda.Stream(device=engine.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._body(model)
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        count = getattr(engine.ops, "launch_count", None)
        n0 = count() if count else 0
        with torch.cuda.graph(g):
            self.hidden = self._body(model)
        self.launches = (count() - n0) if count else 0
        self.graph = g

    def replay(self, model) -> torch.Tensor:
        if self.graph is not None:
            self.graph.replay()
            return self.hidden
        return self._body(model)


class PrefillGraphs:
    """Captured prefill passes for short spans (a session's next turn on top of its cached context, a short prompt):
    such a pass is bound by its launches, not by its arithmetic. One graph per padded row count; a pass that packs
    several requests, or a span longer than the largest graph, runs kernel by kernel as before."""

    def __init__(self, engine) -> None:
        self.engine = engine
        cfg = engine.mcfg
        group = cfg.num_attention_heads // max(cfg.num_key_value_heads, 1)
        self.r_tile = 128 // group if group in (1, 2, 4, 8) else 16
        limit = min(engine.chunk, engine.cfg.prefill_pack_tokens)
        rows = sorted(int(r) for r in engine.cfg.prefill_graph_rows)
        if any(r % GDN_CHUNK_ROWS or r < 2 * GDN_CHUNK_ROWS for r in rows):
            raise ValueError("prefill graph sizes are multiples of 64 rows, 128 at least")
        # sizes beyond the first one that holds a whole chunk are never picked
        self.sizes = [r for i, r in enumerate(rows) if i == 0 or rows[i - 1] - GDN_CHUNK_ROWS < limit]
        # the filler spans count their positions from 0 on the scratch page: the table has to be that wide at least
        self.width = max(engine.max_pages_per_seq, self.sizes[-1] // GDN_CHUNK_ROWS)
        self.buckets: dict = {}
        self.errors: dict = {}

    @staticmethod
    def supported(engine) -> bool:
        """Single-process engines whose spans take the native kernels on a GPU (their calls read device tables only)
        or the PyTorch forms on the CPU (tests of the padding logic)."""
        if engine.multi_rank or engine.tick is not None:
            return False
        if engine.device.type != "cuda":
            return bool(engine.cfg.graphs_on_cpu)
        c = engine.mcfg
        group = c.num_attention_heads // max(c.num_key_value_heads, 1)
        attn = c.head_dim in (64, 128, 256) and group in (1, 2, 4, 8) and c.num_attention_heads % c.num_key_value_heads == 0
        dk, dv = c.linear_key_head_dim, c.linear_value_head_dim
        gdn = dk == dv and dk in (32, 64, 128) and c.linear_conv_kernel_dim == 4 and (c.linear_num_key_heads * dk) % 4 == 0
        return attn and gdn

    def _bucket(self, n: int) -> _PrefillBucket | None:
        rows = next((r for r in self.sizes if r - GDN_CHUNK_ROWS >= n), None)
        if rows is None:
            return None
        b = self.buckets.get(rows)
        if b is None and rows not in self.errors:
            try:
                b = _PrefillBucket(self.engine, rows, self.width, self.r_tile)
                b.capture(self.engine)
            except Exception as e:  # noqa: BLE001 - remember the failure; such spans run kernel by kernel
                self.errors[rows] = repr(e)
                return None
            self.buckets[rows] = b
        return b

    def warm(self) -> None:
        for r in self.sizes:
            self._bucket(r - GDN_CHUNK_ROWS)

    def pick(self, gens, spans) -> _PrefillBucket | None:
        """The graph for this pass, or None when it has to run kernel by kernel."""
        if len(gens) != 1:
            return None
        g, (a, b) = gens[0], spans[0]
        if len(g.pages) > self.width:
            return None
        if self.engine.spec is not None and b == len(g.prompt) and g.next_token is not None:
            return None  # a resumed request drafts from its last prompt row right away: the general path does that
        return self._bucket(b - a)

    def run(self, bucket: _PrefillBucket, gen, a: int, b: int):
        """Run ``gen``'s span ``[a, b)``; returns ``(hidden [rows, H], batch)`` with the span in rows ``0 .. b - a``."""
        toks = gen.prompt[a:b]
        nxt = gen.prompt[a + 1 : b + 1]
        if len(nxt) < len(toks):
            nxt = nxt + [0]  # the last prompt row's partner is the first sampled token: its row is redone at decode
        bucket.fill(toks, nxt, a, gen.slot, gen.pages)
        start, stop = looptimers.gpu_span("gpu_prefill_graph")
        start()
        hidden = bucket.replay(self.engine.model)
        stop()
        return hidden, bucket.batch
