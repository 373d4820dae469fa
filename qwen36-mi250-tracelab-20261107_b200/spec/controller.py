"""MTP speculative decoding: draft chain, multi-token verify, acceptance bookkeeping, depth policy.

Every decode step of an engine with an MTP head is a *verify step* of ``G = k + 1`` rows per
sequence: the last sampled token followed by ``k`` draft tokens. The base model scores all rows in
one pass (GDN states after every row are kept in a ring), row ``j``'s greedy pick verifies draft
``j + 1``; with ``a`` leading drafts accepted the step yields ``a + 1`` tokens. The MTP block then
runs on every row (keeping its own KV cache complete) and, starting from the last accepted row,
proposes the next chain: link 1 from ``(pick, base hidden)``, link ``j`` from ``(link j-1, its own
previous normed output)`` (reference: ``engine/speculative.py:108-117, 296-339, 391-464``;
``engine/fast/model.py:1768-1832``). ``k = 0`` is plain decode that still feeds the MTP cache.

Speculation never changes outputs: a draft only survives if it equals the base model's greedy
pick. Rows that sample (temperature > 0) or mask EOS (``min_tokens``) take no drafts.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from ..models.qwen36 import PackedBatch
from ..sched.sampling import pick_tokens

DECAY = 0.9


@dataclass
class DepthPolicy:
    """Chooses the draft depth from measured acceptance and a step-cost model.

    ``accept[j]`` is a decayed estimate of P(draft j+1 accepted | drafts 1..j accepted). The
    expected tokens of a depth-k step are ``1 + sum_j prod_{i<=j} accept[i]``; the cost is
    ``cost(B, k)`` in arbitrary units (a table measured on the target, or the default model of a
    fixed part plus a per-row part). Depth 0 is always available.
    """

    kmax: int = 3
    fixed: int = 0  # > 0: always this depth
    accept: list[float] = field(default_factory=lambda: [0.7, 0.6, 0.5, 0.45, 0.4, 0.35, 0.3])
    table: dict[tuple[int, int], float] = field(default_factory=dict)  # (batch bucket, k) -> ms
    row_cost: float = 0.04  # default model: relative cost of one more row per sequence
    max_rows: int = 256  # B * (k + 1) bound of one verify pass

    def cost(self, B: int, k: int) -> float:
        """Cost of a depth-``k`` step over ``B`` sequences. With a measured table: the entry of the smallest measured
        batch bucket that holds ``B`` (the largest one beyond it); a depth the bucket was not measured at lies on
        the line through its measured neighbours, or through the two deepest measured depths when it is deeper (a verify step grows by k + 1 rows per sequence and
        one more draft link per depth). Without a table: a fixed part plus a per-row part."""
        if self.table:
            buckets = sorted({b for (b, _k) in self.table})
            b = next((x for x in buckets if x >= B), buckets[-1])
            if (b, k) in self.table:
                return self.table[(b, k)]
            ks = sorted(kk for (bb, kk) in self.table if bb == b)
            if len(ks) >= 2:
                below = [kk for kk in ks if kk < k]
                above = [kk for kk in ks if kk > k]
                # between two measured depths: on the line through them; beyond the deepest: on the last two's line
                k1, k2 = (below[-1], above[0]) if below and above else (ks[-2], ks[-1]) if below else (ks[0], ks[1])
                slope = (self.table[(b, k2)] - self.table[(b, k1)]) / (k2 - k1)
                return self.table[(b, k1)] + slope * (k - k1)
            return math.inf
        return 1.0 + self.row_cost * k * max(1.0, math.log2(B + 1))

    def load_table(self, path) -> None:
        """Read a ``{"ms": {batch: {depth: ms}}}`` file as written next to this module (measured with
        ``bench/mtp_bench.py``; the reference keeps such a table per (slot bucket, k), engine/speculative.py:127-136)."""
        import json
        from pathlib import Path

        data = json.loads(Path(path).read_text())["ms"]
        self.table = {(int(b), int(k)): float(ms) for b, row in data.items() for k, ms in row.items()}

    def expected_tokens(self, k: int) -> float:
        e, p = 1.0, 1.0
        for j in range(k):
            p *= self.accept[min(j, len(self.accept) - 1)]
            e += p
        return e

    def choose(self, B: int, available: int) -> int:
        """Depth for a step over ``B`` sequences when every one of them holds ``available`` drafts."""
        cap = min(self.kmax, available, max(0, self.max_rows // max(B, 1) - 1))
        if self.fixed:
            return min(self.fixed, cap)
        best, best_rate = 0, self.expected_tokens(0) / self.cost(B, 0)
        for k in range(1, cap + 1):
            rate = self.expected_tokens(k) / self.cost(B, k)
            if rate > best_rate * 1.02:  # hysteresis: deeper only when clearly better
                best, best_rate = k, rate
        return best

    def observe(self, proposed: int, accepted: int) -> None:
        for j in range(proposed):
            hit = 1.0 if j < accepted else 0.0
            if j <= accepted:  # depth j was actually tested only if all shallower drafts passed
                i = min(j, len(self.accept) - 1)
                self.accept[i] = DECAY * self.accept[i] + (1 - DECAY) * hit


class SpecController:
    def __init__(self, engine) -> None:
        self.engine = engine
        c = engine.cfg
        self.policy = DepthPolicy(kmax=max(1, min(c.spec_kmax, 7)), fixed=c.spec_k)
        # the step-cost model: a measured table for this hardware when serving on a GPU (ENGINE_SPEC_COST names another
        # file, "model" selects the built-in formula); the formula on CPU
        import os
        from pathlib import Path

        src = os.environ.get("ENGINE_SPEC_COST", "")
        if src != "model" and (src or engine.device.type == "cuda"):
            self.policy.load_table(src or Path(__file__).with_name("cost_table_b200.json"))
        self.k_hist: dict[int, int] = {}
        self.draft_override = None  # tests: callable(gen, k) -> list[int] forcing the drafts of a step
        self._ring_store = None
        self._ring_cap = 0
        self._vgraphs = None

    # ------------------------------------------------------------------ helpers
    def eligible(self, g) -> bool:
        return g.sampling.greedy and len(g.output) >= g.sampling.min_tokens

    def _ring(self, B: int, G: int):
        """State-after-row buffers ``[layers, B, G, ...]`` of a verify pass: contiguous views of ONE storage sized for
        the largest batch and depth, shared by every step shape (only one step runs at a time, and its accepted rows
        are committed before the next). Captured graphs keep pointers into it, so it never moves once graphs exist."""
        model = self.engine.model
        n_gdn = model.conv_state.shape[0]
        conv_row = model.conv_state[0, 0].numel()
        rec_row = model.rec_state[0, 0].numel()
        if self._ring_store is None or B * G > self._ring_cap:
            if self._ring_store is not None and self._vgraphs is not None and self._vgraphs.buckets:
                raise RuntimeError("the verify ring cannot grow after graphs were captured")
            cap = max(B * G, self.engine.cfg.max_seqs * (self.policy.kmax + 1)) if self.engine._graphs is not None else B * G
            self._ring_cap = cap
            self._ring_store = (torch.empty(n_gdn * cap * conv_row, dtype=model.dtype, device=model.device),
                                torch.empty(n_gdn * cap * rec_row, dtype=torch.float32, device=model.device))
        conv, rec = self._ring_store
        return (conv[: n_gdn * B * G * conv_row].view(n_gdn, B, G, *model.conv_state.shape[2:]),
                rec[: n_gdn * B * G * rec_row].view(n_gdn, B, G, *model.rec_state.shape[2:]))

    # ------------------------------------------------------------------ prefill hooks
    def after_prefill(self, gens, spans, batch: PackedBatch, hidden: torch.Tensor) -> None:
        """Feed the MTP block the prompt rows ``(x[t+1], H[t])`` and draft from each finished prompt."""
        eng = self.engine
        nxt: list[int] = []
        last_rows, last_gens = [], []
        for i, (g, (a, b)) in enumerate(zip(gens, spans)):
            toks = g.prompt[a + 1 : b + 1]
            if b == len(g.prompt):
                toks = toks + [g.next_token if g.next_token is not None else 0]
                if not g.done and g.next_token is not None:
                    last_rows.append(batch.seg_starts[i + 1] - 1)
                    last_gens.append(g)
            nxt.extend(toks)
        y = eng.model.mtp_forward(hidden, torch.tensor(nxt, dtype=torch.int64, device=eng.device), batch)
        for g, (a, b) in zip(gens, spans):
            g.mtp_computed = b
        if last_gens:
            rows = torch.tensor(last_rows, device=eng.device)
            h = y[rows]
            d = eng.model.draft_pick(h)
            drafts = [d]
            pos = torch.tensor([g.computed for g in last_gens], dtype=torch.int64, device=eng.device)
            self._chain_links(last_gens, h, d, pos, drafts)
            cols = torch.stack(drafts, dim=1).tolist()
            for g, ds in zip(last_gens, cols):
                g.draft = ds

    def first_drafts(self, gens) -> None:
        return None

    def _chain_links(self, gens, h, d, pos, drafts) -> None:
        """Links 2..kmax: the MTP block on (previous link, its own previous normed output)."""
        eng = self.engine
        kmax = self.policy.kmax
        if kmax <= 1:
            return
        for g in gens:
            eng._ensure_pages(g, g.computed + 2 * kmax + 2)
        tables = eng._table(gens).to(eng.device)
        slots = torch.tensor([g.slot for g in gens], dtype=torch.int32, device=eng.device)
        seq = torch.arange(len(gens), dtype=torch.int32, device=eng.device)
        for j in range(1, kmax):
            b = PackedBatch(d, pos + (j - 1), seq, slots, tables, 1)
            h = eng.model.mtp_forward(h, d, b)
            d = eng.model.draft_pick(h)
            drafts.append(d)

    # ------------------------------------------------------------------ the verify step
    def step(self, running) -> bool:
        eng = self.engine
        gens = []
        for g in list(running):
            try:
                eng._ensure_pages(g, g.computed + 2 * self.policy.kmax + 3)
                gens.append(g)
            except Exception:  # noqa: BLE001 - out of pages: let the plain path report it
                return False
        if not gens:
            return False
        B = len(gens)
        elig = [self.eligible(g) for g in gens]
        avail = min((len(g.draft) if e else self.policy.kmax) for g, e in zip(gens, elig)) if any(elig) else 0
        room = min(max(1, g.remaining or 1) for g in gens) - 1  # never draft past the shortest remaining budget
        k = self.policy.choose(B, min(avail, max(room, 0))) if any(elig) else 0
        G = k + 1
        self.k_hist[k] = self.k_hist.get(k, 0) + 1
        tokens, positions, n_valid = [], [], []
        for g, e in zip(gens, elig):
            ds = list(g.draft[:k]) if e else []
            if e and self.draft_override is not None:
                ds = list(self.draft_override(g, k))[:k]
            n_valid.append(len(ds))
            ds = ds + [0] * (k - len(ds))
            tokens.extend([g.next_token] + ds)
            positions.extend(range(g.computed, g.computed + G))
        res = None
        if eng._graphs is not None and eng._graphs.usable(gens) and not any(eng._needs_logits(g) for g in gens):
            if self._vgraphs is None:
                from ..sched.graphs import VerifyGraphs

                self._vgraphs = VerifyGraphs(eng, eng._graphs, self.policy.kmax, self._ring)
            res = self._vgraphs.run(gens, tokens, positions, n_valid, k)
        if res is not None:
            picks_h, acc_h, drafts_h, ring, slots_t = res
        else:
            picks_h, acc_h, drafts_h, ring, slots_t = self._eager_step(gens, elig, tokens, positions, n_valid, k)
        self._book(gens, elig, n_valid, k, picks_h, acc_h, drafts_h, ring, slots_t)
        return True

    def _eager_step(self, gens, elig, tokens, positions, n_valid, k):
        """The same step launched kernel by kernel (CPU, sampled rows, or a shape without a captured graph)."""
        eng = self.engine
        B, G = len(gens), k + 1
        batch = PackedBatch.uniform(tokens, positions, [g.slot for g in gens], eng._table(gens), G, eng.device)
        ring = self._ring(B, G)
        hidden = eng.model.forward(batch, ring=ring)
        picks = eng.model.greedy(hidden)
        tok = batch.tokens.view(B, G)
        pk = picks.view(B, G)
        valid = torch.arange(k, device=eng.device)[None, :] < torch.tensor(n_valid, device=eng.device)[:, None]
        match = ((tok[:, 1:] == pk[:, :-1]) & valid).long()
        acc = torch.cumprod(match, dim=1).sum(dim=1) if k > 0 else torch.zeros(B, dtype=torch.long, device=eng.device)
        # sampled / EOS-masked rows: their row-0 token comes from the sampler, not the argmax
        sampled: dict[int, int] = {}
        need = [i for i, g in enumerate(gens) if eng._needs_logits(g)]
        if need:
            rows0 = torch.tensor([i * G for i in need], device=eng.device)
            rows = [gens[i] for i in need]
            chosen = pick_tokens(eng.model.logits(hidden[rows0]), [g.sampling for g in rows], [g.rng for g in rows],
                                 [eng.eos if len(g.output) < g.sampling.min_tokens else None for g in rows])
            sampled.update(zip(need, chosen))
            fix = torch.tensor([[i * G, t] for i, t in sampled.items()], device=eng.device)
            picks = picks.clone()
            picks[fix[:, 0]] = fix[:, 1]
        # MTP on every row keeps its KV complete; the next chain starts at the last accepted row
        y = eng.model.mtp_forward(hidden, picks, batch)
        sel = torch.arange(B, device=eng.device) * G + acc
        h = y[sel]
        d = eng.model.draft_pick(h)
        drafts = [d]
        base_pos = batch.positions.view(B, G)[:, 0] + acc + 1
        self._chain_links(gens, h, d, base_pos, drafts)
        eng.flush_events()
        eng.check_device()
        return picks.view(B, G).tolist(), acc.tolist(), torch.stack(drafts, dim=1).tolist(), ring, batch.slots

    def _book(self, gens, elig, n_valid, k, picks_h, acc_h, drafts_h, ring, slots_t) -> None:
        eng = self.engine
        B = len(gens)
        # Phase 1: how many picks each request can book (EOS and the token budget end the run early),
        # hence which row's state to keep. The cache must be settled before any request retires.
        keep, book = [], []
        for i, g in enumerate(gens):
            a = acc_h[i] if elig[i] else 0
            n, eos = 0, False
            for j in range(a + 1):
                if picks_h[i][j] in eng.eos and not g.sampling.ignore_eos:
                    eos = True
                    break
                n += 1
                if len(g.output) + n >= g.sampling.max_tokens:
                    break
            used = n + 1 if eos else n  # rows whose tokens are confirmed: the EOS pick confirms its row too
            keep.append(used - 1)
            book.append((n, eos, used, a))
        eng.model.commit_ring(ring, slots_t, torch.tensor(keep, device=eng.device))
        # Phase 2: book the tokens (this may finish requests and park their state as session tails)
        for i, g in enumerate(gens):
            n, eos, used, a = book[i]
            g.computed += used
            g.mtp_computed = g.computed
            g.draft = drafts_h[i] if (used == a + 1 and not eos) else []
            for j in range(n + (1 if eos else 0)):
                eng._accept_token(g, picks_h[i][j])
            if g.done:
                g.draft = []
            if elig[i] and k > 0:
                g.spec_proposed += n_valid[i]
                g.spec_accepted += min(a, n_valid[i])
                self.policy.observe(n_valid[i], a)
        st = eng.stats
        st["decode_steps"] += 1
        st["decoded_tokens"] += B
        st["largest_batch"] = max(st["largest_batch"], B)
        if k > 0:
            st["mtp_verify_steps"] += 1
            st["mtp_proposed"] += sum(n_valid)
            st["mtp_accepted"] += sum(min(a, n) for a, n, e in zip(acc_h, n_valid, elig) if e)

    def reset(self) -> None:
        """After the engine failed everything in flight: no per-request state lives here beyond the requests'."""
        return None

    def settle(self, gen) -> None:
        """Nothing to undo: a verify step commits exactly the rows whose tokens were booked."""
        return None

    def stats(self) -> dict:
        return {"spec_k_hist": dict(self.k_hist), "spec_accept": [round(a, 3) for a in self.policy.accept[: self.policy.kmax]]}
