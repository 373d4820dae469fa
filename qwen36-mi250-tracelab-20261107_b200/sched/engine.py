"""Continuous-batching engine: admission, chunked packed prefill, batched decode, retirement.

One thread owns the model and calls ``step()`` in a loop (the reference's ``Worker`` is the
only thread that touches its model as well, ``engine/server.py:94-296``). Each iteration

1. drains the submission queue and admits requests (prefix-cache claim, slot and page
   allocation),
2. runs at most one packed prefill pass: the next chunk-aligned span of every pending
   request under a token budget (reference: ``PackedPrefill``, ``engine/generator.py:1127-1230``),
3. runs one decode step for every running request (a CUDA graph per batch bucket on GPU),
4. emits tokens, finishes requests and parks their state as session tails.

Prefill rows and decode rows never share a forward pass, and span boundaries depend only on
(prompt, cached start, chunk size); with batch-invariant kernels this makes every request's
greedy tokens identical to the same request served alone.
"""

from __future__ import annotations

import queue
import time
from typing import Iterable

import torch

from ..cache.pools import OutOfCapacity, PagePool, SlotPool
from ..cache.prefix import PrefixCache
from ..config import PAGE_SIZE, EngineConfig, ModelConfig
from ..models.checkpoint import Weights
from ..models.qwen36 import Model, PackedBatch
from ..ops import torch_ops
from ..obs import looptimers
from .request import EngineError, Generation, Sampling, TokenEvent
from .sampling import pick_tokens


def _select_ops(device: torch.device):
    if device.type == "cuda":
        from ..ops import cuda_ops

        cuda_ops.lib()  # raises when the kernel library is missing: never fall back silently on a GPU
        return cuda_ops
    return torch_ops


class Engine:
    def __init__(self, weights: Weights, cfg: EngineConfig | None = None, ops=None, tp=None, ep=None, pp=None) -> None:
        """``tp``: a ``parallel.tp.TPContext`` when ``weights`` is one rank's shard; all ranks of the group
        then run the same engine on the same requests in lockstep. ``ep``: a ``parallel.ep.EpMoE`` for data-parallel
        attention with expert-parallel MoE: every rank serves its own requests, but all ranks must issue the same
        sequence of forward passes (same number of prefill passes and decode steps), which the caller arranges.
        ``pp``: a ``parallel.pp.PPContext`` when ``weights`` is one rank's run of layers (``parallel.pp.split_layers``);
        the ranks run in lockstep like a tensor-parallel replica, launch eagerly and do not speculate."""
        self.cfg = cfg or EngineConfig()
        if pp is not None:
            import dataclasses

            self.cfg = dataclasses.replace(self.cfg, cuda_graphs=False, mtp=False)
        self.tp = tp
        self.pp = pp
        self.coordinator = None  # parallel.lockstep.Coordinator in a multi-rank replica
        self.tick = None  # parallel.dpep.TickCoordinator: data-parallel replicas that share expert-parallel MoE blocks
        self.mcfg: ModelConfig = weights.config
        self.device = weights.device
        self.ops = ops or _select_ops(self.device)
        c = self.cfg
        self.chunk = max(PAGE_SIZE, (c.prefill_chunk_tokens + PAGE_SIZE - 1) // PAGE_SIZE * PAGE_SIZE)
        self.max_model_len = c.max_model_len
        self.max_pages_per_seq = (self.max_model_len + PAGE_SIZE - 1) // PAGE_SIZE + 1
        draft_index = None
        if c.draft_ivf and c.mtp and weights.mtp is not None and tp is None and pp is None:
            from ..spec.ivf import IvfIndex

            # from the plain head, before it is tile-packed; deterministic, so every restart builds the same index
            if getattr(weights.lm_head, "b200_packed", None):
                raise ValueError("draft_ivf needs the LM head in its plain layout: build the engine before packing")
            draft_index = IvfIndex.build(weights.lm_head, n_clusters=c.draft_ivf, probes=c.draft_ivf_probes)
        if c.pack_weights and tp is None and hasattr(self.ops, "pack_weights"):
            self.ops.pack_weights(weights)  # before the KV pool is sized: padded copies replace a few tensors
        n_slots = c.state_slots or (c.max_seqs * 2 + 2)
        n_pages = c.kv_pages or self._agree_min(self._auto_pages(weights, n_slots), tp if tp is not None else pp)
        self.model = Model(weights, n_pages, n_slots, ops=self.ops, tp=tp, ep=ep, pp=pp)
        self.model.draft_index = draft_index
        self.pages = PagePool(n_pages)
        self.slots = SlotPool(n_slots)
        page_bytes = self.model.kv[:, 0].numel() * self.model.kv.element_size()
        slot_bytes = self.mcfg.gdn_state_bytes()
        self.cache = PrefixCache(
            self.pages, self.slots, page_bytes, slot_bytes, c.prefix_cache_entries, c.prefix_cache_tokens,
            int(c.prefix_cache_gib * (1 << 30)),
        )
        self.pages.on_pressure = self.cache.evict_one
        self.slots.on_pressure = self.cache.evict_one
        self.eos = set(self.mcfg.eos_token_ids)
        self._inbox: "queue.SimpleQueue[Generation]" = queue.SimpleQueue()
        self.waiting: list[Generation] = []
        self.prefilling: list[Generation] = []
        self.running: list[Generation] = []
        self._deferred: list = []
        self._flushed = False
        self.multi_rank = tp is not None or ep is not None or pp is not None
        self.broken: str | None = None  # set when a rank group can no longer be trusted to be in step
        self.device_error_pending = False  # multi-rank: a device-side failure seen since the last agreement
        self.stats = dict(
            decode_steps=0, decoded_tokens=0, largest_batch=0, prefill_passes=0, prefill_segments=0,
            prefilled_tokens=0, cached_tokens=0, requests=0, finished=0, failed=0,
            mtp_verify_steps=0, mtp_proposed=0, mtp_accepted=0, device_errors=0, step_errors=0, ahead_steps=0,
            prefill_graph_passes=0,
        )
        if c.loop_timers:  # the switches also come in through the configuration, not only the environment
            looptimers.ENABLED = True
        if c.req_stamps:
            from ..obs import reqstamps

            reqstamps.ENABLED = True
        self._graphs = None
        # library collectives (the NCCL baseline path) stay out of CUDA graphs; the fused NVLink kernels go in
        emulate = c.cuda_graphs and c.graphs_on_cpu and self.device.type != "cuda"
        if (self.device.type == "cuda" or emulate) and c.cuda_graphs and (tp is None or getattr(tp.comm, "fused", False) or emulate):
            from .graphs import DecodeGraphs

            self._graphs = DecodeGraphs(self)
        self._pending = None  # a decode step in flight (launched ahead of the host's bookkeeping)
        self._pgraphs = None  # captured prefill passes (built after the speculative controller: they include its block)
        self.spec = None
        if c.mtp and weights.mtp is not None:
            from ..spec.controller import SpecController

            self.spec = SpecController(self)
        if c.prefill_graphs and c.cuda_graphs:
            from .graphs import PrefillGraphs

            if PrefillGraphs.supported(self):
                self._pgraphs = PrefillGraphs(self)

    # ------------------------------------------------------------------ sizing
    def _auto_pages(self, weights: Weights, n_slots: int) -> int:
        c, m = self.cfg, self.mcfg
        per_page = m.kv_bytes_per_token(2 if weights.dtype != torch.float32 else 4) * PAGE_SIZE
        if self.device.type != "cuda":
            return min(4096, c.max_seqs * (min(self.max_model_len, 8192) // PAGE_SIZE + 2) + 64)
        free, _total = torch.cuda.mem_get_info(self.device)
        ring_rows = c.max_seqs * (max(1, c.spec_kmax) + 1) if (c.mtp and m.mtp_num_hidden_layers) else 0  # verify ring
        budget = free * c.kv_fraction - c.reserve_gb * (1 << 30) - (n_slots + ring_rows) * m.gdn_state_bytes()
        pages = int(budget // per_page)
        need = self.max_pages_per_seq + 8  # at least one full-length sequence (reference: model.py:492-521)
        if pages < min(need, 64):
            raise RuntimeError(f"not enough device memory for the KV pool ({pages} pages)")
        return pages

    def _agree_min(self, value: int, tp) -> int:
        """The smallest ``value`` over the ranks of a tensor-parallel or layer-split replica. Capacities derived from a rank's own
        free memory differ between GPUs (other contexts, other users' jobs), but the lockstep design needs every rank
        to allocate, evict and refuse identically, so all ranks adopt the tightest budget."""
        if tp is None:
            return value
        import torch.distributed as dist

        group = getattr(getattr(tp, "comm", None), "group", None)
        if group is None and hasattr(tp, "is_last"):  # a layer-split replica: its own group, or all ranks
            group = tp.group if tp.group is not None else dist.group.WORLD
        if group is None:
            return value

        on_gpu = dist.get_backend(group) == "nccl"
        t = torch.tensor([value], dtype=torch.int64, device=self.device if on_gpu else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
        return int(t.item())

    # ------------------------------------------------------------------ public API
    def submit(self, gen: Generation) -> Generation:
        self._inbox.put(gen)
        return gen

    def has_work(self) -> bool:
        return bool(self.waiting or self.prefilling or self.running or self._pending) or not self._inbox.empty()

    def generate(self, prompts: Iterable[list[int]], sampling: Sampling | list[Sampling]) -> list[Generation]:
        """Offline convenience: run the given prompts to completion and return their generations."""
        prompts = list(prompts)
        samplings = sampling if isinstance(sampling, list) else [sampling] * len(prompts)
        gens = [self.submit(Generation(p, s)) for p, s in zip(prompts, samplings)]
        while any(not g.done for g in gens):
            self.step()
        return gens

    def validate(self, prompt: list[int], sampling: Sampling) -> None:
        if not prompt:
            raise EngineError("the prompt is empty")
        if len(prompt) >= self.max_model_len:
            raise EngineError(
                f"the prompt has {len(prompt)} tokens; this model's context is {self.max_model_len} tokens"
            )
        if sampling.max_tokens is not None and len(prompt) + sampling.max_tokens > self.max_model_len:
            raise EngineError(
                f"prompt ({len(prompt)} tokens) plus max_tokens ({sampling.max_tokens}) exceeds the "
                f"context of {self.max_model_len} tokens"
            )
        v = self.mcfg.vocab_size
        if any((t < 0 or t >= v) for t in prompt):
            raise EngineError(f"the prompt contains a token id outside [0, {v})")

    # ------------------------------------------------------------------ admission
    def _spans(self, start: int, end: int) -> list[tuple[int, int]]:
        """Chunk-aligned spans covering ``[start, end)`` exactly once."""
        spans, a = [], start
        while a < end:
            b = min(end, (a // self.chunk + 1) * self.chunk)
            spans.append((a, b))
            a = b
        return spans

    def _claim(self, gen: Generation) -> None:
        """Give the request a state slot and any cached prefix (reference: ``_claim``, generator.py:932-973)."""
        entry = self.cache.lookup(gen.prompt)
        if entry is not None and entry.kind == "tail":
            gen.slot, gen.pages, gen.computed = entry.slot, list(entry.pages), entry.length
        elif entry is not None:
            try:
                gen.slot = self.slots.alloc()
            except OutOfCapacity:
                raise EngineError("all sequence slots are busy", 503, "service_unavailable") from None
            self.model.copy_slot(entry.slot, gen.slot)
            self.pages.incref(entry.pages)
            gen.pages, gen.computed = list(entry.pages), entry.length
        else:
            try:
                gen.slot = self.slots.alloc()
            except OutOfCapacity:
                raise EngineError("all sequence slots are busy", 503, "service_unavailable") from None
            self.model.reset_slot(gen.slot)
            gen.pages, gen.computed = [], 0
        gen.cached_tokens = gen.computed
        gen.mtp_computed = 0
        L = len(gen.prompt)
        if 0 < self.cfg.one_pass_max and L - gen.computed <= self.cfg.one_pass_max:
            # the uncached part in ONE span, the last token included: one pass, and no state snapshot on the way (the
            # reference's default for parts of up to 4096 tokens, engine/generator.py:795-816; its sessions resume
            # from their tails). Off by default here: the snapshot at the last chunk boundary is what lets DIFFERENT
            # requests share a common prefix such as a system prompt.
            gen.spans = [(gen.computed, L)]
            gen.snapshot_at = 0
        else:
            gen.spans = self._spans(gen.computed, L)
            boundary = (L - 1) // self.chunk * self.chunk
            gen.snapshot_at = boundary if boundary > gen.computed else 0
        if gen.sampling.max_tokens is None:
            gen.sampling.max_tokens = self.max_model_len - L
        if gen.sampling.seed is not None or not gen.sampling.greedy:
            gen.rng = torch.Generator(device="cpu")
            gen.rng.manual_seed(gen.sampling.seed if gen.sampling.seed is not None else gen.id * 7919)

    def _poll_local(self) -> None:
        """Single-process mode: take new submissions and latch cancellations at the iteration boundary."""
        while True:
            try:
                g = self._inbox.get_nowait()
            except queue.Empty:
                break
            if g.sampling.seed is None and not g.sampling.greedy:
                g.sampling.seed = (g.id * 7919 + int(time.time() * 1e3)) % (2**31)
            self.waiting.append(g)
        for g in self.waiting:
            g.cancel_now = g.cancel_now or g.cancelled.is_set()
        for g in self.prefilling:
            g.cancel_now = g.cancel_now or g.cancelled.is_set()
        for g in self.running:
            g.cancel_now = g.cancel_now or g.cancelled.is_set()

    def _admit(self) -> None:
        while self.waiting and len(self.prefilling) + len(self.running) < self.cfg.max_seqs:
            gen = self.waiting.pop(0)
            self.stats["requests"] += 1
            if gen.cancel_now:
                self._finish(gen, "cancelled", retire=False)
                continue
            try:
                self.validate(gen.prompt, gen.sampling)
                if gen.sampling.max_tokens == 0:
                    self._finish(gen, "length", retire=False)
                    continue
                self._claim(gen)
            except EngineError as e:
                self._fail(gen, e)
                continue
            self.stats["cached_tokens"] += gen.cached_tokens
            self.prefilling.append(gen)

    # ------------------------------------------------------------------ pages
    def _ensure_pages(self, gen: Generation, upto_tokens: int) -> None:
        need = (upto_tokens + PAGE_SIZE - 1) // PAGE_SIZE - len(gen.pages)
        if need > 0:
            gen.pages.extend(self.pages.alloc(need))

    def _table(self, gens: list[Generation], width: int | None = None) -> torch.Tensor:
        width = width or max(1, max(len(g.pages) for g in gens))
        t = torch.zeros(len(gens), width, dtype=torch.int32)
        for i, g in enumerate(gens):
            if g.pages:
                t[i, : len(g.pages)] = torch.tensor(g.pages, dtype=torch.int32)
        return t

    # ------------------------------------------------------------------ prefill
    def _prefill_pass(self) -> bool:
        budget = self.cfg.prefill_pack_tokens
        picked: list[Generation] = []
        for gen in list(self.prefilling):
            if gen.cancel_now:
                self.prefilling.remove(gen)
                self._finish(gen, "cancelled")
                continue
            a, b = gen.spans[0]
            if picked and b - a > budget:
                continue
            try:
                self._ensure_pages(gen, b)
            except OutOfCapacity:
                if not picked and not self.running:
                    self.prefilling.remove(gen)
                    self._fail(gen, EngineError("the KV cache is full", 503, "service_unavailable"))
                continue
            picked.append(gen)
            budget -= b - a
            if budget <= 0:
                break
        if self.tick is not None:
            # Replicas that share their MoE blocks run every pass together: a prefill pass happens on all of them as
            # soon as one has a span to compute; a replica without one joins with an empty pass (it still hosts
            # experts for the others' rows).
            if not self.tick.any(self, bool(picked), "prefill"):
                return False
            if not picked:
                return self._empty_pass()
        if not picked:
            return False
        spans = [g.spans[0] for g in picked]
        graph = self._pgraphs.pick(picked, spans) if self._pgraphs is not None else None
        try:
            if graph is not None:  # one request's short span: a single replay instead of a launch-bound pass
                hidden, batch = self._pgraphs.run(graph, picked[0], *spans[0])
                self.stats["prefill_graph_passes"] += 1
            else:
                batch = PackedBatch.prefill(
                    [g.prompt[a:b] for g, (a, b) in zip(picked, spans)], [g.slot for g in picked],
                    [a for a, _ in spans], self._table(picked), self.device,
                )
                hidden = self.model.forward(batch)
            self.check_device()
            if self.tick is not None and self.tick.trace:
                print(f"pass done: prefill of {batch.tokens.shape[0]} rows", flush=True)
        except Exception as e:  # fail the packed requests only; the engine keeps serving
            print(f"engine: prefill pass of {sum(b - a for a, b in spans)} tokens failed: {e!r}", flush=True)
            for g in picked:
                self.prefilling.remove(g)
                self._fail(g, EngineError(f"prefill failed: {e}", 500, "internal_error"))
            if self.multi_rank:
                # the pass stopped part-way: the other ranks ran kernels that this one never launched
                self.device_error_pending = True
            return True
        self.stats["prefill_passes"] += 1
        self.stats["prefill_segments"] += len(picked)
        self.stats["prefilled_tokens"] += sum(b - a for a, b in spans)
        finished_rows, finished = [], []
        for i, (g, (a, b)) in enumerate(zip(picked, spans)):
            g.spans.pop(0)
            g.computed = b
            if g.snapshot_at and b == g.snapshot_at:
                self._snapshot(g)
            if not g.spans:
                finished_rows.append(batch.seg_starts[i + 1] - 1)
                finished.append(g)
        if self.spec is not None:
            if graph is not None:  # the captured pass ran the MTP block over the span already
                picked[0].mtp_computed = spans[0][1]
            else:
                self.spec.after_prefill(picked, spans, batch, hidden)
        if finished:
            rows = torch.tensor(finished_rows, device=self.device)
            self._sample_and_emit(finished, hidden[rows])
            for g in finished:
                self.prefilling.remove(g)
                if not g.done:
                    self.running.append(g)
            if self.spec is not None:
                self.spec.first_drafts([g for g in finished if not g.done])
        return True

    def _snapshot(self, gen: Generation) -> None:
        if self.cache.has_snapshot(gen.prompt, gen.computed):
            return
        try:
            slot = self.slots.alloc()
        except OutOfCapacity:
            return
        self.model.copy_slot(gen.slot, slot)
        if not self.cache.store_snapshot(gen.prompt, gen.computed, gen.pages, slot):
            self.slots.release(slot)

    def _empty_pass(self) -> bool:
        """This replica's part of a pass in which it has no rows of its own."""
        try:
            self.model.forward_empty()
            self.check_device()
            if self.tick is not None and self.tick.trace:
                print("pass done: empty", flush=True)
        except Exception as e:  # noqa: BLE001
            print(f"engine: empty pass failed: {e!r}", flush=True)
            self.device_error_pending = True
        return True

    # ------------------------------------------------------------------ decode
    def _ahead_ok(self, gens) -> bool:
        """May the step AFTER the one in flight be launched for the same requests before the host has seen the one in
        flight? Only when that next step is certain to run unchanged: nothing waits to be admitted or prefilled, the
        requests in flight are all the running ones, none of them can stop on a token (greedy, ``ignore_eos``, no
        EOS masking pending), none is cancelled, and each still needs a token after the step in flight
        (reference: ``_ahead_safe``, engine/speculative.py:266-274)."""
        c = self.cfg
        if not c.run_ahead or self.tick is not None or self.spec is not None:
            return False
        if self.waiting or self.prefilling or (self.coordinator is None and not self._inbox.empty()):
            return False
        if len(gens) != len(self.running) or any(a is not b for a, b in zip(gens, self.running)):
            return False
        for g in gens:
            s = g.sampling
            if not (s.greedy and s.ignore_eos) or g.cancel_now or len(g.output) < s.min_tokens:
                return False
            if len(g.output) + 1 >= s.max_tokens:  # it finishes at the step in flight
                return False
        return True

    def _collect_pending(self) -> None:
        """Read the step in flight, book its tokens."""
        h, self._pending = self._pending, None
        gens = h["gens"]
        try:
            hidden, greedy = self._graphs.collect(h)
        except Exception as e:
            for g in gens:
                if g in self.running:
                    self.running.remove(g)
                self._fail(g, EngineError(f"decode failed: {e}", 500, "internal_error"))
            return
        for g in gens:
            g.computed += 1
        B = len(gens)
        self.stats["decode_steps"] += 1
        self.stats["decoded_tokens"] += B
        self.stats["largest_batch"] = max(self.stats["largest_batch"], B)
        need_logits = any(self._needs_logits(g) for g in gens)
        self._sample_and_emit(gens, hidden, greedy if not need_logits else None)
        self._reap()

    def _decode_step(self) -> bool:
        if self._pending is not None:
            # a step launched ahead is in flight for exactly these requests: maybe start the one after it, then read it
            h = self._pending
            if self._ahead_ok(h["gens"]):
                try:
                    for g in h["gens"]:
                        self._ensure_pages(g, g.computed + 3)
                    nxt = self._graphs.launch_next(h)
                    self.stats["ahead_steps"] += 1
                except OutOfCapacity:
                    nxt = None
                self._collect_pending()
                self._pending = nxt
            else:
                self._collect_pending()
            return True
        for gen in list(self.running):
            if gen.cancel_now:
                self.running.remove(gen)
                self._finish(gen, "cancelled")
        if not self.running and self.tick is None:
            return False
        if self.spec is not None:
            try:
                stepped = self.spec.step(self.running)
            except Exception as e:  # a failed verify step fails its requests; the engine keeps serving
                for g in list(self.running):
                    self.running.remove(g)
                    self._fail(g, EngineError(f"decode failed: {e}", 500, "internal_error"))
                return True
            if stepped:
                self._reap()
                return True
        batch_gens = []
        for gen in list(self.running):
            try:
                self._ensure_pages(gen, gen.computed + 1)
                batch_gens.append(gen)
            except OutOfCapacity:
                self.running.remove(gen)
                self._fail(gen, EngineError("the KV cache is full", 503, "service_unavailable"))
        if self.tick is not None:
            if not self.tick.any(self, bool(batch_gens), "decode"):
                return False
            if not batch_gens:
                return self._empty_pass()
        if not batch_gens:
            return False
        B = len(batch_gens)
        tokens = [g.next_token for g in batch_gens]
        positions = [g.computed for g in batch_gens]
        need_logits = any(self._needs_logits(g) for g in batch_gens)
        try:
            if self._graphs is not None and self._graphs.usable(batch_gens):
                handle = self._graphs.launch(batch_gens, tokens, positions)
                if handle is not None:
                    # in flight: the step after it may start before this one is read (see _ahead_ok)
                    self._pending = handle
                    return self._decode_step()
            batch = PackedBatch.uniform(tokens, positions, [g.slot for g in batch_gens], self._table(batch_gens), 1, self.device)
            hidden = self.model.forward(batch)
            greedy = None
            self.check_device()
        except Exception as e:
            print(f"engine: decode step of {len(batch_gens)} rows failed: {e!r}", flush=True)
            for g in batch_gens:
                self.running.remove(g)
                self._fail(g, EngineError(f"decode failed: {e}", 500, "internal_error"))
            if self.multi_rank:
                self.device_error_pending = True
            return True
        for g in batch_gens:
            g.computed += 1
        self.stats["decode_steps"] += 1
        self.stats["decoded_tokens"] += B
        self.stats["largest_batch"] = max(self.stats["largest_batch"], B)
        self._sample_and_emit(batch_gens, hidden, greedy if not need_logits else None)
        self._reap()
        return True

    def _reap(self) -> None:
        self.running = [g for g in self.running if not g.done]

    # ------------------------------------------------------------------ sampling / emission
    def _needs_logits(self, g: Generation) -> bool:
        s = g.sampling
        return (not s.greedy) or (len(g.output) < s.min_tokens and bool(self.eos))

    def _sample_and_emit(self, gens: list[Generation], hidden: torch.Tensor, greedy: torch.Tensor | None = None) -> None:
        """Pick the next token of each request from its hidden row, emit it and finish on EOS / length."""
        need = [i for i, g in enumerate(gens) if self._needs_logits(g)]
        picks: list[int]
        if not need:
            if greedy is None:
                greedy = self.model.greedy(hidden)
            picks = greedy[: len(gens)].tolist()
        else:
            if greedy is None:
                greedy = self.model.greedy(hidden)
            picks = greedy[: len(gens)].tolist()
            # sampled / EOS-masked rows: filtered and drawn on the device, only the picked ids come back
            logits = self.model.logits(hidden[torch.tensor(need, device=self.device)])
            rows = [gens[i] for i in need]
            chosen = pick_tokens(logits, [g.sampling for g in rows], [g.rng for g in rows],
                                 [self.eos if len(g.output) < g.sampling.min_tokens else None for g in rows])
            for i, tok in zip(need, chosen):
                picks[i] = tok
        for g, tok in zip(gens, picks):
            self._accept_token(g, int(tok))

    def _accept_token(self, g: Generation, tok: int) -> None:
        """Book one sampled token: EOS ends the request without emitting it (unless ignored)."""
        if g.done:
            return
        if tok in self.eos and not g.sampling.ignore_eos:
            self._finish(g, "stop")
            return
        g.output.append(tok)
        g.next_token = tok
        if len(g.output) >= g.sampling.max_tokens:
            self._emit(g, TokenEvent(tok, "length"))
            self._finish(g, "length", emit=False)
        else:
            self._emit(g, TokenEvent(tok, None))

    # ------------------------------------------------------------------ retirement
    def _finish(self, g: Generation, reason: str, retire: bool = True, emit: bool = True) -> None:
        if g.done:
            return
        g.finish_reason = reason
        self.stats["finished"] += 1
        if retire and g.slot:
            if self.spec is not None:
                self.spec.settle(g)
            covered = g.tokens[: g.computed]
            if g.computed > 0 and len(covered) == g.computed:
                keep = (g.computed + PAGE_SIZE - 1) // PAGE_SIZE
                if len(g.pages) > keep:
                    self.pages.release(g.pages[keep:])
                    g.pages = g.pages[:keep]
                self.cache.store_tail(covered, g.pages, g.slot)
            else:
                self.pages.release(g.pages)
                self.slots.release(g.slot)
            g.slot, g.pages = 0, []
        if emit:
            self._emit(g, TokenEvent(None, reason))

    def _fail(self, g: Generation, err: EngineError) -> None:
        self.stats["failed"] += 1
        if g.slot:
            self.pages.release(g.pages)
            self.slots.release(g.slot)
            g.slot, g.pages = 0, []
        g.finish_reason = "error"
        self._emit(g, TokenEvent(None, "error", err))

    # ------------------------------------------------------------------ failures
    def check_device(self, code: int | None = None) -> None:
        """Raise if a kernel of the pass just run recorded a failure in the device error word (a bounded wait that
        gave up, an index out of range): the kernels then skipped their stores, so whatever the pass produced must
        not be sampled from. ``code`` is the word when the caller has already copied it to the host; otherwise it is
        read here (synchronises). The word is cleared, since a set word makes every later peer wait give up at once.
        In a multi-rank engine the failure is also latched for the ranks' next agreement."""
        if not hasattr(self.ops, "err_word"):
            return
        word = self.ops.err_word(self.device)
        if code is None:
            code = int(word.item())
        if code:
            word.zero_()
            self.stats["device_errors"] += 1
            if self.multi_rank:
                self.device_error_pending = True
            names = {1: "a TMA stage never arrived", 2: "no pipeline stage became free", 3: "an accumulator never completed",
                     4: "a peer's flag never arrived", 5: "an index was out of range"}
            print(f"engine: device-side failure {code} ({names.get(code, 'unknown')}) in the pass just run", flush=True)
            raise self.ops.KernelError(f"device-side failure {code} in this pass")

    def fail_all(self, reason: str, status: int = 500) -> None:
        """Fail every request the engine holds and give their slots and pages back."""
        err = EngineError(reason, status, "internal_error" if status == 500 else "service_unavailable")
        while True:
            try:
                self.waiting.append(self._inbox.get_nowait())
            except queue.Empty:
                break
        for g in self.waiting + self.prefilling + self.running:
            if not g.done:
                self._fail(g, err)
        self.waiting, self.prefilling, self.running = [], [], []
        self._pending = None
        if self.spec is not None and hasattr(self.spec, "reset"):
            self.spec.reset()
        self.flush_events()

    def tear_down(self, reason: str) -> None:
        """A rank group whose members may be out of step (a peer wait ran out, a rank raised where the others did
        not) cannot serve correct tokens any more: fail what is in flight, refuse what comes, report it on
        ``/health`` so that the front takes the replica out (reference: the router stops everything when a replica
        dies, ``engine/router.py:568-578``)."""
        if self.broken is None:
            self.broken = reason
            print(f"engine: rank group torn down: {reason}", flush=True)
        self.fail_all(f"replica unavailable: {reason}", 503)

    # ------------------------------------------------------------------ event delivery
    def _emit(self, g: Generation, ev: TokenEvent) -> None:
        """Token events are handed to their consumers (the HTTP handler threads) only at points where this thread
        is about to wait for the GPU: right after the next decode step has been launched, or when the engine goes
        idle. Waking a hundred handler threads any earlier makes this thread queue behind them for the interpreter
        lock while the GPU has nothing to do (the reference launches step n+1 before it reads step n for the same
        reason, ``engine/speculative.py`` run-ahead)."""
        self._deferred.append((g, ev))

    def flush_events(self) -> None:
        self._flushed = True
        if self._deferred:
            pending, self._deferred = self._deferred, []
            for g, ev in pending:
                g.emit(ev)

    # ------------------------------------------------------------------ loop
    def step(self, synced: bool = False) -> bool:
        """One scheduler iteration. Returns False when there was nothing to do.

        In a tensor-parallel replica the ranks first exchange the iteration's new requests and
        cancellations (``parallel.lockstep``); ``synced`` says the caller has already done so."""
        self._flushed = False
        if self.coordinator is None:
            self._poll_local()
        elif not synced and not self.coordinator.sync(self):
            return False
        if self.broken is not None:
            self.fail_all(f"replica unavailable: {self.broken}", 503)
            return False
        if self.device_error_pending and self.coordinator is None:
            # no agreement channel (the caller steps the ranks itself): this rank stops trusting the group at once
            self.tear_down("a device-side wait or check failed on this rank")
            return False
        try:
            with looptimers.stage("admit"):
                self._admit()
            if self.prefilling:
                self.flush_events()  # a prefill pass is long: do not hold decode tokens behind it
            self._flushed = False  # only a delivery after this iteration's passes counts below
            with looptimers.stage("prefill"):
                did = self._prefill_pass()
            with looptimers.stage("decode"):
                did = self._decode_step() or did
        except Exception as e:  # noqa: BLE001
            # Anything that escapes the per-pass handlers (sampling, emission, bookkeeping) would otherwise leave
            # requests half-advanced and fail again on every iteration: fail everything in flight, start clean
            # (reference: a failed step is reported to every request of the step, engine/server.py:291-296)
            import traceback

            traceback.print_exc()
            self.stats["step_errors"] += 1
            self.fail_all(f"engine step failed: {e!r}")
            if self.multi_rank:
                self.device_error_pending = True  # the ranks can no longer be assumed to be in step
            return True
        if not self.running or self._graphs is None or not self._flushed:
            # no graph launch is coming that would deliver them, or this iteration ran without one (eager fallback
            # after a failed capture, a batch outside the buckets): tokens must still stream once per step
            self.flush_events()
        return did

    def warmup(self) -> None:
        """Run one short request and capture every decode graph before serving, so that no request pays for
        first-use work (the reference warms its kernels and captures its graphs before ``/health`` answers,
        ``engine/generator.py:706-728``). Counters and caches are reset afterwards."""
        n = min(self.chunk + 8, self.max_model_len - 8)
        g = self.generate([[1 + (i % 7) for i in range(n)]], Sampling(max_tokens=3, ignore_eos=True))[0]
        assert g.done
        if self._pgraphs is not None:
            self._pgraphs.warm()
        if self._graphs is not None:
            self._graphs.warm()
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
        if self.device.type == "cuda" and hasattr(self.ops, "check_errors"):
            self.ops.check_errors(self.device)  # a failure of the warm-up stops the start, not the first request
        if self.tick is not None:
            self.tick.rendezvous(self)
        self.cache.clear()
        for k in self.stats:
            self.stats[k] = 0
        self.cache.stats = type(self.cache.stats)()

    def health(self) -> dict:
        out = dict(self.stats)
        cs = self.cache.stats
        out.update(
            broken=self.broken,
            prefix_cache_entries=len(self.cache), prefix_cache_bytes=self.cache.bytes,
            prefix_cache_tail_hits=cs.tail_hits, prefix_cache_snapshot_hits=cs.snapshot_hits,
            prefix_cache_evictions=cs.evictions, kv_pages_free=self.pages.free, kv_pages_total=self.pages.num_pages - 1,
            slots_free=self.slots.free, running=len(self.running), prefilling=len(self.prefilling),
            waiting=len(self.waiting),
        )
        return out
