"""Scheduler, caches and batching on the CPU fp32 path with a tiny random model."""

import pytest
import torch

from b200serve.config import EngineConfig, ModelConfig
from b200serve.models.checkpoint import random_weights
from b200serve.sched.engine import Engine
from b200serve.sched.request import Generation, Sampling


@pytest.fixture(scope="module")
def weights():
    torch.manual_seed(0)
    cfg = ModelConfig.tiny()
    cfg.eos_token_ids = [2]
    return random_weights(cfg, seed=0, dtype=torch.float32, std=0.02, lm_head_std=0.5)


def _engine(weights, **kw):
    cfg = EngineConfig(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=8, mtp=False, **kw)
    return Engine(weights, cfg)


def _prompts(n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(3, 1024, (int(torch.randint(16, 200, (1,), generator=g)),), generator=g).tolist() for _ in range(n)]


def test_batched_equals_solo_and_exact_lengths(weights):
    prompts = _prompts(8)
    s = Sampling(max_tokens=32, ignore_eos=True)
    eng = _engine(weights)
    batched = [g.output for g in eng.generate(prompts, s)]
    assert all(len(o) == 32 for o in batched)
    assert eng.stats["decoded_tokens"] > eng.stats["decode_steps"]  # requests shared decode steps
    for p, out in zip(prompts[:4], batched[:4]):
        solo = _engine(weights).generate([p], s)[0].output
        assert solo == out


def test_repeated_prompt_hits_tail_cache_and_keeps_tokens(weights):
    eng = _engine(weights)
    p = _prompts(1, seed=3)[0]
    s = Sampling(max_tokens=9, ignore_eos=True)
    a = eng.generate([p], s)[0]
    b = eng.generate([p], s)[0]
    assert a.cached_tokens == 0
    assert b.cached_tokens > 0 and b.cached_tokens <= len(p) - 1
    assert a.output == b.output
    # next round of the session: prompt + output + new tokens reuses everything but the last token
    nxt = p + a.output + [5, 6, 7]
    c = eng.generate([nxt], s)[0]
    cold = _engine(weights).generate([nxt], s)[0]
    assert c.cached_tokens >= len(p)
    assert c.output == cold.output


def test_growing_prefix_reuses_chunk_boundary_and_equals_cold(weights):
    eng = _engine(weights)
    base = _prompts(1, seed=5)[0]
    base = (base * 12)[:150]
    s = Sampling(max_tokens=6, ignore_eos=True)
    eng.generate([base], s)
    other = base[:140] + [9, 9, 9, 9]
    got = eng.generate([other], s)[0]
    assert got.cached_tokens == 128  # the chunk-boundary snapshot, not the diverged tail
    cold = _engine(weights).generate([other], s)[0]
    assert got.output == cold.output


def test_eos_stops_and_min_tokens_masks(weights):
    eng = _engine(weights)
    p = _prompts(1, seed=7)[0]
    free = eng.generate([p], Sampling(max_tokens=40, ignore_eos=True))[0].output
    eng.eos = {free[3]}
    eng.cache.clear()
    stopped = eng.generate([p], Sampling(max_tokens=40))[0]
    assert stopped.finish_reason == "stop" and stopped.output == free[:3]
    eng.cache.clear()
    forced = eng.generate([p], Sampling(max_tokens=8, min_tokens=6))[0]
    assert len(forced.output) >= 6 and free[3] not in forced.output[:6]


def test_pages_return_after_eviction_and_pressure_evicts(weights):
    eng = _engine(weights, kv_pages=40)
    total = eng.pages.free
    s = Sampling(max_tokens=4, ignore_eos=True)
    for p in _prompts(12, seed=11):
        eng.generate([p], s)
    assert eng.cache.stats.evictions > 0  # 12 tails do not fit in 39 pages
    eng.cache.clear()
    assert eng.pages.free == total
    assert eng.slots.free == eng.slots.num_slots - 1


def test_validation_errors(weights):
    eng = _engine(weights)
    events = []
    g = Generation(list(range(3, 2000)), Sampling(max_tokens=4), on_event=lambda g, e: events.append(e))
    eng.submit(g)
    eng.step()
    assert g.finish_reason == "error" and events[-1].error.status == 400
    g2 = Generation([5000], Sampling(max_tokens=4), on_event=lambda g, e: events.append(e))
    eng.submit(g2)
    eng.step()
    assert g2.finish_reason == "error"


def test_seeded_sampling_is_reproducible(weights):
    p = _prompts(1, seed=13)[0]
    s = Sampling(max_tokens=12, temperature=0.8, top_p=0.9, top_k=50, seed=42, ignore_eos=True)
    a = _engine(weights).generate([p], s)[0].output
    b = _engine(weights).generate([p], s)[0].output
    assert a == b and len(a) == 12


def test_one_pass_prefill_runs_a_short_prompt_as_one_span_without_a_snapshot(weights):
    """``one_pass_max``: the uncached part of a prompt in one pass, the reference's default for up to 4096 tokens;
    same tokens as the chunked form, tails still resume, but no chunk-boundary state is kept for other requests."""
    p = _prompts(1, seed=21)[0] * 3  # several chunks long
    s = Sampling(max_tokens=6, ignore_eos=True)
    chunked, one = _engine(weights), _engine(weights, one_pass_max=4096)
    a = chunked.generate([p], s)[0]
    b = one.generate([p], s)[0]
    assert a.output == b.output
    assert one.stats["prefill_passes"] == 1 < chunked.stats["prefill_passes"]
    other = p[: len(p) - 5] + [3, 4, 5, 6, 7, 8]  # diverges near the end: only a chunk-boundary snapshot could help
    assert chunked.generate([other], s)[0].cached_tokens > 0
    assert one.generate([other], s)[0].cached_tokens == 0
    nxt = p + a.output + [9, 9, 9]  # the next turn of the same session resumes from the tail either way
    ra, rb = chunked.generate([nxt], s)[0], one.generate([nxt], s)[0]
    assert ra.output == rb.output and rb.cached_tokens >= len(p)
    long_one = _engine(weights, one_pass_max=50)  # a part longer than the limit is chunked as before
    assert long_one.generate([p], s)[0].output == a.output and long_one.stats["prefill_passes"] > 1
