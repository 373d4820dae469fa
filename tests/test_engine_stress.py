"""Randomised scheduler stress on the CPU: arrivals, cancellations and shared prefixes in random order must never
change a request's greedy tokens, leak a page or a slot, or leave a request unfinished."""

import random

import pytest
import torch

from b200serve.config import EngineConfig, ModelConfig
from b200serve.models.checkpoint import random_weights
from b200serve.sched.engine import Engine
from b200serve.sched.request import Generation, Sampling


@pytest.fixture(scope="module")
def weights():
    return random_weights(ModelConfig.tiny(), seed=0, dtype=torch.float32, std=0.05, lm_head_std=0.5)


def _engine(weights, **kw):
    base = dict(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=6, kv_pages=96, device="cpu", mtp=False,
                decode_buckets=(1, 2, 4, 8))
    base.update(kw)
    return Engine(weights, EngineConfig(**base))


CONFIGS = [
    dict(),
    dict(mtp=True, spec_k=2),
    dict(graphs_on_cpu=True, run_ahead=True),
    dict(graphs_on_cpu=True, run_ahead=True, prefill_graphs=True, mtp=True, spec_k=0),
]


@pytest.mark.parametrize("seed,cfg", [(s, c) for s, c in zip(range(4), CONFIGS)] + [(s + 10, c) for s, c in zip(range(4), CONFIGS)]
                         + [(20, dict(kv_pages=24)), (21, dict(kv_pages=24, graphs_on_cpu=True, run_ahead=True, mtp=True, spec_k=2))])
def test_random_traffic_keeps_tokens_and_accounting(weights, seed, cfg):
    rng = random.Random(seed)
    eng = _engine(weights, **cfg)
    total_pages, total_slots = eng.pages.free, eng.slots.free
    shared = [rng.randrange(3, 1000) for _ in range(150)]  # sessions that share a long prefix
    plan = []
    for i in range(14):
        if rng.random() < 0.4:
            prompt = shared[: rng.randrange(70, 150)] + [rng.randrange(3, 1000) for _ in range(rng.randrange(1, 40))]
        else:
            prompt = [rng.randrange(3, 1000) for _ in range(rng.randrange(1, 200))]
        plan.append(dict(at=rng.randrange(0, 60), prompt=prompt, max_tokens=rng.randrange(1, 30),
                         cancel_after=rng.randrange(2, 25) if rng.random() < 0.25 else None))
    gens: list[Generation | None] = [None] * len(plan)
    steps = 0
    while steps < 3000:
        for i, p in enumerate(plan):
            if gens[i] is None and p["at"] <= steps:
                gens[i] = eng.submit(Generation(p["prompt"], Sampling(max_tokens=p["max_tokens"], ignore_eos=True)))
                p["born"] = steps
            if gens[i] is not None and p["cancel_after"] is not None and steps - p["born"] >= p["cancel_after"]:
                gens[i].cancelled.set()
        busy = eng.step()
        steps += 1
        if not busy and all(g is not None and g.done for g in gens):
            break
    assert all(g is not None and g.done for g in gens), [None if g is None else g.finish_reason for g in gens]
    solo = _engine(weights, prefix_cache_entries=0)
    for g, p in zip(gens, plan):
        want = solo.generate([p["prompt"]], Sampling(max_tokens=p["max_tokens"], ignore_eos=True))[0].output
        if g.finish_reason == "cancelled":
            assert g.output == want[: len(g.output)] and p["cancel_after"] is not None
        elif g.finish_reason == "error":  # refused for lack of KV pages (the small-pool cases): whatever came out is right
            assert cfg.get("kv_pages", 96) < 96 and g.output == want[: len(g.output)]
        else:
            assert g.finish_reason == "length" and g.output == want, (len(p["prompt"]), p["max_tokens"])
    assert not eng.running and not eng.prefilling and not eng.waiting and eng._pending is None
    # what is still taken belongs to cached tails and snapshots, and goes back with them
    eng.cache.clear()
    assert eng.pages.free == total_pages and eng.slots.free == total_slots
    if cfg.get("mtp"):
        assert eng.stats["mtp_verify_steps"] > 0
    if cfg.get("prefill_graphs"):
        assert eng.stats["prefill_graph_passes"] > 0
