"""More rank-group scenarios for ``dist_worker.py`` (host-side failure handling; all of them run on CPU ranks)."""

import torch
import torch.distributed as dist


def _tiny_engine(rank, world, dev, **over):
    from b200serve.config import EngineConfig, ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.parallel.tp import DistComm, TPContext, shard_weights
    from b200serve.sched.engine import Engine

    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    cfg = ModelConfig.tiny()
    full = random_weights(cfg, seed=0, device="cpu", dtype=torch.float32, std=0.05, lm_head_std=0.5).to(dev, dtype)
    kw = dict(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=4, mtp=False, kv_pages=128)
    kw.update(over)
    return Engine(shard_weights(full, rank, world), EngineConfig(**kw), tp=TPContext(rank, world, DistComm(dist.group.WORLD)))


def mode_kv_agree(rank, world, dev):
    """Ranks whose own memory budgets differ must end up with the same (smallest) KV pool."""
    from b200serve.sched.engine import Engine

    local = 300 - 40 * rank
    orig = Engine._auto_pages
    Engine._auto_pages = lambda self, weights, n_slots: local
    try:
        eng = _tiny_engine(rank, world, dev, kv_pages=0)
    finally:
        Engine._auto_pages = orig
    assert eng.pages.num_pages == 300 - 40 * (world - 1), (rank, eng.pages.num_pages)


def mode_lockstep_failure(rank, world, dev):
    """One rank of a lockstep replica reports a device-side failure: at the next agreement EVERY rank fails what is
    in flight, refuses new requests and marks itself unavailable; nobody is left waiting in a collective."""
    from b200serve.parallel.lockstep import Coordinator
    from b200serve.sched.request import Generation, Sampling

    eng = _tiny_engine(rank, world, dev)
    eng.coordinator = Coordinator(dist.new_group(backend="gloo"), rank)
    if rank != 0:
        n = 0
        while eng.coordinator.sync(eng):
            eng.step(synced=True)
            n += 1
            if n == 4 and rank == world - 1:
                eng.device_error_pending = True  # what Engine.check_device latches when the error word was set
        assert eng.broken is not None and not eng.running and not eng.prefilling
        return
    g = torch.Generator().manual_seed(5)
    gens = [eng.submit(Generation(torch.randint(3, 1024, (n,), generator=g).tolist(), Sampling(max_tokens=200, ignore_eos=True)))
            for n in (40, 90)]
    for _ in range(12):
        eng.step()
    assert eng.broken is not None
    for x in gens:
        assert x.done and x.finish_reason == "error" and 0 < len(x.output) < 200, (x.finish_reason, len(x.output))
    seen = []
    late = eng.submit(Generation([5, 6, 7, 8], Sampling(max_tokens=4, ignore_eos=True), on_event=lambda g, ev: seen.append(ev)))
    eng.step()
    assert late.finish_reason == "error" and seen and seen[-1].error is not None and seen[-1].error.status == 503
    assert eng.health()["broken"]
    eng.coordinator.stop(eng)
