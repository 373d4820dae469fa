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


def mode_dp_ep_served(rank, world, dev):
    """Data-parallel replicas that share expert-parallel MoE blocks, driven like the server drives them: every replica
    loops over ``Engine.step`` on its own, requests arrive at different times in different numbers and lengths, idle
    replicas join with empty passes, decode runs from the graphs captured at warm-up. Every request must produce the
    tokens of the unsharded engine."""
    from b200serve.config import EngineConfig, ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.parallel.dpep import GlooEpMoE, TickCoordinator
    from b200serve.parallel.ep import shard_experts
    from b200serve.sched.engine import Engine
    from b200serve.sched.request import Generation, Sampling

    cuda = dev.type == "cuda"
    cfg = ModelConfig.tiny(num_experts=8)
    dtype = torch.bfloat16 if cuda else torch.float32
    full = random_weights(cfg, seed=0, device="cpu", dtype=torch.float32, std=0.05, lm_head_std=0.5).to(dev, dtype)
    ecfg = EngineConfig(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=8, mtp=False, kv_pages=256,
                        decode_buckets=(1, 2, 4, 8))
    # (arrival step, prompt length) per replica: bursts, gaps, a replica that starts late and one that ends early
    plans = [[(0, 20), (0, 150), (9, 70), (40, 33)], [(5, 33), (18, 200), (18, 64), (18, 18), (19, 90)]]
    plan = plans[rank % 2]
    g = torch.Generator().manual_seed(70 + rank)
    prompts = [torch.randint(3, 1024, (n,), generator=g).tolist() for _, n in plan]
    samp = Sampling(max_tokens=14, ignore_eos=True)
    ref = [x.output for x in Engine(full, ecfg).generate(prompts, samp)]
    cpu_group = dist.new_group(backend="gloo")
    if cuda:
        from b200serve.ops import cuda_ops
        from b200serve.parallel.ep import EpMoE

        ep = EpMoE(dev, dist.group.WORLD, cfg.num_experts, cfg.hidden_size, cfg.num_experts_per_tok, max_rows=512)
    else:
        ep = GlooEpMoE(dist.group.WORLD, cfg.num_experts, cfg.num_experts_per_tok)
    eng = Engine(shard_experts(full, rank, world), ecfg, ep=ep)
    eng.tick = TickCoordinator(cpu_group)
    eng.warmup()
    gens: list = [None] * len(plan)
    it = 0
    while True:
        for i, (at, _n) in enumerate(plan):
            if at == it:
                gens[i] = eng.submit(Generation(prompts[i], samp))
        eng.step()
        it += 1
        mine = all(x is not None and x.done for x in gens) and not eng.has_work()
        flag = torch.tensor([0 if mine else 1], dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=cpu_group)  # everyone finished: leave together
        if int(flag.item()) == 0:
            break
        assert it < 2000 and eng.broken is None, (it, eng.broken)
    if cuda:
        cuda_ops.check_errors(dev)
    got = [x.output for x in gens]
    assert all(x.finish_reason == "length" for x in gens), [x.finish_reason for x in gens]
    assert got == ref, (rank, got, ref)
    if rank == 0:
        print(f"dp_ep_served world={world}: {len(plan)} requests on this replica, {it} loop iterations, "
              f"{eng.stats['prefill_passes']} prefill passes, {eng.stats['decode_steps']} decode steps, tokens equal", flush=True)
    if cuda:
        dist.barrier()
        ep.close()
