"""Multi-rank checks run as ``python -m torch.distributed.run --nproc-per-node N tests/dist_worker.py MODE``.

Ranks are processes, one per GPU (NCCL) or CPU ranks over gloo when no GPU is visible.
Each mode prints ``OK <mode>`` from rank 0 on success; any assertion makes the launcher fail.
"""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def setup():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    return rank, world, dev


def mode_allreduce(rank, world, dev):
    from b200serve.ops import cuda_ops
    from b200serve.parallel.symm import SymmComm

    comm = SymmComm(dev, dist.group.WORLD, slot_elems=1 << 20, max_blocks=1024)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    gc = torch.Generator(device=dev).manual_seed(7)  # replicated tensors: same on every rank
    for T, H in ((1, 2048), (16, 2048), (128, 2048), (7, 512)):
        for dtype in (torch.float32, torch.bfloat16):
            for rep in range(3):
                x = torch.randn(T, H, device=dev, generator=g).to(dtype)
                res = torch.randn(T, H, device=dev, generator=gc).to(torch.bfloat16)
                got = comm.allreduce(x, res)
                ref = x.float().clone()
                dist.all_reduce(ref)
                want = (ref.to(torch.bfloat16).float() + res.float()).to(torch.bfloat16)
                assert torch.equal(got, want), (T, H, dtype, rep, (got.float() - want.float()).abs().max().item())
                # every rank holds the same bits
                gathered = [torch.empty_like(got) for _ in range(world)]
                dist.all_gather(gathered, got)
                assert all(torch.equal(gathered[0], t) for t in gathered)
    # timing: 128 x 2048 (decode batch) and 4 x 2048, device-timed, max over ranks
    for T in (4, 128):
        x = torch.randn(T, 2048, device=dev).to(torch.bfloat16)
        for _ in range(5):
            comm.allreduce(x)
        torch.cuda.synchronize(); dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(50):
            comm.allreduce(x)
        b.record(); torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / 50 * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        y = x.clone()
        for _ in range(5):
            dist.all_reduce(y)
        torch.cuda.synchronize(); dist.barrier()
        a.record()
        for _ in range(50):
            dist.all_reduce(y)
        b.record(); torch.cuda.synchronize()
        t2 = torch.tensor([a.elapsed_time(b) / 50 * 1e3], device=dev)
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        if rank == 0:
            print(f"allreduce {T}x2048 bf16 world={world}: push kernel {t.item():.1f} us, NCCL {t2.item():.1f} us", flush=True)
    cuda_ops.check_errors(dev)
    dist.barrier()
    comm.close()


def mode_tp_model(rank, world, dev):
    """Tensor + expert parallel engine against the unsharded engine on the same requests."""
    from b200serve.config import EngineConfig, ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.parallel.tp import DistComm, FusedComm, TPContext, shard_weights
    from b200serve.sched.engine import Engine
    from b200serve.sched.request import Sampling

    cuda = dev.type == "cuda"
    dtype = torch.bfloat16 if cuda else torch.float32
    # more than 2 ranks need more heads than the default tiny model has (and share KV heads between ranks)
    wide = dict(linear_num_key_heads=4, linear_num_value_heads=8, num_attention_heads=8, num_key_value_heads=2) if world > 2 else {}
    cfg = ModelConfig.tiny(num_experts=8, **wide)
    full = random_weights(cfg, seed=0, device="cpu", dtype=torch.float32, std=0.05, lm_head_std=0.5).to(dev, dtype)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(3, 1024, (n,), generator=g).tolist() for n in (20, 70, 150, 33)]
    s = Sampling(max_tokens=12, ignore_eos=True)
    ecfg = EngineConfig(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=4, mtp=False, kv_pages=128)
    ref = [x.output for x in Engine(full, ecfg).generate(prompts, s)]
    comms = {"library": DistComm(dist.group.WORLD)}
    if cuda:
        comms["fused"] = FusedComm(dev, dist.group.WORLD, slot_elems=1 << 20, max_blocks=1024)
    def note(msg):
        print(f"[rank {rank}] {msg}", file=sys.stderr, flush=True)

    note("reference engine done")
    for name, comm in comms.items():
        shard = shard_weights(full, rank, world)
        eng = Engine(shard, ecfg, tp=TPContext(rank, world, comm))
        note(f"{name}: engine built, graphs={'on' if eng._graphs is not None else 'off'}")
        got = [x.output for x in eng.generate(prompts, s)]
        note(f"{name}: generated")
        # every rank produced the same tokens
        mine = torch.tensor(got, device=dev)
        allr = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        assert all(torch.equal(allr[0], t) for t in allr), name
        same = sum(a == b for x, y in zip(got, ref) for a, b in zip(x, y))
        total = sum(len(x) for x in ref)
        if rank == 0:
            print(f"tp_model[{name}] world={world}: {same}/{total} tokens equal the unsharded engine", flush=True)
        # sharded sums are reordered: allow rare flips of near-tied tokens in bf16 (a flip changes the rest of that
        # sequence, and four-way sums flip more often than two-way ones), none in fp32
        assert same >= ((0.9 if world == 2 else 0.7) if cuda else 1.0) * total, (name, same, total)
        assert all(x[0] == y[0] for x, y in zip(got, ref)), "first tokens differ"
        if cuda:
            from b200serve.ops import cuda_ops

            cuda_ops.check_errors(dev)
    # Teacher forced: the unsharded model's tokens through the sharded model, hidden states and logits compared
    # position by position (a free-running token comparison cannot tell reordered bf16 sums from a sharding error:
    # one flipped near-tie changes the rest of that sequence). One packed prefill pass over prompt + continuation,
    # then decode steps on the caches it wrote.
    from b200serve.models.qwen36 import Model, PackedBatch
    from b200serve.ops import torch_ops

    ops = torch_ops
    if cuda:
        from b200serve.ops import cuda_ops as ops
    n = len(prompts)
    tables = torch.arange(n * 8, dtype=torch.int32).view(n, 8) + 1
    slots = list(range(1, n + 1))
    seqs = [p + o[:-4] for p, o in zip(prompts, ref)]
    for name, comm in comms.items():
        one = Model(full, num_pages=n * 8 + 1, state_slots=n + 1, ops=ops)
        tpm = Model(shard_weights(full, rank, world), num_pages=n * 8 + 1, state_slots=n + 1, ops=ops,
                    tp=TPContext(rank, world, comm))
        pairs = []
        batch = PackedBatch.prefill(seqs, slots, [0] * n, tables, dev)
        pairs.append((one.forward(batch), tpm.forward(batch)))
        for j in range(4, 1, -1):  # the held-back continuation tokens, one decode step each
            toks = [o[-j] for o in ref]
            pos = [len(p) + len(o) - j for p, o in zip(prompts, ref)]
            batch = PackedBatch.uniform(toks, pos, slots, tables, 1, dev)
            pairs.append((one.forward(batch), tpm.forward(batch)))
        h1, h2 = torch.cat([a for a, _ in pairs]), torch.cat([b for _, b in pairs])
        l1, l2 = one.logits(h1).float(), tpm.logits(h2).float()
        rel_h = ((h2.float() - h1.float()).norm() / h1.float().norm()).item()
        rel_l = ((l2 - l1).norm() / l1.norm()).item()
        top2 = l1.topk(2, dim=-1).values
        sure = (top2[:, 0] - top2[:, 1]) >= 0.5 * l1.std(dim=-1)
        hit = l1.argmax(-1) == l2.argmax(-1)
        top1, top1_sure = hit.float().mean().item(), hit[sure].float().mean().item() if bool(sure.any()) else 1.0
        if rank == 0:
            print(f"tp_model[{name} teacher-forced] world={world}: hidden rel err {rel_h:.2e}, logits rel err {rel_l:.2e}, "
                  f"top-1 {top1:.4f} ({int(sure.sum())} of {len(hit)} decided positions: {top1_sure:.4f})", flush=True)
        if cuda:
            ops.check_errors(dev)
            assert rel_h <= 0.05 and rel_l <= 0.05, (name, rel_h, rel_l)
            assert top1_sure >= 0.985, (name, top1_sure)
        else:
            assert rel_h <= 1e-4 and rel_l <= 1e-4 and top1 == 1.0, (name, rel_h, rel_l, top1)
        del one, tpm
    # MTP speculation inside the sharded replica: every rank drafts, verifies and accepts identically, and the outputs
    # stay those of plain decoding
    import dataclasses

    for name, comm in comms.items():
        eng = Engine(shard_weights(full, rank, world), dataclasses.replace(ecfg, mtp=True, spec_k=2, spec_kmax=2),
                     tp=TPContext(rank, world, comm))
        got = [x.output for x in eng.generate(prompts, s)]
        mine = torch.tensor(got, device=dev)
        allr = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        assert all(torch.equal(allr[0], t) for t in allr), name
        same = sum(a == b for x, y in zip(got, ref) for a, b in zip(x, y))
        assert eng.stats["mtp_verify_steps"] > 0
        assert same >= ((0.9 if world == 2 else 0.7) if cuda else 1.0) * sum(len(x) for x in ref), (name, same)
        if rank == 0:
            print(f"tp_model[{name} + mtp] world={world}: {same} tokens equal, {eng.stats['mtp_verify_steps']} verify steps, "
                  f"graphs={'on' if getattr(eng.spec, '_vgraphs', None) is not None else 'off'}", flush=True)
    if cuda:
        # prefill passes of >= 512 rows take the sequence-parallel kernels (GEMM -> reduce-scatter, norm + all-gather
        # push, shard-gated GEMM): same hidden states as the all-reduce path of the same sharded model
        from b200serve.models.qwen36 import Model, PackedBatch
        from b200serve.ops import cuda_ops

        shard = shard_weights(full, rank, world)
        tp = TPContext(rank, world, comms["fused"])
        model = Model(shard, num_pages=64, state_slots=4, ops=cuda_ops, tp=tp)
        lens = (300, 417)   # 717 rows: padded to a multiple of world * 128
        toks = [torch.randint(3, 1024, (n,), generator=g).tolist() for n in lens]
        tables = torch.arange(1, 17, dtype=torch.int32).view(2, 8)
        batch = PackedBatch.prefill(toks, [1, 2], [0, 0], tables, dev)
        assert model._sp(sum(lens)) is not None
        h_sp = model.forward(batch)
        state_sp = model.rec_state.clone()
        model.SP_MIN_ROWS = 1 << 30
        model.rec_state.zero_(); model.conv_state.zero_()
        h_ar = model.forward(batch)
        torch.cuda.synchronize()
        cuda_ops.check_errors(dev)
        err = (h_sp.float() - h_ar.float()).abs().max().item()
        note(f"sequence-parallel prefill vs all-reduce prefill: max err {err:.4g} (max {h_ar.float().abs().max().item():.3g})")
        assert err <= 0.05 * h_ar.float().abs().max().item() + 0.05, err
        assert (state_sp - model.rec_state).abs().max().item() < 0.05
        if rank == 0:
            print(f"tp_model[seq_parallel prefill] world={world}: max err {err:.4g}", flush=True)


def mode_pp_model(rank, world, dev):
    """Layer-split engine (each rank a run of layers) against the unsplit engine on the same requests."""
    from b200serve.config import EngineConfig, ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.parallel.pp import PPContext, layer_range, split_layers
    from b200serve.sched.engine import Engine
    from b200serve.sched.request import Sampling

    cuda = dev.type == "cuda"
    dtype = torch.bfloat16 if cuda else torch.float32
    cfg = ModelConfig.tiny(num_experts=8, num_hidden_layers=8)
    full = random_weights(cfg, seed=0, device="cpu", dtype=torch.float32, std=0.05, lm_head_std=0.5).to(dev, dtype)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(3, 1024, (n,), generator=g).tolist() for n in (20, 70, 150, 33)]
    greedy = Sampling(max_tokens=12, ignore_eos=True)
    sampled = Sampling(max_tokens=12, ignore_eos=True, temperature=0.8, top_p=0.9, seed=11)
    ecfg = EngineConfig(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=4, mtp=False, kv_pages=128)
    ref = [x.output for x in Engine(full, ecfg).generate(prompts, [greedy, greedy, sampled, greedy])]
    part = split_layers(full, rank, world)
    first, end = layer_range(8, rank, world)
    assert len(part.layers) == end - first and part.config.layer_types == cfg.layer_types[first:end]
    eng = Engine(part, ecfg, pp=PPContext(rank, world))
    assert eng._graphs is None and eng.spec is None
    got = [x.output for x in eng.generate(prompts, [greedy, greedy, sampled, greedy])]
    # a follow-up request that reuses the parked prefix: the per-rank caches stay consistent
    nxt = prompts[1] + ref[1] + [7, 8, 9]
    more = eng.generate([nxt], Sampling(max_tokens=6, ignore_eos=True))[0]
    if cuda:
        from b200serve.ops import cuda_ops

        cuda_ops.check_errors(dev)
        same = sum(a == b for x, y in zip(got, ref) for a, b in zip(x, y))
        total = sum(len(x) for x in ref)
        # same kernels, same order of operations: only the placement differs
        assert same == total, (same, total)
    else:
        assert got == ref, (got, ref)
        want = Engine(full, ecfg).generate([nxt], Sampling(max_tokens=6, ignore_eos=True))[0]
        assert more.output == want.output and more.cached_tokens > 0
    mine = torch.tensor(got, device=dev)
    allr = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(allr, mine)
    assert all(torch.equal(allr[0], t) for t in allr)
    if rank == 0:
        print(f"pp_model world={world}: tokens equal the unsplit engine on every rank (layers {first}..{end - 1} here)", flush=True)


def mode_lockstep(rank, world, dev):
    """Leader/follower replica: only rank 0 sees the requests (and a cancellation); followers mirror it."""
    from b200serve.config import EngineConfig, ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.parallel.lockstep import Coordinator
    from b200serve.parallel.tp import DistComm, TPContext, shard_weights
    from b200serve.sched.engine import Engine
    from b200serve.sched.request import Generation, Sampling

    cuda = dev.type == "cuda"
    dtype = torch.bfloat16 if cuda else torch.float32
    cfg = ModelConfig.tiny()
    full = random_weights(cfg, seed=0, device="cpu", dtype=torch.float32, std=0.05, lm_head_std=0.5).to(dev, dtype)
    ecfg = EngineConfig(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=4, mtp=False, kv_pages=128)
    cpu_group = dist.new_group(backend="gloo")
    eng = Engine(shard_weights(full, rank, world), ecfg, tp=TPContext(rank, world, DistComm(dist.group.WORLD)))
    eng.coordinator = Coordinator(cpu_group, rank)
    if rank != 0:
        eng.coordinator.follow(eng)
        assert not eng.running and not eng.prefilling
        return
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(3, 1024, (n,), generator=g).tolist() for n in (40, 90, 25)]
    samp = [Sampling(max_tokens=10, ignore_eos=True), Sampling(max_tokens=200, ignore_eos=True),
            Sampling(max_tokens=8, temperature=0.8, seed=11, ignore_eos=True)]
    gens = [eng.submit(Generation(p, s)) for p, s in zip(prompts, samp)]
    steps = 0
    while not (gens[0].done and gens[2].done):
        eng.step()
        steps += 1
        if steps == 6:
            gens[1].cancelled.set()  # a client went away mid-stream
    late = eng.submit(Generation(prompts[0] + gens[0].output + [9, 9], Sampling(max_tokens=5, ignore_eos=True)))
    while not (late.done and gens[1].done):
        eng.step()
    eng.coordinator.stop(eng)
    ref_eng = Engine(full, ecfg)
    ref = ref_eng.generate([prompts[0], prompts[2]], [samp[0], samp[2]])
    assert gens[0].output == ref[0].output and gens[2].output == ref[1].output
    assert gens[1].finish_reason == "cancelled" and 0 < len(gens[1].output) < 200
    assert late.cached_tokens > 0 and len(late.output) == 5
    print("lockstep: leader finished after", steps, "steps", flush=True)


def mode_ep_moe(rank, world, dev):
    """Expert-parallel MoE on token-sharded rows: dispatch / combine over peer memory vs the PyTorch block."""
    from b200serve.ops import cuda_ops, torch_ops
    from b200serve.parallel.ep import EpMoE

    E, H, I, k = 64, 512, 256, 4
    g = torch.Generator(device=dev).manual_seed(11)  # weights: same on every rank
    router = (torch.randn(E + 1, H, device=dev, generator=g) * 0.3).to(torch.bfloat16)
    wgu = (torch.randn(E + 1, 2 * I, H, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(E + 1, H, I, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    ep = EpMoE(dev, dist.group.WORLD, E, H, k, max_rows=2100)
    lgu, ld = ep.local_experts(wgu, wd)
    gx = torch.Generator(device=dev).manual_seed(100 + rank)  # rows: different on every rank
    # the last size: wide token tiles (the expert-sorted copy of the received rows) on a rank that receives several
    # times the rows it sends
    for T in (1, 37 + 5 * rank, 256, 0 if rank == 0 else 9, 280 if rank == 0 else 2000):
        x = torch.randn(T, H, device=dev, generator=gx).to(torch.bfloat16)
        got = ep.forward(x, router, lgu, ld)
        cuda_ops.check_errors(dev)
        if T:
            logits = cuda_ops.linear(x, router, out_dtype=torch.float32)
            wts, idx = torch_ops.router_topk(logits[:, :E], k)
            wts = torch.cat([wts, torch.sigmoid(logits[:, E:E + 1])], 1).to(torch.bfloat16)
            idx = torch.cat([idx, torch.full_like(idx[:, :1], E)], 1)
            ref = torch_ops.moe_experts(x.float(), wts.float(), idx, wgu.float(), wd.float())
            err = (got.float() - ref).abs().max().item()
            assert err <= 3e-2 * max(1.0, ref.abs().max().item()), (T, err)
    cuda_ops.check_errors(dev)
    dist.barrier()
    ep.close()


def mode_seq_parallel(rank, world, dev):
    """GEMM -> reduce-scatter, norm + all-gather push, gathered GEMM: numerics against NCCL + fp32 (the timing of the
    same pipeline against the library collectives lives in bench/collective_bench.py)."""
    from b200serve.ops import cuda_ops, torch_ops
    from b200serve.parallel.sp import SeqParallel

    H, eps = 2048, 1e-6
    sp = SeqParallel(dev, dist.group.WORLD, max_rows=8192, hidden=H)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    gc = torch.Generator(device=dev).manual_seed(7)
    for T, Ks, N2 in ((32 * world, 512, 1024), (128 * world, 2048, 4096), (1024, 1024, 12352 // world // 8 * 8)):
        rpr = T // world
        x = (torch.randn(T, Ks, device=dev, generator=g) * 0.5).to(torch.bfloat16)          # K-shard of the input
        w_o = (torch.randn(H, Ks, device=dev, generator=g) * 0.05).to(torch.bfloat16)       # K-shard of out_proj
        res = torch.randn(T, H, device=dev, generator=gc).to(torch.bfloat16)                # replicated residual
        w_n = (torch.randn(H, device=dev, generator=gc) * 0.1).to(torch.bfloat16)
        w_i = (torch.randn(N2, H, device=dev, generator=g) * 0.05).to(torch.bfloat16)       # column shard of in_proj
        for rep in range(3):
            rows = sp.gemm_reduce_scatter(x, w_o)
            mine, full = sp.reduce_norm_allgather(rows, res[rank * rpr:(rank + 1) * rpr].contiguous(), w_n, eps)
            y = sp.gemm_gathered(full, w_i)
            torch.cuda.synchronize()
            cuda_ops.check_errors(dev)
            part = x.float() @ w_o.float().t()
            dist.all_reduce(part)
            want_res = (part.to(torch.bfloat16).float() + res.float()).to(torch.bfloat16)
            got_res = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(got_res, mine)
            got_res = torch.cat(got_res)
            err = (got_res.float() - want_res.float()).abs().max().item()
            assert err <= 0.02 * want_res.float().abs().max().item() + 1e-3, ("reduce_scatter", T, rep, err)
            want_full = torch_ops.rmsnorm(got_res, w_n, eps)
            assert torch.equal(full, want_full.to(torch.bfloat16)) or \
                (full.float() - want_full.float()).abs().max().item() < 0.05, ("allgather", T, rep)
            want_y = full.float() @ w_i.float().t()
            e2 = (y.float() - want_y).abs().max().item()
            assert e2 <= 0.02 * want_y.abs().max().item() + 1e-3, ("gathered", T, rep, e2)
            dist.barrier()
    cuda_ops.check_errors(dev)
    dist.barrier()
    sp.close()


def mode_dp_ep_model(rank, world, dev):
    """Data-parallel attention + expert-parallel MoE: every rank serves its OWN requests through an engine that holds
    1 / world of the routed experts; outputs must equal the unsharded engine's on the same requests."""
    from b200serve.config import EngineConfig, ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.ops import cuda_ops
    from b200serve.parallel.ep import EpMoE, shard_experts
    from b200serve.sched.engine import Engine
    from b200serve.sched.request import Sampling

    cfg = ModelConfig.tiny(num_experts=8)
    full = random_weights(cfg, seed=0, device="cpu", dtype=torch.float32, std=0.05, lm_head_std=0.5).to(dev, torch.bfloat16)
    g = torch.Generator().manual_seed(50 + rank)  # different requests on every rank, same shapes (ranks step together)
    prompts = [torch.randint(3, 1024, (n,), generator=g).tolist() for n in (20, 70, 150, 33)]
    s = Sampling(max_tokens=12, ignore_eos=True)
    ecfg = EngineConfig(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=4, mtp=False, kv_pages=128)
    ref = [x.output for x in Engine(full, ecfg).generate(prompts, s)]
    ep = EpMoE(dev, dist.group.WORLD, cfg.num_experts, cfg.hidden_size, cfg.num_experts_per_tok, max_rows=512)
    for graphs in (False, True):
        import dataclasses

        eng = Engine(shard_experts(full, rank, world), dataclasses.replace(ecfg, cuda_graphs=graphs), ep=ep)
        got = [x.output for x in eng.generate(prompts, s)]
        cuda_ops.check_errors(dev)
        same = sum(a == b for x, y in zip(got, ref) for a, b in zip(x, y))
        total = sum(len(x) for x in ref)
        t = torch.tensor([same], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        if rank == 0:
            print(f"dp_ep_model world={world} graphs={graphs}: at least {t.item()}/{total} tokens equal the unsharded engine", flush=True)
        assert same == total, (graphs, same, total)  # the sharded MoE block is bitwise equal to the local one
        dist.barrier()
    ep.close()


MODES = {"allreduce": mode_allreduce, "ep_moe": mode_ep_moe, "tp_model": mode_tp_model, "lockstep": mode_lockstep,
         "seq_parallel": mode_seq_parallel, "dp_ep_model": mode_dp_ep_model, "pp_model": mode_pp_model}

if __name__ == "__main__":
    mode = sys.argv[1]
    rank, world, dev = setup()
    try:
        from importlib import import_module

        fn = MODES.get(mode) or getattr(import_module("dist_modes"), "mode_" + mode)
        fn(rank, world, dev)
        dist.barrier()
        if rank == 0:
            print(f"OK {mode}", flush=True)
    finally:
        dist.destroy_process_group()
