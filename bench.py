"""Headline benchmark: decode throughput of Qwen3.6-35B-A3B (bf16, random init) on N B200s.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched by torch.distributed.run)

Config: every GPU serves ``--batch`` concurrent requests with ``--prompt-len`` uniform-random
prompt tokens (greedy, ignore_eos); a *step* is one decode iteration of the engine, i.e. one
new token for every running request. ``value`` is the whole-job output tokens/s over exactly K
steps timed on the device with CUDA events (max over ranks). ``e2e`` is the same K steps driven
through the public engine API (``Engine.submit`` / ``Engine.step``): each step copies its inputs
from pinned host memory to the device and reads the sampled tokens back.

On several GPUs every rank serves its own ``--batch`` requests (weak scaling). ``--parallelism``: ``dp`` = independent
replicas with all weights on every GPU; ``dp_ep`` (what ``auto`` picks for N > 1) = data-parallel attention / GDN with
expert-parallel MoE: each GPU holds 1 / N of the routed experts and the rows of all ranks meet their experts through the
fused dispatch / combine kernels over NVLink peer memory, so the expert weights streamed per GPU and step shrink with N;
``tp_ep`` = ONE tensor + expert parallel replica over all GPUs serving one batch (strong scaling).

With ``--impl reference`` the unmodified reference under ``baseline/_ref`` is run for the same
metric, or a one-line reason is printed when it cannot run in this image.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

BASELINE_TOK_S = None  # the reference publishes no number for this hardware


def parse() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=128, help="concurrent requests per GPU")
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--kernel-table", action="store_true",
                    help="after the timed run, replay a few steps under the CUDA activity profiler on rank 0 and print "
                         "per-kernel device time per step to stderr")
    ap.add_argument("--parallelism", default="auto", choices=["auto", "dp", "tp_ep", "dp_ep"],
                    help="auto: one GPU -> dp; several -> dp_ep (data-parallel attention, expert-parallel MoE over NVLink "
                         "peer memory), falling back to independent dp replicas if its set-up or trial step fails")
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (result marked invalid)")
    ap.add_argument("--mtp", type=int, default=0, help="MTP draft depth (0 = plain decode)")
    ap.add_argument("--no-serving-config", action="store_true",
                    help="skip the second measurement (256 concurrent requests in total, 2048-token prompts, 256 output "
                         "tokens, prefill included), reported under the key 'serving_256x2048x256'")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


REF_ENV = {
    # what the reference needs to start on a CUDA machine (its defaults assume two MI250 GCDs per replica):
    "ENGINE_TP": "1",            # its TP all-reduce loads libamdhip64.so (engine/fast/tp.py:341-343, 517-518)
    "ENGINE_GDN_HIP": "0",       # its served GDN kernel is compiled with hipRTC (engine/fast/gdn_hip.py:163)
    "ENGINE_MTP": "0",           # plain decode, as the other arm measures
}


def reference_unavailable() -> str | None:
    """Why the unmodified reference under baseline/_ref cannot run here, or None when it can be tried."""
    import importlib.util

    if not (ROOT / "baseline" / "_ref" / "engine").exists():
        return ("reference is not pip-installable (no setup.py/pyproject.toml) and baseline/_ref/engine "
                "is absent on this box")
    if importlib.util.find_spec("accelerate") is None:
        return ("reference Generator.load calls from_pretrained(device_map='auto') on CUDA "
                "(engine/generator.py:651-663), which needs the accelerate package: not in this image "
                "nor in /opt/wheelhouse")
    return None


def reference_arm(args: argparse.Namespace) -> None:
    """The same metric through the reference's own public API (`Generator.load / start_many / decode`,
    engine/generator.py:636, 766, 1026), stock code path, none of this repository's kernels or engine on it."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    why = reference_unavailable()
    if why is not None:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return
    try:
        line = _reference_run(args, rank, world)
    except Exception as e:  # noqa: BLE001 - the arm must always print one line and exit 0
        import traceback

        tb = traceback.extract_tb(e.__traceback__)[-1]
        line = {"impl": "reference", "unavailable": f"reference run failed at {Path(tb.filename).name}:{tb.lineno}: {e!r}"[:400]}
    if rank == 0 and line is not None:
        print(json.dumps(line), flush=True)


def _reference_run(args: argparse.Namespace, rank: int, world: int) -> dict | None:
    import tempfile

    import torch
    import torch.distributed as dist

    os.environ.update({k: os.environ.get(k, v) for k, v in REF_ENV.items()})
    B, P, K, W = args.batch, args.prompt_len, args.steps, max(args.warmup, 3)
    os.environ.setdefault("ENGINE_SLOTS", str(B))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ["CUDA_VISIBLE_DEVICES"] = os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",")[local] \
        if os.environ.get("CUDA_VISIBLE_DEVICES") else str(local)  # one GPU per rank: a data-parallel replica each
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    # a random-init checkpoint of the named architecture in HF layout, written by this repository's checkpoint writer
    # (the only part of this repository the arm uses; it is input data, not on the timed path)
    from b200serve.config import ModelConfig
    from b200serve.models.checkpoint import random_weights, save_checkpoint
    from b200serve.models.tiny import build_tokenizer

    ckpt = Path(os.environ.get("BENCH_REF_CKPT") or tempfile.mkdtemp(prefix=f"ref-ckpt-{rank}-"))
    if not (ckpt / "config.json").exists():
        mcfg = ModelConfig.qwen36_35b_a3b()
        save_checkpoint(random_weights(mcfg, seed=1234 + rank, device="cpu", dtype=torch.bfloat16), ckpt)
        build_tokenizer(512).save_pretrained(str(ckpt))
    sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
    from engine.generator import Generator
    from engine.protocol import Sampling

    total_out = K + W + 8
    gen = Generator.load(str(ckpt), None, max_model_len=P + total_out + 64, chunk_tokens=2048,
                         prefix_cache_tokens=0, prefix_cache_entries=0)
    vocab = gen.model.config.get_text_config().vocab_size
    g = torch.Generator().manual_seed(99 + rank)
    reqs = [(tuple(torch.randint(0, vocab, (P,), generator=g).tolist()),
             Sampling(max_tokens=total_out, temperature=0.0, ignore_eos=True)) for _ in range(B)]
    gens = gen.start_many(reqs)
    bad = [x for x in gens if isinstance(x, Exception)]
    if bad:
        raise bad[0]

    def step() -> None:
        for x in gens:
            x.next_step()  # picks the token from the stored logits (a device-to-host read per request)
        gen.decode(gens)

    for _ in range(W):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    a.record()
    for _ in range(K):
        step()
    b.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ms = a.elapsed_time(b)
    if world > 1:
        t = torch.tensor([ms, wall], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, wall = float(t[0]), float(t[1])
        dist.destroy_process_group()
    value = world * B * K / (ms / 1e3)
    return {
        "metric": "output tok/s (whole box, max over ranks), decode", "value": round(value, 1), "unit": "tok/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (uniform-random prompt tokens, random-init weights)", "impl": "reference",
        "config": {"model": "Qwen3.6-35B-A3B", "global_batch": B * world, "seq_len": P, "parallelism": f"dp{world}",
                   "flags": {k: os.environ[k] for k in list(REF_ENV) + ["ENGINE_SLOTS"]}},
        "e2e": {"value": round(world * B * K / wall, 1), "unit": "tok/s",
                "note": "the reference's step reads every request's token on the host; same loop as the timed one"},
    }


def main() -> None:
    args = parse()
    if args.impl == "reference":
        reference_arm(args)
        return
    import torch
    import torch.distributed as dist

    from b200serve.config import EngineConfig, ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.ops import cuda_ops
    from b200serve.sched.engine import Engine
    from b200serve.sched.request import Generation, Sampling

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # NCCL only carries barriers and a few scalars here; keep it off NVLink multicast objects so that a rank that
        # dies cannot fault its peers' GPUs through a bound multicast mapping
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    B, P, K, W = args.batch, args.prompt_len, args.steps, args.warmup

    mcfg = ModelConfig.qwen36_35b_a3b() if not args.layers else ModelConfig(num_hidden_layers=args.layers)
    mode = args.parallelism
    if mode == "auto":
        mode = "dp_ep" if world > 1 else "dp"
    tp_mode = mode == "tp_ep" and world > 1
    ep_mode = mode == "dp_ep" and world > 1
    tp_ctx = ep_ctx = None
    if tp_mode:  # one replica over all ranks: same weights and the same requests everywhere, sharded TP + EP
        from b200serve.parallel.tp import FusedComm, TPContext, shard_weights

        full = random_weights(mcfg, seed=1234, device=dev, dtype=torch.bfloat16)
        weights = shard_weights(full, rank, world)
        del full
        torch.cuda.empty_cache()
        tp_ctx = TPContext(rank, world, FusedComm(dev, dist.group.WORLD, slot_elems=1 << 21, max_blocks=4096))
    elif ep_mode:
        # data-parallel attention + expert-parallel MoE: every rank serves its own B requests with full dense weights
        # and 1 / world of the routed experts; rows travel to their experts and back inside every MoE block
        # (parallel/ep.py). All ranks run identical schedules here, so their forward passes pair up.
        from b200serve.parallel.ep import EpMoE, shard_experts

        full = random_weights(mcfg, seed=1234, device=dev, dtype=torch.bfloat16)
        weights = shard_experts(full, rank, world)
        del full
        torch.cuda.empty_cache()
        ep_ctx = EpMoE(dev, dist.group.WORLD, mcfg.num_experts, mcfg.hidden_size, mcfg.num_experts_per_tok, max_rows=8192,
                       wait_s=5.0)  # the ranks step on their own clocks in the serving workload
    else:
        weights = random_weights(mcfg, seed=1234 + rank, device=dev, dtype=torch.bfloat16)
    total_out = K + max(W, 3) + 64 + (B * P) // 4096  # room for the tokens decoded while later prompts prefill
    # second workload: 256 concurrent requests over the whole job, 2048-token prompts, 256 output tokens
    S_REQ, S_PROMPT, S_OUT = 256, 2048, 256
    serving = not args.no_serving_config and not args.layers and not args.mtp
    n_serv = (S_REQ if tp_mode else S_REQ // world) if serving else 0
    seqs = max(B, n_serv)
    pages = max(B * ((P + 2 * total_out) // 64 + 2), n_serv * ((S_PROMPT + S_OUT) // 64 + 3)) + 2
    ecfg = EngineConfig(
        max_model_len=max(P + 2 * total_out + 64, S_PROMPT + S_OUT + 64), max_seqs=seqs, state_slots=seqs + 2,
        prefill_chunk_tokens=2048, prefill_pack_tokens=8192, kv_pages=pages, mtp=bool(args.mtp),
        spec_k=args.mtp, decode_buckets=tuple(sorted({B, seqs})), pack_weights=not tp_mode,
    )
    if ep_mode:
        ecfg.mtp = False
    engine = Engine(weights, ecfg, tp=tp_ctx, ep=ep_ctx)
    replicas = 1 if tp_mode else world  # independent request streams in the job

    def all_ranks_ok(ok: bool) -> bool:
        t = torch.tensor([0 if ok else 1], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() == 0

    if ep_mode and args.parallelism == "auto":
        # trial: one short request through prefill and a few decode steps on every rank; any failure anywhere (a
        # bounded wait that ran out, an allocation) sends every rank to independent replicas instead
        ok = True
        try:
            trial = engine.generate([[1 + ((i * (j + 3)) % 997) for i in range(200)] for j in range(8)],
                                    Sampling(max_tokens=4, ignore_eos=True))
            cuda_ops.check_errors(dev)
            ok = all(t.done and len(t.output) == 4 for t in trial)
            if os.environ.get("BENCH_FAIL_EP_TRIAL") == str(rank):  # exercises the fallback below
                raise RuntimeError("trial failure requested")
        except Exception as e:  # noqa: BLE001
            print(f"bench: dp_ep trial failed on rank {rank}: {e!r}", file=sys.stderr, flush=True)
            ok = False
        if not all_ranks_ok(ok):
            if rank == 0:
                print("bench: falling back to independent data-parallel replicas", file=sys.stderr, flush=True)
            try:
                cuda_ops.err_word(dev).zero_()
            except Exception:  # noqa: BLE001
                pass
            try:
                ep_ctx.close()
            except Exception:  # noqa: BLE001
                pass
            del engine, weights, ep_ctx
            import gc

            gc.collect()
            torch.cuda.empty_cache()
            mode, ep_mode, ep_ctx = "dp", False, None
            weights = random_weights(mcfg, seed=1234 + rank, device=dev, dtype=torch.bfloat16)
            engine = Engine(weights, ecfg)

    def run_phase(timed_steps: int, warm: int, e2e: bool, table: bool = False):
        """Prefill B fresh requests, run `warm` untimed decode steps, then time `timed_steps` steps. With `table`,
        the replays are recorded with the CUDA activity profiler and rank 0 prints per-kernel time per step to stderr
        (a diagnostic: numbers of such a pass are never reported as the bench value; with programmatic dependent
        launch a kernel's duration includes its wait for the kernel before it, ENGINE_PDL=0 gives plain durations)."""
        engine.cache.clear()
        g = torch.Generator().manual_seed(99 + (0 if tp_mode else rank) + (1000 if e2e else 0))
        gens = [
            engine.submit(Generation(torch.randint(0, mcfg.vocab_size, (P,), generator=g).tolist(),
                                     Sampling(max_tokens=total_out, ignore_eos=True)))
            for _ in range(B)
        ]
        t_limit = time.perf_counter() + 600.0
        while engine.prefilling or engine.waiting or not engine._inbox.empty():
            engine.step()  # prefill passes (each also advances already-running requests by one token)
            if engine.stats["device_errors"] or engine.broken or time.perf_counter() > t_limit:
                raise RuntimeError(f"prefill phase did not complete: device_errors={engine.stats['device_errors']}, "
                                   f"broken={engine.broken}")
        if not e2e:  # the device-resident loop runs ahead of the host: give every request its pages now
            for x in gens:
                engine._ensure_pages(x, x.computed + timed_steps + 2)
        for _ in range(warm):
            engine.step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        produced0 = sum(len(x.output) for x in gens)
        t0 = time.perf_counter()
        prof = None
        if table:  # every rank records (the ranks wait on one another: all of them must run equally slowed)
            from torch.profiler import ProfilerActivity, profile

            prof = profile(activities=[ProfilerActivity.CUDA])
            prof.__enter__()
        start.record()
        if e2e:
            for _ in range(timed_steps):
                engine.step()
        else:
            bucket = next((b for b in engine._graphs.buckets.values() if b.size == B), None)
            if bucket is None:
                raise RuntimeError(f"no captured decode graph for batch {B}: {engine._graphs.errors}")
            for _ in range(timed_steps):
                bucket.graph.replay()
                bucket.tokens.copy_(bucket.picks)  # feed the picks back on the device
                bucket.positions.add_(1)
        end.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        if prof is not None:
            prof.__exit__(None, None, None)
        if prof is not None and rank == 0:
            rows = sorted(prof.key_averages(), key=lambda r: -r.device_time_total)
            print(f"per-kernel device time per step over {timed_steps} replays (rank 0):", file=sys.stderr)
            for r in rows[:40]:
                print(f"  {r.device_time_total / timed_steps:9.1f} us  {r.count / timed_steps:6.1f} launches  {r.key[:110]}",
                      file=sys.stderr)
            sys.stderr.flush()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
        produced = sum(len(x.output) for x in gens) - produced0 if e2e else timed_steps * B
        for x in gens:
            x.cancelled.set()
        engine.step()
        return ms, wall, produced

    def run_serving():
        """All requests of the second workload arrive at once on every replica; timed from submission to the last
        token through the public engine API (prefill included), wall clock around a device synchronise."""
        engine.cache.clear()
        g = torch.Generator().manual_seed(7 + (0 if tp_mode else rank))
        first, last = {}, {}

        def on_event(gen, ev):
            if ev.token is not None:
                now = time.perf_counter()
                first.setdefault(gen.id, now)
                last[gen.id] = now

        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        gens = [engine.submit(Generation(torch.randint(0, mcfg.vocab_size, (S_PROMPT,), generator=g).tolist(),
                                         Sampling(max_tokens=S_OUT, ignore_eos=True), on_event=on_event))
                for _ in range(n_serv)]
        t_limit = time.perf_counter() + 900.0
        while any(not x.done for x in gens):
            engine.step()
            if engine.broken or time.perf_counter() > t_limit:
                raise RuntimeError(f"serving workload did not complete: broken={engine.broken}")
        engine.flush_events()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        ok = all(len(x.output) == S_OUT for x in gens)
        ttft = sorted(first[x.id] - t0 for x in gens)
        tpot = sorted((last[x.id] - first[x.id]) / (S_OUT - 1) for x in gens)
        return wall, ok, ttft[len(ttft) // 2] * 1e3, tpot[len(tpot) // 2] * 1e3

    sampler = ClockSampler(local)
    # e2e first (through the public API), then the device-resident kernel loop on the same engine. The headline e2e
    # number copies every step's inputs from pinned host memory (run-ahead off); with run-ahead, the engine's default,
    # a step's tokens and positions are built on the device from the step before and only page-table growth is
    # copied, which is reported beside it.
    engine.cfg.run_ahead = False
    e2e_ms, e2e_wall, e2e_tokens = run_phase(K, W, e2e=True)
    engine.cfg.run_ahead = True
    ra_ms, ra_wall, ra_tokens = run_phase(K, W, e2e=True)
    launches_per_step = None
    sampler.start()
    ms, _wall, tokens = run_phase(K, max(W, 3), e2e=False)
    clocks = sampler.stop()
    cuda_ops.check_errors(dev)
    if args.kernel_table:
        run_phase(min(K, 5), 3, e2e=False, table=True)
        cuda_ops.check_errors(dev)
    serving_line = None
    if serving:
        s_wall, s_ok, s_ttft, s_tpot = run_serving()
        cuda_ops.check_errors(dev)

    def reduce_max(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if serving:
        s_wall = reduce_max(s_wall)
        s_bad = reduce_max(0.0 if s_ok else 1.0)
        serving_line = {
            "value": round(S_REQ * S_OUT / s_wall, 1), "unit": "output tok/s, prefill included", "wall_s": round(s_wall, 3),
            "ttft_p50_ms": round(reduce_max(s_ttft), 1), "tpot_p50_ms": round(reduce_max(s_tpot), 2),
            "complete": s_bad == 0.0,
            "config": {"requests": S_REQ, "prompt_len": S_PROMPT, "output_len": S_OUT, "requests_per_gpu": n_serv,
                       "arrival": "all at once", "timing": "wall clock around a device synchronise, max over ranks; "
                       "TTFT / TPOT are each rank's medians, the slowest rank reported"},
        }
    ms = reduce_max(ms)
    e2e_s = reduce_max(max(e2e_wall, e2e_ms / 1e3))
    ra_s = reduce_max(max(ra_wall, ra_ms / 1e3))
    value = replicas * tokens / (ms / 1e3)
    e2e_value = replicas * e2e_tokens / e2e_s
    bucket = next(b for b in engine._graphs.buckets.values() if b.size == B)
    h2d = bucket.host_buf.numel()  # tokens, positions, slots and page tables: one pinned buffer, one copy per step
    d2h = bucket.h_picks.numel() * 8
    # kernels of this library inside one replay of the captured decode step, counted by its launchers at capture
    launches_per_step = bucket.launches
    if rank == 0:
        line = {
            "metric": "output tok/s (whole box, max over ranks), decode", "value": round(value, 1), "unit": "tok/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 4), "higher_is_better": True,
            "scaling": "strong" if tp_mode else "weak", "vs_baseline": None if BASELINE_TOK_S is None else value / BASELINE_TOK_S,
            "dtype": "bf16", "data": "synthetic (uniform-random prompt tokens, random-init weights)",
            "impl": "ours",
            "config": {
                "model": "Qwen3.6-35B-A3B" + (f"[{args.layers} layers: INVALID]" if args.layers else ""),
                "global_batch": B * replicas, "seq_len": P, "parallelism": f"{mode}{world}",
                "batch_per_gpu": B, "l2": "working set per step (weights + KV + GDN state) far exceeds the 126 MB L2",
                "mtp_depth": args.mtp,
            },
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_s * 1e3 / K, 4),
                    "with_run_ahead": {"value": round(replicas * ra_tokens / ra_s, 1), "ahead_steps": engine.stats["ahead_steps"],
                                       "note": "engine default: step n + 1 launched from device-built inputs before "
                                               "step n is read; H2D only when a page table grows"}},
            "gpu_launches": launches_per_step * K,
            "gpu_launches_note": "kernels of this library inside the timed region (counted at graph capture, times "
                                 "steps); torch adds two elementwise launches per step to feed the picks back",
        }
        if serving_line is not None:
            line["serving_256x2048x256"] = serving_line
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
