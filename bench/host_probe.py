"""Where the host's time goes, without a GPU: three probes of the serving path's CPU-side parts.

    python bench/host_probe.py tokenize --model DIR [--rounds 8] [--turn-chars 1500] [--sessions 16]
    python bench/host_probe.py kv-pool [--sessions 64] [--prompt-tokens 4096] [--rounds 6]
    python bench/host_probe.py cpu-place [--replicas 4] [--gpus-per-replica 2]

``tokenize``: multi-round sessions whose prompt grows by one turn per round, encoded with the incremental
encoder (``api/tokenizer.py`` ``PromptEncoder``: re-encodes only the text after the longest cached prefix) and
by full encodes; ms per request both ways, and whether the ids agree (reference: ``tools/tokenize_bench.py``).
``kv-pool``: the page pool, the slot pool and the prefix / session-tail cache driven the way the engine drives
them for multi-round sessions (claim, grow by pages, store the tail, look the next turn up); microseconds per
operation and the hit rate (reference: ``tools/kv_pool_probe.py``).
``cpu-place``: the CPU slices and per-rank CPUs that the data-parallel front would give each replica on this
machine (reference: ``tools/cpu_place_probe.py``).
Each probe prints one JSON line."""

from __future__ import annotations

import argparse
import json
import random
import statistics
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

WORDS = ("state cache token page slot router expert draft verify graph kernel stream copy span chunk prompt answer "
         "session round latency batch decode prefill window table index value weight layer norm gate").split()


def _turn(rng: random.Random, chars: int) -> str:
    out, n = [], 0
    while n < chars:
        w = rng.choice(WORDS)
        out.append(w)
        n += len(w) + 1
    return " ".join(out) + ".\n"


def probe_tokenize(args) -> dict:
    from b200serve.api.tokenizer import PromptEncoder, TextCodec

    codec = TextCodec(args.model)
    backend = getattr(codec.tok, "backend_tokenizer", None)
    if backend is None:
        raise SystemExit("this tokenizer has no offset-giving backend: the incremental encoder does not apply")
    inc = PromptEncoder(backend, capacity=4 * args.sessions)
    rng = random.Random(0)
    texts = ["<|im_start|>user\n" + _turn(rng, args.turn_chars) for _ in range(args.sessions)]
    t_inc, t_full, same, total_ids = [], [], True, 0
    for _ in range(args.rounds):
        for s in range(args.sessions):
            texts[s] += "<|im_start|>assistant\n" + _turn(rng, args.turn_chars // 3) + "<|im_start|>user\n" + _turn(rng, args.turn_chars)
            t0 = time.perf_counter()
            a = inc.encode(texts[s])
            t1 = time.perf_counter()
            b = backend.encode(texts[s], add_special_tokens=False).ids
            t2 = time.perf_counter()
            t_inc.append((t1 - t0) * 1e3)
            t_full.append((t2 - t1) * 1e3)
            same = same and a == list(b)
            total_ids += len(b)
    return {"probe": "tokenize", "requests": len(t_inc), "mean_prompt_tokens": total_ids // len(t_inc),
            "incremental_ms_median": round(statistics.median(t_inc), 3), "full_ms_median": round(statistics.median(t_full), 3),
            "incremental_ms_last_round": round(statistics.median(t_inc[-args.sessions:]), 3),
            "full_ms_last_round": round(statistics.median(t_full[-args.sessions:]), 3),
            "reused_chars": inc.stats["tokenize_reused_chars"], "encoded_chars": inc.stats["tokenize_encoded_chars"],
            "ids_equal": same}


def probe_kv_pool(args) -> dict:
    from b200serve.cache.pools import PagePool, SlotPool
    from b200serve.config import PAGE_SIZE
    from b200serve.cache.prefix import PrefixCache

    rng = random.Random(0)
    per_session = (args.prompt_tokens + args.rounds * (args.turn_tokens + args.out_tokens)) // PAGE_SIZE + 2
    cache_box = []
    pages = PagePool(args.sessions * per_session * 2 + 1, on_pressure=lambda: cache_box[0].evict_one())
    slots = SlotPool(2 * args.sessions + 1, on_pressure=lambda: cache_box[0].evict_one())
    cache = PrefixCache(pages, slots, page_bytes=1 << 16, slot_bytes=1 << 21, max_entries=4 * args.sessions)
    cache_box.append(cache)
    prompts = [[rng.randrange(3, 150000) for _ in range(args.prompt_tokens)] for _ in range(args.sessions)]
    t = {"lookup": [], "alloc": [], "store_tail": []}
    hits = cached = asked = 0
    for _ in range(args.rounds):
        for s in range(args.sessions):
            p = prompts[s]
            t0 = time.perf_counter()
            e = cache.lookup(p)
            t["lookup"].append(time.perf_counter() - t0)
            asked += len(p)
            if e is not None and e.kind == "tail":
                slot, mine, have = e.slot, list(e.pages), e.length
                hits += 1
                cached += have
            else:
                slot, mine, have = slots.alloc(), [], 0
            total = len(p) + args.out_tokens
            t0 = time.perf_counter()
            need = (total + PAGE_SIZE - 1) // PAGE_SIZE - len(mine)
            if need > 0:
                mine.extend(pages.alloc(need))
            t["alloc"].append(time.perf_counter() - t0)
            done = p + [rng.randrange(3, 150000) for _ in range(args.out_tokens)]
            t0 = time.perf_counter()
            cache.store_tail(done, mine, slot)
            t["store_tail"].append(time.perf_counter() - t0)
            prompts[s] = done + [rng.randrange(3, 150000) for _ in range(args.turn_tokens)]
    us = {k: round(statistics.median(v) * 1e6, 1) for k, v in t.items()}
    return {"probe": "kv-pool", "sessions": args.sessions, "rounds": args.rounds, "final_prompt_tokens": len(prompts[0]),
            "lookup_us": us["lookup"], "page_alloc_us": us["alloc"], "store_tail_us": us["store_tail"],
            "tail_hit_rate": round(hits / (args.sessions * args.rounds), 3), "cached_token_share": round(cached / asked, 3),
            "pages_used": pages.used, "entries": len(cache)}


def probe_cpu_place(args) -> dict:
    from b200serve.router.cpu_place import Topology, format_cpu_list, gpu_bdfs, replica_slices, thread_caps

    topo = Topology.read(gpu_bdfs=gpu_bdfs())
    replicas = [[r * args.gpus_per_replica + j for j in range(args.gpus_per_replica)] for r in range(args.replicas)]
    plan = replica_slices(topo, replicas)
    return {"probe": "cpu-place", "allowed_cpus": format_cpu_list(sorted(topo.allowed)), "physical_cores": len(topo.physical_cores()),
            "gpu_numa_nodes": list(topo.gpu_nodes),
            "replicas": [{"gpus": g, "cpus": format_cpu_list(p.cpus), "rank_cpus": p.rank_cpus, "env": thread_caps(len(p.cpus))}
                         for g, p in zip(replicas, plan)]}


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="probe", required=True)
    p = sub.add_parser("tokenize")
    p.add_argument("--model", required=True)
    p.add_argument("--rounds", type=int, default=8)
    p.add_argument("--turn-chars", type=int, default=1500)
    p.add_argument("--sessions", type=int, default=16)
    p = sub.add_parser("kv-pool")
    p.add_argument("--sessions", type=int, default=64)
    p.add_argument("--prompt-tokens", type=int, default=4096)
    p.add_argument("--turn-tokens", type=int, default=300)
    p.add_argument("--out-tokens", type=int, default=200)
    p.add_argument("--rounds", type=int, default=6)
    p = sub.add_parser("cpu-place")
    p.add_argument("--replicas", type=int, default=4)
    p.add_argument("--gpus-per-replica", type=int, default=2)
    args = ap.parse_args(argv)
    out = {"tokenize": probe_tokenize, "kv-pool": probe_kv_pool, "cpu-place": probe_cpu_place}[args.probe](args)
    print(json.dumps(out), flush=True)
    return out


if __name__ == "__main__":
    main()
