"""MTP speculative decoding through the engine: output tok/s, step count and acceptance by draft depth.

    python bench/mtp_bench.py [--batches 1,8,64] [--depths 0,1,2,3] [--prompt-len 4096] [--output-len 256] [--draft-ivf 4096]

Random-init Qwen3.6-35B-A3B (``--tiny`` for the CPU-sized model), synthetic prompts, greedy, exact output length.
Depth 0 is plain decoding. With random weights the draft head agrees with the model only by chance, so the
acceptance column is a floor, not what a trained checkpoint gives; the point of this benchmark is the cost of a
verify step of k+1 rows per sequence against a plain step (the reference tabulates the same cost per
(slot bucket, k), ``engine/speculative.py:134-136``, and measures acceptance with ``tools/chain_gate.py``).
One JSON line per (depth, batch): wall-clock of the decode phase (prompt passes excluded) after a warm-up run.
"""

from __future__ import annotations

import argparse
import gc
import json
import sys
import time
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from b200serve.config import EngineConfig, ModelConfig  # noqa: E402
from b200serve.models.checkpoint import random_weights  # noqa: E402
from b200serve.sched.engine import Engine  # noqa: E402
from b200serve.sched.request import Generation, Sampling  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batches", default="1,8,64")
    ap.add_argument("--depths", default="0,1,2,3")
    ap.add_argument("--prompt-len", type=int, default=4096)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--draft-ivf", type=int, default=0,
                    help="clusters of the vocabulary shortlist index for draft picks (0: drafts read the whole LM head)")
    a = ap.parse_args()
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda" if cuda else "cpu")
    cfg = ModelConfig.tiny() if a.tiny else ModelConfig()
    w = random_weights(cfg, seed=0, device=dev, dtype=torch.bfloat16 if cuda else torch.float32)
    batches = [int(x) for x in a.batches.split(",")]
    g = torch.Generator().manual_seed(0)
    for depth in [int(x) for x in a.depths.split(",")]:
        ecfg = EngineConfig(max_model_len=a.prompt_len + a.output_len + 64, max_seqs=max(batches), mtp=depth > 0,
                            spec_k=depth, spec_kmax=max(depth, 1), prefix_cache_entries=0, draft_ivf=a.draft_ivf)
        eng = Engine(w, ecfg)
        for B in batches:
            prompts = [torch.randint(3, cfg.vocab_size, (a.prompt_len,), generator=g).tolist() for _ in range(B)]
            eng.generate(prompts, Sampling(max_tokens=6, ignore_eos=True))  # warm-up: captures this batch size's graphs
            outs = [eng.submit(Generation(p, Sampling(max_tokens=a.output_len, ignore_eos=True))) for p in prompts]
            while eng.prefilling or eng.waiting or not eng._inbox.empty():
                eng.step()  # prompt passes are not part of the timed region
            if cuda:
                torch.cuda.synchronize()
            before = dict(eng.stats)
            done0 = sum(len(o.output) for o in outs)
            steps = 0
            t0 = time.perf_counter()
            while any(not o.done for o in outs):
                eng.step()
                steps += 1
            if cuda:
                torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            st = {k: eng.stats[k] - before.get(k, 0) for k in ("mtp_verify_steps", "mtp_proposed", "mtp_accepted") if k in eng.stats}
            n = sum(len(o.output) for o in outs) - done0
            print(json.dumps({"bench": "mtp", "depth": depth, "batch": B, "prompt_len": a.prompt_len, "output_tokens": n,
                              "decode_s": round(dt, 3), "ms_per_step": round(dt / max(steps, 1) * 1e3, 2), "output_tok_s": round(n / dt, 1), **st,
                              "acceptance": round(st["mtp_accepted"] / st["mtp_proposed"], 4) if st.get("mtp_proposed") else None}),
                  flush=True)
        del eng
        gc.collect()  # engine, controller and captured graphs reference each other
        if cuda:
            torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
