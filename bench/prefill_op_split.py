"""Where a prefill pass spends its device time: per-kernel totals of one pass of packed prompts.

    python bench/prefill_op_split.py [--seqs 8] [--len 1024] [--layers 8] [--top 22]

Random weights of the flagship architecture with ``--layers`` decoder layers (0 = all 40), tile-packed; one pass of
``--seqs`` prompts of ``--len`` tokens through ``Model.forward``. Prints one JSON line with the pass time (CUDA
events, median of 3 after 2 warm-up passes) and the prefill rate scaled to 40 layers, then the kernels of one
pass by total device time (torch profiler, CUDA activities only; run with ``ENGINE_PDL=0`` so that durations of
neighbouring kernels do not overlap). Reference: ``tools/prefill_op_split.py``."""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
from pathlib import Path

os.environ.setdefault("ENGINE_PDL", "0")
sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--seqs", type=int, default=8)
    ap.add_argument("--len", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--top", type=int, default=22)
    args = ap.parse_args()

    from torch.profiler import ProfilerActivity, profile

    from b200serve.config import ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.models.qwen36 import Model, PackedBatch
    from b200serve.ops import cuda_ops

    dev = torch.device("cuda")
    cfg = ModelConfig(**({"num_hidden_layers": args.layers} if args.layers else {}))
    w = random_weights(cfg, seed=0, device=dev, dtype=torch.bfloat16)
    cuda_ops.pack_weights(w)
    S, L = args.seqs, args.len
    per_seq = L // 64 + 2
    model = Model(w, num_pages=S * per_seq + 1, state_slots=S + 1, ops=cuda_ops)
    tables = torch.arange(S * per_seq, dtype=torch.int32).view(S, per_seq) + 1
    g = torch.Generator().manual_seed(0)
    toks = [torch.randint(3, cfg.vocab_size, (L,), generator=g).tolist() for _ in range(S)]
    batch = PackedBatch.prefill(toks, list(range(1, S + 1)), [0] * S, tables, dev)
    for _ in range(2):
        model.forward(batch)
    torch.cuda.synchronize()
    cuda_ops.check_errors(dev)
    times = []
    for _ in range(3):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        model.forward(batch)
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    ms = statistics.median(times)
    layers = cfg.num_hidden_layers
    print(json.dumps({"seqs": S, "len": L, "layers": layers, "ms_per_pass": round(ms, 3),
                      "tok_s_scaled_to_40_layers": round(S * L / (ms * 40 / layers) * 1e3)}), flush=True)
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        model.forward(batch)
        torch.cuda.synchronize()
    cuda_ops.check_errors(dev)
    rows = sorted(prof.key_averages(), key=lambda r: -r.device_time_total)
    total = sum(r.device_time_total for r in rows) or 1.0
    for r in rows[: args.top]:
        print(f"{r.device_time_total:10.1f} us {100 * r.device_time_total / total:5.1f} % {r.count:5d} x  {r.key[:110]}")


if __name__ == "__main__":
    main()
