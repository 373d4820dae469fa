"""Prefill pass of the tensor + expert parallel model: fused sequence-parallel kernels against library collectives.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29700 \
        bench/tp_prefill_bench.py [--layers 8] [--seqs 8] [--len 1024]

Every rank holds its shard of a random-init Qwen3.6-35B-A3B (``--layers`` of its 40 layers, to bound memory) and
runs the same packed prefill pass twice: with the row-sharded residual stream of ``parallel/sp.py`` (GEMM ->
reduce-scatter epilogue, RMSNorm + all-gather push, shard-gated GEMM) and with one all-reduce per projection
(NCCL at this size). Device-timed with CUDA events, max over ranks; prints one JSON line from rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--seqs", type=int, default=8)
    ap.add_argument("--len", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from b200serve.config import ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.models.qwen36 import Model, PackedBatch
    from b200serve.ops import cuda_ops
    from b200serve.parallel.tp import FusedComm, TPContext, shard_weights

    cfg = ModelConfig(num_hidden_layers=a.layers)
    full = random_weights(cfg, seed=0, device=dev, dtype=torch.bfloat16)
    shard = shard_weights(full, rank, world)
    del full
    torch.cuda.empty_cache()
    pp = a.len // 64 + 2
    model = Model(shard, num_pages=a.seqs * pp + 1, state_slots=a.seqs + 1, ops=cuda_ops,
                  tp=TPContext(rank, world, FusedComm(dev, dist.group.WORLD)))
    g = torch.Generator().manual_seed(1)
    toks = [torch.randint(0, cfg.vocab_size, (a.len,), generator=g).tolist() for _ in range(a.seqs)]
    tables = torch.arange(a.seqs * pp, dtype=torch.int32).view(a.seqs, pp) + 1
    batch = PackedBatch.prefill(toks, list(range(1, a.seqs + 1)), [0] * a.seqs, tables, dev)
    out = {}
    for name, min_rows in (("seq_parallel_fused", 512), ("allreduce_library", 1 << 30)):
        model.SP_MIN_ROWS = min_rows
        for _ in range(2):
            model.forward(batch)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            model.forward(batch)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name] = round(t.item(), 3)
    cuda_ops.check_errors(dev)
    if rank == 0:
        T = a.seqs * a.len
        print(json.dumps({"bench": "tp_prefill", "world": world, "layers": a.layers, "rows": T, "ms": out,
                          "tok_s_40_layers": {k: round(T / (v / a.layers * 40) * 1e3) for k, v in out.items()}}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
