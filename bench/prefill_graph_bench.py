"""Captured prefill passes against the same passes run kernel by kernel, through the engine's own pass.

    python bench/prefill_graph_bench.py [--layers 8] [--start 3600] [--news 61,180,440,900] [--reps 8]

Builds a single-GPU engine (random weights of the flagship architecture, ``--layers`` decoder layers; 0 = all 40)
with ``prefill_graphs`` on, prefills a ``--start``-token context into one request's slot and then, per N, times
the pass that adds N new tokens to it (a session's next turn) both ways, interleaved: the graph of the padded
size, and ``Model.forward`` over the same span kernel by kernel. Times are wall clock around a synchronised
pass (what a request waits for), median of ``--reps``. Also checks that both forms give the same last-row
hidden state bit for bit (the GDN rows of the slot are restored before each run). One JSON line per N
(reference: ``tools/prefill_graph_bench.py``)."""

from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--start", type=int, default=3600)
    ap.add_argument("--news", default="61,180,440,900")
    ap.add_argument("--reps", type=int, default=8)
    ap.add_argument("--tiny", action="store_true", help="the tiny test architecture instead of the flagship's")
    args = ap.parse_args()

    from b200serve.config import EngineConfig, ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.models.qwen36 import PackedBatch
    from b200serve.sched.engine import Engine
    from b200serve.sched.request import Generation, Sampling

    on_gpu = torch.cuda.is_available()
    dev = torch.device("cuda" if on_gpu else "cpu")  # without a GPU: the same passes kernel by kernel (a dry run)
    sync = torch.cuda.synchronize if on_gpu else (lambda: None)
    if args.tiny:
        cfg = ModelConfig.tiny(head_dim=64, num_attention_heads=4, num_key_value_heads=1)
    else:
        cfg = ModelConfig(**({"num_hidden_layers": args.layers} if args.layers else {}))
    w = random_weights(cfg, seed=0, device=dev, dtype=torch.bfloat16 if on_gpu else torch.float32)
    eng = Engine(w, EngineConfig(max_model_len=8192, prefill_chunk_tokens=2048, max_seqs=4, mtp=False, kv_pages=512,
                                 prefill_graphs=True, pack_weights=on_gpu and not args.tiny, decode_buckets=(1,),
                                 device=dev.type, graphs_on_cpu=not on_gpu))
    assert eng._pgraphs is not None, "this model's spans do not take the native prefill kernels"
    g = torch.Generator().manual_seed(0)
    news = [int(x) for x in args.news.split(",")]
    model, ops = eng.model, eng.ops
    gen = Generation(prompt=torch.randint(3, cfg.vocab_size, (args.start + max(news) + 1,), generator=g).tolist(),
                     sampling=Sampling(max_tokens=1, ignore_eos=True))
    eng._claim(gen)
    a = args.start
    for lo, hi in eng._spans(0, a):  # the context, chunk by chunk, kernel by kernel
        eng._ensure_pages(gen, hi)
        model.forward(PackedBatch.prefill([gen.prompt[lo:hi]], [gen.slot], [lo], eng._table([gen]), dev))
    sync()
    if on_gpu:
        ops.check_errors(dev)
    conv, rec = model.conv_state[:, gen.slot].clone(), model.rec_state[:, gen.slot].clone()
    for n in news:
        b = a + n
        eng._ensure_pages(gen, b)
        bucket = eng._pgraphs._bucket(n)
        if bucket is None:
            print(json.dumps({"new_tokens": n, "error": eng._pgraphs.errors}))
            continue

        def restore():
            model.conv_state[:, gen.slot].copy_(conv)
            model.rec_state[:, gen.slot].copy_(rec)

        def graphed():
            h, _ = eng._pgraphs.run(bucket, gen, a, b)
            return h[n - 1]

        def eager():
            batch = PackedBatch.prefill([gen.prompt[a:b]], [gen.slot], [a], eng._table([gen]), dev)
            return model.forward(batch)[n - 1]

        times = {"graph": [], "eager": []}
        last = {}
        for rep in range(args.reps + 2):
            for name, fn in (("graph", graphed), ("eager", eager)):
                restore()
                sync()
                t0 = time.perf_counter()
                out = fn()
                sync()
                if rep >= 2:
                    times[name].append((time.perf_counter() - t0) * 1e3)
                last[name] = out.clone()
        if on_gpu:
            ops.check_errors(dev)
        ms = {k: statistics.median(v) for k, v in times.items()}
        print(json.dumps({"new_tokens": n, "context": a, "layers": cfg.num_hidden_layers, "graph_rows": bucket.rows,
                          "graph_ms": round(ms["graph"], 3), "eager_ms": round(ms["eager"], 3),
                          "speedup": round(ms["eager"] / ms["graph"], 2), "launches_in_graph": bucket.launches,
                          "last_row_bitwise_equal": bool(torch.equal(last["graph"], last["eager"])),
                          "last_row_max_abs_diff": float((last["graph"].float() - last["eager"].float()).abs().max())}),
              flush=True)


if __name__ == "__main__":
    main()
