"""The server with a stand-in model whose decode step costs a fixed amount of VIRTUAL GPU time: isolates the host path.

    python bench/null_model_server.py --port 8124 [--step-ms 17] [--max-seqs 128] &
    python bench/serve_bench.py --url http://127.0.0.1:8124 --model q --vocab 1000 --concurrency 128 --requests 128 \
        --prompt-len 64 --output-len 256

Everything above the model is the real thing: HTTP handlers, tokenizer, scheduler, the decode-graph scheduling with
run-ahead (on its kernel-by-kernel form, no GPU needed), event delivery, detokenisation, SSE writes. The model's
passes return at once and advance a virtual GPU clock (``--step-ms`` per decode step, 10 us per prefill token); a
step's result becomes readable when that clock says so. With a perfect host path the served TPOT equals
``--step-ms``; what is above it is the host's share. ``/health`` works as usual (``ENGINE_LOOP_TIMERS=1`` adds the
loop's stage timers). Runs on the CPU; tokens are meaningless."""

from __future__ import annotations

import argparse
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
os.environ.setdefault("ENGINE_MTP", "0")
os.environ["CUDA_VISIBLE_DEVICES"] = ""

import torch  # noqa: E402


def install(step_s: float, prefill_s_per_token: float = 1e-5) -> None:
    """Replace the model's passes by stand-ins on a virtual GPU timeline."""
    from b200serve import config as cfgmod
    from b200serve.models import qwen36
    from b200serve.sched import graphs

    clock = {"ready": 0.0, "n": 0}
    zeros: dict[int, torch.Tensor] = {}

    def forward(self, batch, ring=None):
        rows = batch.tokens.shape[0]
        cost = step_s if batch.G > 0 else prefill_s_per_token * rows
        clock["ready"] = max(clock["ready"], time.perf_counter()) + cost
        if batch.G == 0:  # a prefill pass is read back right away
            time.sleep(max(0.0, clock["ready"] - time.perf_counter()))
        if rows not in zeros:
            zeros[rows] = torch.zeros(rows, self.cfg.hidden_size)
        return zeros[rows]

    def greedy(self, hidden, out=None):
        clock["n"] += 1
        picks = (torch.arange(hidden.shape[0]) * 7 + clock["n"]) % 900 + 3
        if out is not None:
            out.copy_(picks)
            return out
        return picks

    qwen36.Model.forward = forward
    qwen36.Model.greedy = greedy
    start, collect = graphs.DecodeGraphs._start, graphs.DecodeGraphs.collect

    def start_with_clock(self, bucket, gens):
        handle = start(self, bucket, gens)
        handle["ready"] = clock["ready"]  # when this step's result exists on the virtual GPU
        return handle

    def collect_when_ready(self, handle):
        time.sleep(max(0.0, handle["ready"] - time.perf_counter()))
        return collect(self, handle)

    graphs.DecodeGraphs._start = start_with_clock
    graphs.DecodeGraphs.collect = collect_when_ready
    from_env = cfgmod.EngineConfig.from_env.__func__

    def from_env_on_cpu(cls, **kw):
        cfg = from_env(cls, **kw)
        cfg.graphs_on_cpu = True  # the decode-graph scheduling (buckets, run-ahead) without a device
        return cfg

    cfgmod.EngineConfig.from_env = classmethod(from_env_on_cpu)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--port", type=int, required=True)
    ap.add_argument("--step-ms", type=float, default=17.0)
    ap.add_argument("--max-seqs", type=int, default=128)
    args = ap.parse_args()
    install(args.step_ms / 1e3)
    from b200serve.api import server

    server.main(["--model", "random:tiny", "--served-model-name", "q", "--host", "127.0.0.1", "--port", str(args.port),
                 "--device", "cpu", "--max-seqs", str(args.max_seqs), "--max-model-len", "4096"])


if __name__ == "__main__":
    main()
