"""Served A/B of two settings of the engine: the same requests against a server started with setting A, then B,
then A and B again; identical-token counts between the settings and tok/s / TTFT / TPOT of each run.

    python bench/serve_ab.py --model random:qwen36 --a ENGINE_RUNAHEAD=0 --b ENGINE_RUNAHEAD=1 \
        [--requests 32 --concurrency 32 --prompt-len 1024 --output-len 128] [--server-flags "--max-seqs 64"]

A setting is a comma-separated list of ``NAME=value`` environment variables for the server process (every switch of
the engine has one: ``config.EngineConfig.from_env``, ``ENGINE_PDL``, ``ENGINE_ATTN_SPLIT_PAGES``, ...). The prompts
are fixed by ``--seed``; greedy decoding, ``ignore_eos``, exact output lengths, token ids streamed back. Settings that
must not change a request's tokens (launch chaining, run-ahead, graphs, speculation, packing) should report
``identical`` = number of requests; settings that are part of the numerics contract (attention split, token tiles)
show how many requests stay identical. The order A B A B separates the settings' effect from drift between runs
(reference: ``tools/serve_probe.py`` and its off / on / off / on gates, e.g. ``tools/combine37_gate.sh:1-48``).
One JSON line per run and a final summary line.
"""

from __future__ import annotations

import argparse
import json
import os
import random
import signal
import socket
import subprocess
import sys
import threading
import time
from pathlib import Path

import requests

sys.path.insert(0, str(Path(__file__).resolve().parent))
from serve_bench import pct, stream_once  # noqa: E402

ROOT = Path(__file__).resolve().parents[1]


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def start_server(model: str, flags: list[str], env: dict, wait_s: float):
    port = free_port()
    cmd = [sys.executable, str(ROOT / "main.py"), "--model", model, "--served-model-name", "ab", "--host", "127.0.0.1",
           "--port", str(port), *flags]
    proc = subprocess.Popen(cmd, env={**os.environ, **env}, start_new_session=True,
                            stdout=subprocess.DEVNULL, stderr=subprocess.STDOUT)
    url = f"http://127.0.0.1:{port}"
    deadline = time.time() + wait_s
    while time.time() < deadline:
        if proc.poll() is not None:
            raise RuntimeError(f"server exited with code {proc.returncode}")
        try:
            if requests.get(url + "/health", timeout=2).status_code == 200:
                return proc, url
        except requests.RequestException:
            pass
        time.sleep(0.5)
    stop_server(proc)
    raise RuntimeError("server did not come up")


def stop_server(proc) -> None:
    try:
        os.killpg(proc.pid, signal.SIGTERM)  # the server's own process group: front, replicas, follower ranks
        proc.wait(timeout=20)
    except Exception:  # noqa: BLE001
        try:
            os.killpg(proc.pid, signal.SIGKILL)
        except Exception:  # noqa: BLE001
            pass


def run_load(url: str, prompts: list[list[int]], out_len: int, concurrency: int) -> dict:
    results: list = [None] * len(prompts)
    nxt = iter(range(len(prompts)))
    lock = threading.Lock()

    def worker():
        while True:
            with lock:
                i = next(nxt, None)
            if i is None:
                return
            results[i] = stream_once(url, "ab", prompts[i], out_len)

    t0 = time.perf_counter()
    threads = [threading.Thread(target=worker) for _ in range(concurrency)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    ttft = [r["stamps"][0] - r["start"] for r in results if r["stamps"]]
    tpot = [(r["stamps"][-1] - r["stamps"][0]) / (len(r["ids"]) - 1) for r in results if len(r["ids"]) > 1]
    return {"ids": [r["ids"] for r in results], "failed": sum(1 for r in results if r["error"]), "output_tok_s": round(sum(len(r["ids"]) for r in results) / wall, 1),
            "ttft_p50_ms": round(1e3 * pct(ttft, 0.5), 2), "tpot_p50_ms": round(1e3 * pct(tpot, 0.5), 3),
            "tpot_p90_ms": round(1e3 * pct(tpot, 0.9), 3)}


def parse_env(text: str) -> dict:
    return dict(kv.split("=", 1) for kv in text.split(",") if kv)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="random:qwen36")
    ap.add_argument("--a", default="", help="setting A: NAME=value[,NAME=value...] for the server's environment")
    ap.add_argument("--b", required=True, help="setting B")
    ap.add_argument("--server-flags", default="")
    ap.add_argument("--requests", type=int, default=32)
    ap.add_argument("--concurrency", type=int, default=32)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=128)
    ap.add_argument("--vocab", type=int, default=248320)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--rounds", type=int, default=2, help="A B pairs (2 = A B A B)")
    ap.add_argument("--health-wait", type=float, default=600.0)
    a = ap.parse_args()
    rng = random.Random(a.seed)
    prompts = [[rng.randrange(3, a.vocab) for _ in range(a.prompt_len)] for _ in range(a.requests)]
    runs = []
    for rnd in range(a.rounds):
        for name, text in (("A", a.a), ("B", a.b)):
            proc, url = start_server(a.model, a.server_flags.split(), parse_env(text), a.health_wait)
            try:
                run_load(url, prompts[: min(4, len(prompts))], 8, 4)  # warm the path the load takes
                res = run_load(url, prompts, a.output_len, a.concurrency)
            finally:
                stop_server(proc)
            res.update(setting=name, env=text, round=rnd)
            runs.append(res)
            print(json.dumps({k: v for k, v in res.items() if k != "ids"}), flush=True)
    base = runs[0]["ids"]
    same = {f"{r['setting']}{r['round']}": sum(x == y for x, y in zip(r["ids"], base)) for r in runs[1:]}

    def mean(name, key):
        vals = [r[key] for r in runs if r["setting"] == name]
        return round(sum(vals) / len(vals), 3)

    print(json.dumps({"summary": True, "requests": a.requests, "identical_to_first_run": same,
                      "output_tok_s": {"A": mean("A", "output_tok_s"), "B": mean("B", "output_tok_s")},
                      "tpot_p50_ms": {"A": mean("A", "tpot_p50_ms"), "B": mean("B", "tpot_p50_ms")},
                      "ttft_p50_ms": {"A": mean("A", "ttft_p50_ms"), "B": mean("B", "ttft_p50_ms")}}), flush=True)


if __name__ == "__main__":
    main()
