"""The load generator against a CPU server with random-init tiny weights (no checkpoint on disk)."""

import json
import subprocess
import sys

from http_util import ROOT, ServerProc


def test_serve_bench_single_round_and_sessions(tmp_path):
    s = ServerProc("random:tiny")
    try:
        base = [sys.executable, str(ROOT / "bench/serve_bench.py"), "--url", s.url, "--model", s.model, "--vocab", "1024"]
        r = subprocess.run(base + ["--concurrency", "4", "--requests", "6", "--prompt-len", "30-90", "--output-len", "8"],
                           capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        out = json.loads(r.stdout.strip().splitlines()[-1])
        assert out["requests"] == 6 and out["output_tokens"] == 48 and out["ttft_ms"]["p50"] > 0
        r = subprocess.run(base + ["--concurrency", "3", "--sessions", "3", "--rounds", "2-3", "--first-len", "60",
                                   "--max-first-len", "200", "--grow", "5-20", "--output-len", "4-9", "--rate", "20"],
                           capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        out = json.loads(r.stdout.strip().splitlines()[-1])
        assert out["requests"] >= 6 and out["cached_tokens"] > 0  # later rounds reuse their session tails
    finally:
        s.stop()
