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
        trace = tmp_path / "trace.csv"
        trace.write_text("session_id,round_idx,input_len,output_len,prefix_len,tool_wait_after_ms\n"
                         "0,0,70,5,0,10\n0,1,20,6,75,0\n1,0,90,4,0,0\n1,1,10,3,94,5\n1,2,15,2,107,0\n")
        r = subprocess.run(base + ["--concurrency", "2", "--trace", str(trace)], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        out = json.loads(r.stdout.strip().splitlines()[-1])
        assert out["requests"] == 5 and out["output_tokens"] == 20 and out["cached_tokens"] > 0
    finally:
        s.stop()
