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
        assert out["valid"] and out["planned_steps"] == out["success_steps"] == 5 and out["failed_steps"] == 0
        assert out["target_output_tokens"] == 20
        # a replay with failed steps is reported as invalid and the tool exits non-zero
        r = subprocess.run(base[:-4] + ["--model", "no-such-model", "--vocab", "1024", "--concurrency", "2", "--trace", str(trace)],
                           capture_output=True, text=True, timeout=300)
        out = json.loads(r.stdout.strip().splitlines()[-1])
        assert r.returncode == 1 and not out["valid"] and out["failed_steps"] == 2 and out["success_steps"] == 0
    finally:
        s.stop()


def test_host_probes_run_without_a_gpu(tmp_path):
    """The CPU-side probes (incremental tokenizer, page / slot / prefix pools, CPU placement) report sane figures."""
    import importlib.util
    from pathlib import Path

    from b200serve.models.tiny import write_tiny_checkpoint

    spec = importlib.util.spec_from_file_location("host_probe", Path(__file__).resolve().parents[1] / "bench/host_probe.py")
    hp = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(hp)
    write_tiny_checkpoint(tmp_path)
    t = hp.main(["tokenize", "--model", str(tmp_path), "--rounds", "3", "--sessions", "3", "--turn-chars", "600"])
    assert t["ids_equal"] and t["reused_chars"] > t["encoded_chars"] > 0
    k = hp.main(["kv-pool", "--sessions", "8", "--prompt-tokens", "700", "--rounds", "3"])
    assert k["tail_hit_rate"] == round(2 / 3, 3) and 0.5 < k["cached_token_share"] < 1 and k["entries"] == 8
    c = hp.main(["cpu-place", "--replicas", "2", "--gpus-per-replica", "1"])
    assert len(c["replicas"]) == 2 and all(r["rank_cpus"] for r in c["replicas"])


def test_service_checker_against_a_tiny_server(tmp_path):
    """Determinism and stream == non-stream hold on a random-weight server; the echo gate, which needs a real model,
    fails there and turns the overall result (and the exit code) to a failure."""
    import importlib.util
    from pathlib import Path

    from http_util import ServerProc

    from b200serve.models.tiny import write_tiny_checkpoint

    spec = importlib.util.spec_from_file_location("service_check", Path(__file__).resolve().parents[1] / "bench/service_check.py")
    sc = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sc)
    write_tiny_checkpoint(tmp_path, lm_head_std=0.5)
    srv = ServerProc(tmp_path, env={"CUDA_VISIBLE_DEVICES": ""})
    try:
        assert sc.main(["--url", srv.url, "--model", srv.model, "--gates", "determinism,stream", "--n", "4", "--concurrency", "4"]) == 0
        out = sc.run_gates(srv.url, srv.model, ["echo", "determinism"], 3, 3, seed=1)
        assert out["error_count"] == 0 and out["gates"]["determinism"]["pass"]
        assert not out["gates"]["echo"]["pass"] and not out["pass"]
        bad = sc.run_gates(srv.url, "no-such-model", ["determinism"], 2, 2, seed=1)
        assert bad["error_count"] > 0 and not bad["pass"]
    finally:
        srv.stop()
