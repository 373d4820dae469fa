"""The served A/B tool on CPU: speculation on against off must leave every request's tokens identical."""

import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_served_ab_reports_identical_tokens_for_speculation_on_and_off(tmp_path):
    cmd = [sys.executable, str(ROOT / "bench/serve_ab.py"), "--model", "random:tiny", "--vocab", "1000", "--a", "ENGINE_MTP=0",
           "--b", "ENGINE_MTP=1,ENGINE_SPEC_K=2", "--server-flags", "--device cpu --max-model-len 1024 --prefill-chunk-tokens 64",
           "--requests", "5", "--concurrency", "3", "--prompt-len", "70", "--output-len", "12", "--rounds", "1",
           "--health-wait", "180"]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2", ENGINE_CPU_PIN="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(tmp_path))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    lines = [json.loads(x) for x in r.stdout.splitlines() if x.startswith("{")]
    summary = lines[-1]
    assert summary["summary"] and summary["identical_to_first_run"] == {"B0": 5}
    assert [x["setting"] for x in lines[:-1]] == ["A", "B"] and all(x["output_tok_s"] > 0 for x in lines[:-1])
