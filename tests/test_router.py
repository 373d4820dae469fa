"""The data-parallel front with two CPU replicas as real subprocesses."""

import json
import os
import subprocess
import sys
import time

import pytest
import requests

from http_util import ROOT, free_port, ids_of


@pytest.fixture(scope="module")
def front(tmp_path_factory):
    from b200serve.models.tiny import write_tiny_checkpoint

    path = tmp_path_factory.mktemp("tiny-router")
    write_tiny_checkpoint(path, lm_head_std=0.5)
    port = free_port()
    cmd = [sys.executable, "-m", "b200serve.api.server", "--model", str(path), "--served-model-name", "tiny", "--host",
           "127.0.0.1", "--port", str(port), "--max-model-len", "2048", "--prefill-chunk-tokens", "64", "--device", "cpu",
           "--max-seqs", "4", "--replicas", "2"]
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="2", ENGINE_REQ_STAMPS="1", ENGINE_CPU_PIN="0")
    proc = subprocess.Popen(cmd, env=env, cwd=str(ROOT))
    url = f"http://127.0.0.1:{port}"
    deadline = time.time() + 240
    while True:
        assert proc.poll() is None, "front exited"
        try:
            if requests.get(url + "/health", timeout=2).status_code == 200:
                break
        except requests.RequestException:
            pass
        assert time.time() < deadline
        time.sleep(0.3)
    yield url
    proc.terminate()
    proc.wait(timeout=20)


def _complete(url, prompt, n, stream=True):
    body = {"model": "tiny", "prompt": prompt, "max_tokens": n, "temperature": 0, "ignore_eos": True,
            "return_token_ids": True, "stream": stream, "stream_options": {"include_usage": True}}
    if not stream:
        return requests.post(url + "/v1/completions", json=body, timeout=120).json()
    events = []
    with requests.post(url + "/v1/completions", json=body, stream=True, timeout=120) as r:
        assert r.headers["content-type"] == "text/event-stream"
        for ln in r.iter_lines():
            if ln.startswith(b"data: ") and ln != b"data: [DONE]":
                events.append(json.loads(ln[6:]))
    return events


def test_sessions_stay_on_their_replica_and_hit_its_cache(front):
    h0 = requests.get(front + "/health").json()
    assert h0["replicas"] == 2 and len(h0["per_replica"]) == 2
    sessions = [[10 + (i * (3 + s)) % 300 for i in range(120)] for s in range(2)]
    outs = []
    for s in sessions:
        ev = _complete(front, s, 6)
        outs.append(ids_of(ev[:-1]))
    for s, o in zip(sessions, outs):  # second round of each session: prompt + output + new turn
        ev = _complete(front, s + o + [7, 8, 9], 4)
        assert ev[-1]["usage"]["prompt_tokens_details"]["cached_tokens"] == len(s) + 6 - 1
    h1 = requests.get(front + "/health").json()
    assert h1["routed_by_affinity"] >= 2
    per = [b["requests"] for b in h1["per_replica"]]
    assert per == [2, 2]  # two sessions, one per replica, both rounds each
    assert "request_stamps" in h1["per_replica"][0]
    m = requests.get(front + "/metrics")  # the summed counters of both replicas for a scraper
    vals = dict(ln.split(" ") for ln in m.text.splitlines() if ln and not ln.startswith("#"))
    assert m.status_code == 200 and vals["engine_up"] == "1" and int(vals["engine_requests"]) == 4 and vals["engine_replicas"] == "2"


def test_errors_and_non_streaming_pass_through(front):
    r = requests.post(front + "/v1/completions", json={"model": "nope", "prompt": [1, 2, 3]})
    assert r.status_code == 404 and r.json()["error"]["code"] == 404
    whole = _complete(front, [5, 6, 7, 8], 5, stream=False)
    assert whole["usage"]["completion_tokens"] == 5
    assert requests.get(front + "/v1/models").json()["data"][0]["id"] == "tiny"


def test_client_disconnect_frees_the_request(front):
    body = {"prompt": list(range(20, 60)), "max_tokens": 400, "temperature": 0, "ignore_eos": True, "stream": True}
    with requests.post(front + "/v1/completions", json=body, stream=True, timeout=60) as r:
        next(r.iter_lines())
    deadline = time.time() + 30
    while time.time() < deadline:
        h = requests.get(front + "/health").json()
        if h["running"] == 0 and h["prefilling"] == 0:
            break
        time.sleep(0.2)
    assert h["running"] == 0
