"""Replicas that share expert-parallel MoE blocks, served over HTTP on CPU processes (gloo stand-in for the NVLink
kernels): outputs must equal a single-process server's, whichever replica a request lands on and whatever the
other replica is doing at the time; and the front must go down with a replica that dies."""

import os
import subprocess
import sys
import threading
import time

import pytest
import requests

from http_util import ROOT, ServerProc, free_port, ids_of


def _start_front(path, extra, env):
    port = free_port()
    cmd = [sys.executable, "-m", "b200serve.api.server", "--model", str(path), "--served-model-name", "tiny", "--host",
           "127.0.0.1", "--port", str(port), "--max-model-len", "2048", "--prefill-chunk-tokens", "64", "--device", "cpu",
           "--max-seqs", "4", *extra]
    e = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="2", ENGINE_CPU_PIN="0", CUDA_VISIBLE_DEVICES="", **env)
    proc = subprocess.Popen(cmd, env=e, cwd=str(ROOT))
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
    return proc, url


def _complete(url, prompt, n):
    import json

    body = {"model": "tiny", "prompt": prompt, "max_tokens": n, "temperature": 0, "ignore_eos": True,
            "return_token_ids": True, "stream": True, "stream_options": {"include_usage": True}}
    events = []
    with requests.post(url + "/v1/completions", json=body, stream=True, timeout=300) as r:
        r.raise_for_status()
        for ln in r.iter_lines():
            if ln.startswith(b"data: ") and ln != b"data: [DONE]":
                events.append(json.loads(ln[6:]))
    return events


@pytest.fixture(scope="module")
def tiny_dir(tmp_path_factory):
    from b200serve.models.tiny import write_tiny_checkpoint

    path = tmp_path_factory.mktemp("tiny-dpep")
    write_tiny_checkpoint(path, lm_head_std=0.5)
    return path


def test_expert_parallel_replicas_serve_the_tokens_of_a_single_process(tiny_dir):
    proc, url = _start_front(tiny_dir, ["--replicas", "2", "--expert-parallel"], {"ENGINE_MTP": "0"})
    solo = ServerProc(tiny_dir, env={"CUDA_VISIBLE_DEVICES": "", "ENGINE_MTP": "0"})
    try:
        prompts = [[11 + (i * (5 + s)) % 400 for i in range(n)] for s, n in enumerate((30, 150, 75, 200, 12))]
        outs: dict = {}

        def run(j):
            outs[j] = _complete(url, prompts[j], 10 + 3 * j)

        # concurrent requests of different lengths: the replicas hold different batches, one of them is idle at times
        threads = [threading.Thread(target=run, args=(j,)) for j in range(len(prompts))]
        for t in threads:
            t.start()
            time.sleep(0.05)
        for t in threads:
            t.join(timeout=300)
        for j, p in enumerate(prompts):
            want, _ = solo.completion(p, 10 + 3 * j)
            assert ids_of(outs[j][:-1]) == ids_of(want), j
        # a lone request while the other replica has nothing to do (it joins with empty passes)
        ev = _complete(url, prompts[1] + [9, 9, 9], 8)
        want, _ = solo.completion(prompts[1] + [9, 9, 9], 8)
        assert ids_of(ev[:-1]) == ids_of(want)
        assert ev[-1]["usage"]["prompt_tokens_details"]["cached_tokens"] > 0  # the session found its replica's cache
        h = requests.get(url + "/health").json()
        assert h["replicas"] == 2 and all(b["requests"] >= 1 for b in h["per_replica"])
        assert all(b["broken"] is None for b in h["per_replica"])
    finally:
        proc.terminate()
        proc.wait(timeout=30)
        solo.stop()


def test_the_front_stops_when_a_replica_dies(tiny_dir):
    """Router watchdog (reference: engine/router.py:568-578): one replica process is killed between requests; the
    front notices, stops the others and exits, so no client is left talking to half a service."""
    import psutil

    proc, url = _start_front(tiny_dir, ["--replicas", "2"], {"ENGINE_MTP": "0"})
    try:
        assert _complete(url, list(range(20, 60)), 4)
        children = [c for c in psutil.Process(proc.pid).children(recursive=False)]
        assert len(children) == 2
        children[1].kill()
        proc.wait(timeout=30)
        assert proc.returncode not in (None, 0)
        with pytest.raises(requests.RequestException):
            requests.get(url + "/health", timeout=2)
        time.sleep(0.5)
        assert not children[0].is_running() or children[0].status() == psutil.STATUS_ZOMBIE
    finally:
        if proc.poll() is None:
            proc.terminate()
            proc.wait(timeout=30)


def _launch_ranks(mode: str, nproc: int, port: int, env: dict):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), str(ROOT / "tests/dist_worker.py"), mode]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=600, env={**os.environ, **env})


def test_replicas_with_their_own_request_streams_on_cpu_ranks():
    """Each replica loops over ``Engine.step`` on its own; requests arrive at different times, in different numbers and
    lengths; idle replicas join with empty passes: every request's tokens equal the unsharded engine's."""
    r = _launch_ranks("dp_ep_served", 2, 29661, {"CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 0 and "OK dp_ep_served" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.gpu
def test_replicas_with_their_own_request_streams_on_two_gpus():
    """The same on the NVLink kernels: decode from the graphs captured at warm-up, peer waits inside the kernels."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    r = _launch_ranks("dp_ep_served", 2, 29662, {"NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0 and "OK dp_ep_served" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
