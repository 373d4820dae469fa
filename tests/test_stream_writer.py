"""The shared response writer: one thread serves every stream; disconnects, slow readers and the per-handler mode."""

import json
import socket
import time

import pytest
import requests
from http_util import ServerProc, ids_of

from b200serve.models.tiny import write_tiny_checkpoint


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    d = tmp_path_factory.mktemp("tiny")
    write_tiny_checkpoint(d, lm_head_std=0.5)
    return d


@pytest.fixture(scope="module")
def server(model_dir):
    s = ServerProc(model_dir, env={"CUDA_VISIBLE_DEVICES": ""})
    yield s
    s.stop()


def _idle(server, timeout=30):
    deadline = time.time() + timeout
    while time.time() < deadline:
        h = server.health()
        if h["running"] == 0 and h["prefilling"] == 0:
            return h
        time.sleep(0.1)
    return server.health()


def test_streams_go_through_one_writer_thread(server):
    chunks, usage = server.completion(list(range(5, 45)), 12)
    assert len(ids_of(chunks)) == 12 and usage["completion_tokens"] == 12
    h = server.health()
    # the first event of a request is consumed by its own thread (headers follow refusals); the rest by the writer
    assert h["writer_events"] >= 11 and h["writer_batches"] >= 1


def test_disconnect_mid_stream_cancels_the_generation(server):
    body = {"model": server.model, "prompt": list(range(20, 60)), "max_tokens": 1500, "temperature": 0, "ignore_eos": True, "stream": True}
    with requests.post(server.url + "/v1/completions", json=body, stream=True, timeout=60) as r:
        next(r.iter_lines())
    h = _idle(server)
    assert h["running"] == 0 and h["prefilling"] == 0
    chunks, _ = server.completion(list(range(5, 45)), 5)  # and the server keeps serving
    assert len(ids_of(chunks)) == 5


def test_a_client_that_reads_late_gets_every_chunk_and_stalls_nobody(server):
    """A raw socket with a tiny receive buffer that does not read while the request runs: the writer keeps what the
    socket does not take, other streams go on, and the late reader still receives every chunk in order."""
    n = 700
    body = json.dumps({"model": server.model, "prompt": list(range(30, 70)), "max_tokens": n, "temperature": 0, "ignore_eos": True,
                       "stream": True, "return_token_ids": True}).encode()
    sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
    sock.setsockopt(socket.SOL_SOCKET, socket.SO_RCVBUF, 2048)
    sock.connect(("127.0.0.1", server.port))
    sock.sendall(b"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\nContent-Length: "
                 + str(len(body)).encode() + b"\r\n\r\n" + body)
    t0 = time.time()
    other, _ = server.completion(list(range(5, 45)), 20)  # runs beside the stalled reader
    assert len(ids_of(other)) == 20 and time.time() - t0 < 60
    _idle(server, timeout=120)  # the generation finishes although nobody reads
    sock.settimeout(60)
    data = b""
    while True:
        part = sock.recv(1 << 16)
        if not part:
            break
        data += part
    sock.close()
    head, _, payload = data.partition(b"\r\n\r\n")
    assert head.startswith(b"HTTP/1.1 200") and payload.rstrip().endswith(b"data: [DONE]")
    events = [json.loads(ln[6:]) for ln in payload.split(b"\n\n") if ln.startswith(b"data: {")]
    got = [t for ev in events for ch in ev["choices"] for t in (ch.get("token_ids") or [])]
    assert len(got) == n
    again, _ = server.completion(list(range(30, 70)), 40)
    assert ids_of(again) == got[:40]


def test_per_handler_mode_gives_the_same_stream(model_dir, server):
    old = ServerProc(model_dir, env={"CUDA_VISIBLE_DEVICES": "", "ENGINE_STREAM_WRITER": "0"})
    try:
        prompt = list(range(11, 71))
        a, ua = server.completion(prompt, 24)
        b, ub = old.completion(prompt, 24)
        assert ids_of(a) == ids_of(b) and [c["choices"][0]["text"] for c in a] == [c["choices"][0]["text"] for c in b]
        assert ua["completion_tokens"] == ub["completion_tokens"] == 24
        assert "writer_events" not in old.health()
        r1 = server.post("/v1/completions", {"model": server.model, "prompt": prompt, "max_tokens": 9, "temperature": 0})
        r2 = old.post("/v1/completions", {"model": old.model, "prompt": prompt, "max_tokens": 9, "temperature": 0})
        assert r1.status_code == r2.status_code == 200 and r1.json()["choices"][0]["text"] == r2.json()["choices"][0]["text"]
        bad = {"model": server.model, "prompt": list(range(4000)), "max_tokens": 5, "stream": True}
        assert server.post("/v1/completions", bad).status_code == old.post("/v1/completions", bad).status_code == 400
    finally:
        old.stop()


def test_writer_keeps_what_a_socket_does_not_take():
    """The non-blocking send path against a fake socket: partial sends, a full buffer, a reset, an overflow."""
    import threading

    from b200serve.api.server import StreamWriter

    class FakeSock:
        def __init__(self):
            self.room, self.got, self.fail = 0, b"", None

        def send(self, data, flags=0):
            assert flags == socket.MSG_DONTWAIT
            if self.fail is not None:
                raise self.fail
            if self.room == 0:
                raise BlockingIOError()
            n = min(self.room, len(data))
            self.got += bytes(data[:n])
            self.room -= n
            return n

    class FakeStream:  # the fields of ``Stream`` that the send path touches
        def __init__(self):
            self.sock, self.backlog, self.dead, self.finished, self.cancelled = FakeSock(), bytearray(), False, threading.Event(), 0

        def cancel(self):
            self.cancelled += 1

    mk = FakeStream

    w = StreamWriter()
    st = mk()
    st.sock.room = 4
    w._send(st, b"0123456789")
    assert st.sock.got == b"0123" and bytes(st.backlog) == b"456789" and st in w.backlogged
    w._send(st, b"abc")  # nothing fits: the new bytes queue up behind the old ones
    assert bytes(st.backlog) == b"456789abc" and w.stats["writer_partial_sends"] == 2
    st.sock.room = 5
    w._send(st, b"")  # the retry of the writer's loop
    assert st.sock.got == b"012345678" and bytes(st.backlog) == b"9abc"
    st.sock.room = 100
    w._send(st, b"def")
    assert st.sock.got == b"0123456789abcdef" and not st.backlog and st not in w.backlogged and not st.dead
    st.sock.fail = ConnectionResetError()
    w._send(st, b"x")
    assert st.dead and st.cancelled == 1 and st.finished.is_set()
    w._send(st, b"y")  # a dead stream takes nothing more
    assert st.sock.got == b"0123456789abcdef"
    big = mk()
    w.MAX_BACKLOG = 16
    w._send(big, b"z" * 17)  # a reader that never reads is given up once its backlog passes the limit
    assert big.dead and big.cancelled == 1 and big.finished.is_set() and big not in w.backlogged


def test_stand_in_model_server_isolates_the_host_path():
    """``bench/null_model_server.py``: with a 5 ms virtual step and 8 streams the served TPOT stays close to 5 ms."""
    import os
    import subprocess
    import sys

    from http_util import ROOT, free_port

    port = free_port()
    srv = subprocess.Popen([sys.executable, str(ROOT / "bench/null_model_server.py"), "--port", str(port), "--step-ms", "5",
                            "--max-seqs", "8"], env=dict(os.environ, OMP_NUM_THREADS="2"), cwd=str(ROOT))
    try:
        deadline = time.time() + 180
        while time.time() < deadline:
            try:
                if requests.get(f"http://127.0.0.1:{port}/health", timeout=2).status_code == 200:
                    break
            except requests.RequestException:
                time.sleep(0.3)
        r = subprocess.run([sys.executable, str(ROOT / "bench/serve_bench.py"), "--url", f"http://127.0.0.1:{port}", "--model", "q",
                            "--vocab", "1000", "--concurrency", "8", "--requests", "8", "--prompt-len", "32", "--output-len", "100"],
                           capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2000:]
        out = json.loads(r.stdout.strip().splitlines()[-1])
        assert out["valid"] and out["output_tokens"] == 800
        assert 4.5 <= out["tpot_ms"]["p50"] <= 40.0  # never below the virtual step; the host share stays bounded on a busy machine too
        h = requests.get(f"http://127.0.0.1:{port}/health", timeout=5).json()
        assert h["ahead_steps"] > 50  # run-ahead scheduling is what runs
    finally:
        srv.terminate()
        try:
            srv.wait(timeout=10)
        except subprocess.TimeoutExpired:
            srv.kill()


def test_random_clients_with_disconnects_leave_a_clean_server(server):
    """24 concurrent clients, streaming or not, some of which hang up mid-stream: every finished request equals the
    same request sent alone afterwards, and nothing stays behind in the engine."""
    import random
    from concurrent.futures import ThreadPoolExecutor

    rng = random.Random(4)
    jobs = []
    for i in range(24):
        n = rng.randrange(4, 40)
        jobs.append(dict(prompt=[rng.randrange(5, 500) for _ in range(rng.randrange(3, 120))], max_tokens=n,
                         stream=rng.random() < 0.7, hang_up_after=rng.randrange(1, n) if rng.random() < 0.3 else None))

    def body(j):
        return {"model": server.model, "prompt": j["prompt"], "max_tokens": j["max_tokens"], "temperature": 0, "ignore_eos": True,
                "return_token_ids": True}

    def run(j):
        if not j["stream"]:
            r = server.post("/v1/completions", body(j))
            assert r.status_code == 200
            return r.json()["choices"][0]["token_ids"]
        ids = []
        with requests.post(server.url + "/v1/completions", json={**body(j), "stream": True}, stream=True, timeout=120) as r:
            r.raise_for_status()
            for line in r.iter_lines():
                if not line.startswith(b"data: ") or line == b"data: [DONE]":
                    continue
                for ch in json.loads(line[6:]).get("choices", []):
                    ids.extend(ch.get("token_ids") or [])
                if j["hang_up_after"] is not None and len(ids) >= j["hang_up_after"]:
                    return ids  # leaving the block closes the connection mid-stream
        return ids

    with ThreadPoolExecutor(max_workers=24) as pool:
        got = list(pool.map(run, jobs))
    h = _idle(server, timeout=60)
    assert h["running"] == 0 and h["prefilling"] == 0 and h["status"] == "ok"
    for j, ids in zip(jobs, got):
        alone = server.post("/v1/completions", body(j)).json()["choices"][0]["token_ids"]
        if j["stream"] and j["hang_up_after"] is not None:
            assert ids == alone[: len(ids)] and len(ids) >= j["hang_up_after"]
        else:
            assert ids == alone and len(ids) == j["max_tokens"]
