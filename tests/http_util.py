"""Helpers for tests that talk to a real server process over HTTP."""

from __future__ import annotations

import json
import os
import socket
import subprocess
import sys
import time
from pathlib import Path

import requests

ROOT = Path(__file__).resolve().parents[1]
CHUNK = 64


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class ServerProc:
    def __init__(self, model_dir: Path, extra: list[str] | None = None, env: dict | None = None) -> None:
        self.port = free_port()
        self.url = f"http://127.0.0.1:{self.port}"
        self.model = "tiny"
        cmd = [sys.executable, "-m", "b200serve.api.server", "--model", str(model_dir), "--served-model-name",
               self.model, "--host", "127.0.0.1", "--port", str(self.port), "--max-model-len", "2048",
               "--prefill-chunk-tokens", str(CHUNK), "--device", "cpu", "--max-seqs", "8", *(extra or [])]
        e = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="2", **(env or {}))
        self.proc = subprocess.Popen(cmd, env=e, cwd=str(ROOT))
        deadline = time.time() + 180
        while True:
            if self.proc.poll() is not None:
                raise RuntimeError(f"server exited with {self.proc.returncode}")
            try:
                if requests.get(self.url + "/health", timeout=2).status_code == 200:
                    break
            except requests.RequestException:
                pass
            if time.time() > deadline:
                self.stop()
                raise TimeoutError("server did not start")
            time.sleep(0.2)

    def stop(self) -> None:
        if self.proc.poll() is None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=10)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def health(self) -> dict:
        return requests.get(self.url + "/health", timeout=10).json()

    def post(self, route: str, body: dict, **kw):
        return requests.post(self.url + route, json=body, timeout=300, **kw)

    def stream(self, route: str, body: dict) -> list[dict]:
        events = []
        with requests.post(self.url + route, json={**body, "stream": True}, stream=True, timeout=300) as r:
            r.raise_for_status()
            assert r.headers["content-type"] == "text/event-stream"
            lines = [ln.decode() for ln in r.iter_lines() if ln.startswith(b"data: ")]
        assert lines[-1] == "data: [DONE]"
        for ln in lines[:-1]:
            events.append(json.loads(ln[len("data: "):]))
        return events

    def completion(self, prompt, max_tokens: int, **extra):
        body = {"model": self.model, "prompt": prompt, "max_tokens": max_tokens, "temperature": 0, "ignore_eos": True,
                "return_token_ids": True, "stream_options": {"include_usage": True}, **extra}
        *chunks, last = self.stream("/v1/completions", body)
        assert last["choices"] == []
        return chunks, last["usage"]


def ids_of(chunks: list[dict]) -> list[int]:
    return [t for c in chunks for t in c["choices"][0]["token_ids"]]
