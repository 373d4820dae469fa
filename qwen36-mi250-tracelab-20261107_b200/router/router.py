"""Data-parallel front: N replica processes behind one port, with session affinity.

The front resolves a layout (which GPUs each replica gets), starts one server process per replica
with its device list narrowed through ``CUDA_VISIBLE_DEVICES`` and its CPU slice from
``cpu_place``, waits until every replica answers ``/health``, and then relays requests. A request
goes to the replica that remembers the longest prefix of its prompt (token ids, text or chat
messages), because that replica holds the session's prefix cache; otherwise to the least loaded
one. Responses, SSE streams included, are relayed byte for byte. If a replica dies the front
stops everything and exits (reference: ``engine/router.py:76-136, 142-273, 285-583``; the default
there is 2 GPUs per replica because the model does not fit one MI250 GCD — on a 180 GB B200 the
default is one GPU per replica).
"""

from __future__ import annotations

import ctypes
import hashlib
import http.client
import json
import os
import signal
import subprocess
import sys
import threading
import time
from collections import OrderedDict
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any

from . import cpu_place

BLOCK_UNITS = 64  # affinity hashes every 64 tokens / 256 characters / 1 chat message
RECENT_SECONDS = 30.0


# --------------------------------------------------------------------------- layout
def visible_gpus() -> list[int]:
    env = os.environ.get("CUDA_VISIBLE_DEVICES")
    if env is not None:
        return [int(x) for x in env.split(",") if x.strip().lstrip("-").isdigit() and int(x) >= 0]
    try:
        import torch

        return list(range(torch.cuda.device_count()))
    except Exception:  # noqa: BLE001
        return []


def resolve_layout(replicas: int | None, gpus_per_replica: int | None, replica_devices: str | None,
                   gpus: list[int] | None = None) -> list[list[int]] | None:
    """Device ids per replica, or ``None`` to serve in this process.

    ``replica_devices`` ("0,1;2,3") wins; else ``replicas`` x ``gpus_per_replica`` over the visible
    GPUs (default 1 GPU per replica, all GPUs used). With no GPU, ``replicas`` > 1 still gives that
    many CPU replicas (used by tests).
    """
    gpus = visible_gpus() if gpus is None else gpus
    if replica_devices:
        layout = [[int(x) for x in grp.split(",") if x.strip()] for grp in replica_devices.split(";") if grp.strip()]
        flat = [d for grp in layout for d in grp]
        if len(set(flat)) != len(flat):
            raise ValueError("--replica-devices names a device twice")
        return layout
    if not gpus:
        return [[] for _ in range(replicas)] if replicas and replicas > 1 else None
    per = gpus_per_replica or 1
    if per > len(gpus):
        raise ValueError(f"--gpus-per-replica {per} exceeds the {len(gpus)} visible GPUs")
    n = replicas or len(gpus) // per
    if n * per > len(gpus):
        raise ValueError(f"{n} replicas x {per} GPUs exceed the {len(gpus)} visible GPUs")
    if n <= 1 and per == len(gpus):
        return None
    if n <= 1 and replicas is None:
        return None
    return [gpus[i * per : (i + 1) * per] for i in range(n)]


def device_env(devices: list[int]) -> dict[str, str]:
    return {"CUDA_VISIBLE_DEVICES": ",".join(map(str, devices))} if devices else {"CUDA_VISIBLE_DEVICES": ""}


# --------------------------------------------------------------------------- affinity
def affinity_key(path: str, body: dict[str, Any]) -> list[bytes]:
    """Chain of block hashes that identifies the request's prompt prefix by prefix."""
    units: list[bytes]
    if path.endswith("/chat/completions"):
        msgs = body.get("messages") or []
        units = [json.dumps([m.get("role"), m.get("content"), m.get("tool_calls")], sort_keys=True).encode()
                 for m in msgs if isinstance(m, dict)]
        step = 1
    else:
        prompt = body.get("prompt")
        if isinstance(prompt, list) and len(prompt) == 1:
            prompt = prompt[0]
        if isinstance(prompt, str):
            units = [prompt[i : i + 4].encode() for i in range(0, len(prompt), 4)]
        elif isinstance(prompt, list):
            units = [str(t).encode() for t in prompt]
        else:
            units = []
        step = BLOCK_UNITS
    chain, h = [], hashlib.blake2b(digest_size=12)
    for i in range(0, len(units), step):
        for u in units[i : i + step]:
            h.update(u + b"\x1f")
        chain.append(h.copy().digest())
    return chain


class Affinity:
    """Remembers, per replica, the prompt prefixes it has served; balances the rest by load."""

    def __init__(self, n: int, capacity: int = 4096) -> None:
        self.n = n
        self.capacity = capacity
        self.lock = threading.Lock()
        self.seen: "OrderedDict[bytes, int]" = OrderedDict()  # block hash -> replica
        self.inflight = [0] * n
        self.recent: list[list[float]] = [[] for _ in range(n)]  # end times of recently finished requests
        self.routed_by_affinity = 0
        self.routed_by_load = 0

    def load(self, i: int, now: float | None = None) -> float:
        now = time.time() if now is None else now
        self.recent[i] = [t for t in self.recent[i] if now - t < RECENT_SECONDS]
        return self.inflight[i] + 0.5 * len(self.recent[i])

    def route(self, chain: list[bytes]) -> int:
        with self.lock:
            target = None
            for h in reversed(chain):  # longest remembered prefix first
                r = self.seen.get(h)
                if r is not None:
                    target = r
                    break
            if target is None:
                now = time.time()
                target = min(range(self.n), key=lambda i: (self.load(i, now), i))
                self.routed_by_load += 1
            else:
                self.routed_by_affinity += 1
            for h in chain:
                self.seen[h] = target
                self.seen.move_to_end(h)
            while len(self.seen) > self.capacity:
                self.seen.popitem(last=False)
            self.inflight[target] += 1
            return target

    def finish(self, replica: int) -> None:
        with self.lock:
            self.inflight[replica] = max(0, self.inflight[replica] - 1)
            self.recent[replica].append(time.time())


# --------------------------------------------------------------------------- replica processes
def _child_preexec(cpus: list[int] | None):
    def fn() -> None:
        try:  # die with the front (PR_SET_PDEATHSIG = 1)
            ctypes.CDLL("libc.so.6", use_errno=True).prctl(1, signal.SIGTERM)
        except OSError:
            pass
        if cpus:
            try:
                os.sched_setaffinity(0, set(cpus))
            except OSError:
                pass

    return fn


class Replica:
    def __init__(self, index: int, devices: list[int], port: int, proc: subprocess.Popen) -> None:
        self.index, self.devices, self.port, self.proc = index, devices, port, proc


def _free_port() -> int:
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _strip(argv: list[str], flags_with_value: tuple[str, ...]) -> list[str]:
    out, skip = [], False
    for a in argv:
        if skip:
            skip = False
            continue
        if a in flags_with_value:
            skip = True
            continue
        if any(a.startswith(f + "=") for f in flags_with_value):
            continue
        out.append(a)
    return out


def start_replicas(argv: list[str], layout: list[list[int]], pin: bool = True) -> list[Replica]:
    base = _strip(argv, ("--host", "--port", "--replicas", "--gpus-per-replica", "--replica-devices"))
    slices = None
    if pin and os.environ.get("ENGINE_CPU_PIN", "1") == "1":
        try:
            topo = cpu_place.Topology.read(gpu_bdfs=cpu_place.gpu_bdfs())
            if len(topo.physical_cores()) >= 2 * len(layout):
                slices = cpu_place.replica_slices(topo, layout)
        except Exception as e:  # noqa: BLE001
            print(f"cpu_place: placement skipped ({e})", flush=True)
    # ENGINE_EP=1 (--expert-parallel): the replicas form ONE expert-parallel group (parallel/dpep.py): each keeps the
    # dense weights and 1 / N of the routed experts, and their MoE blocks exchange rows over NVLink. Peer memory is
    # mapped by CUDA IPC, so every replica has to see all GPUs of the group; it runs on the one named ENGINE_EP_LOCAL.
    ep_group = os.environ.get("ENGINE_EP", "0") not in ("", "0") and len(layout) > 1
    ep_port = _free_port() if ep_group else 0
    all_devices = [d for grp in layout for d in grp]
    replicas = []
    for i, devices in enumerate(layout):
        port = _free_port()
        env = dict(os.environ)
        env.update(device_env(devices))
        if ep_group:
            if any(len(grp) > 1 for grp in layout):
                raise ValueError("an expert-parallel group takes one GPU per replica")
            env.update(device_env(all_devices))
            env.update(ENGINE_EP_WORLD=str(len(layout)), ENGINE_EP_RANK=str(i), ENGINE_EP_PORT=str(ep_port),
                       ENGINE_EP_LOCAL=str(all_devices.index(devices[0]) if devices else i))
        cpus = None
        if slices is not None:
            cpus = slices[i].cpus
            env.update(cpu_place.thread_caps(len(cpus)))
            env["ENGINE_CPUS"] = cpu_place.format_cpu_list(cpus)
            env["ENGINE_RANK_CPUS"] = cpu_place.format_cpu_list(slices[i].rank_cpus)
        # the children import the package by name whatever directory the front was started from
        import b200serve

        root = os.path.dirname(os.path.dirname(os.path.abspath(b200serve.__file__)))
        env["PYTHONPATH"] = root + (os.pathsep + env["PYTHONPATH"] if env.get("PYTHONPATH") else "")
        cmd = [sys.executable, "-m", "b200serve.api.server", *base, "--host", "127.0.0.1", "--port", str(port),
               "--replicas", "1"]
        proc = subprocess.Popen(cmd, env=env, preexec_fn=_child_preexec(cpus))
        replicas.append(Replica(i, devices, port, proc))
        print(f"router: replica {i} devices={devices or 'cpu'} port={port} pid={proc.pid}"
              + (f" cpus={env.get('ENGINE_CPUS')}" if cpus else ""), flush=True)
    return replicas


def wait_ready(replicas: list[Replica], timeout: float = 3600.0) -> None:
    deadline = time.time() + timeout
    pending = list(replicas)
    while pending:
        for r in list(pending):
            if r.proc.poll() is not None:
                raise RuntimeError(f"replica {r.index} exited with code {r.proc.returncode} while loading")
            try:
                c = http.client.HTTPConnection("127.0.0.1", r.port, timeout=2)
                c.request("GET", "/health")
                if c.getresponse().status == 200:
                    pending.remove(r)
                c.close()
            except OSError:
                pass
        if pending:
            if time.time() > deadline:
                raise TimeoutError("replicas did not become ready")
            time.sleep(0.2)


def stop_replicas(replicas: list[Replica]) -> None:
    for r in replicas:
        if r.proc.poll() is None:
            r.proc.terminate()
    for r in replicas:
        try:
            r.proc.wait(timeout=10)
        except subprocess.TimeoutExpired:
            r.proc.kill()


# --------------------------------------------------------------------------- front server
class FrontHandler(BaseHTTPRequestHandler):
    protocol_version = "HTTP/1.1"

    def log_message(self, fmt: str, *args: Any) -> None:
        return

    def _json(self, status: int, body: dict) -> None:
        data = json.dumps(body).encode()
        self.send_response(status)
        self.send_header("Content-Type", "application/json")
        self.send_header("Content-Length", str(len(data)))
        self.end_headers()
        self.wfile.write(data)

    def do_GET(self) -> None:
        front: Front = self.server  # type: ignore[assignment]
        if self.path == "/health":
            status, body = front.health()
            self._json(status, body)
        elif self.path == "/metrics":  # the summed counters of all replicas, in the scraper's text format
            from ..api.server import metrics_text

            _, body = front.health()
            data = metrics_text(body).encode()
            self.send_response(200)
            self.send_header("Content-Type", "text/plain; version=0.0.4; charset=utf-8")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)
        else:
            self._relay(front.replicas[0], None)

    def do_POST(self) -> None:
        front: Front = self.server  # type: ignore[assignment]
        raw = self.rfile.read(int(self.headers.get("Content-Length") or 0))
        try:
            body = json.loads(raw or b"{}")
            chain = affinity_key(self.path, body) if isinstance(body, dict) else []
        except json.JSONDecodeError:
            chain = []
        idx = front.affinity.route(chain)
        try:
            self._relay(front.replicas[idx], raw)
        finally:
            front.affinity.finish(idx)

    def _relay(self, replica: Replica, raw: bytes | None) -> None:
        try:
            conn = http.client.HTTPConnection("127.0.0.1", replica.port, timeout=3600)
            headers = {"Content-Type": self.headers.get("Content-Type", "application/json"),
                       "X-Engine-Sent": repr(time.time())}
            if raw is None:
                conn.request("GET", self.path, headers=headers)
            else:
                conn.request("POST", self.path, body=raw, headers=headers)
            resp = conn.getresponse()
        except OSError as e:
            self._json(503, {"error": {"message": f"replica {replica.index} is unreachable: {e}",
                                       "type": "ServiceUnavailableError", "code": 503}})
            return
        try:
            self.send_response(resp.status)
            ctype = resp.getheader("Content-Type", "application/json")
            self.send_header("Content-Type", ctype)
            length = resp.getheader("Content-Length")
            if length is not None:
                self.send_header("Content-Length", length)
            else:
                self.send_header("Connection", "close")
                self.close_connection = True
            self.end_headers()
            while True:
                chunk = resp.read1(65536) if length is None else resp.read(65536)
                if not chunk:
                    break
                self.wfile.write(chunk)  # bytes pass through untouched
                self.wfile.flush()
        except (BrokenPipeError, ConnectionResetError, OSError):
            pass  # client went away: closing the upstream connection cancels the request there
        finally:
            conn.close()


class Front(ThreadingHTTPServer):
    daemon_threads = True
    allow_reuse_address = True
    request_queue_size = 256

    def __init__(self, addr: tuple[str, int], replicas: list[Replica]) -> None:
        super().__init__(addr, FrontHandler)
        self.replicas = replicas
        self.affinity = Affinity(len(replicas))

    def health(self) -> tuple[int, dict]:
        blocks, sums = [], {}
        for r in self.replicas:
            try:
                c = http.client.HTTPConnection("127.0.0.1", r.port, timeout=5)
                c.request("GET", "/health")
                resp = c.getresponse()
                body = json.loads(resp.read())
                c.close()
                if resp.status != 200:
                    raise OSError(f"status {resp.status}")
            except (OSError, json.JSONDecodeError) as e:
                return 503, {"status": "unavailable", "replica": r.index, "error": str(e)}
            blocks.append(body)
            for k, v in body.items():
                if isinstance(v, (int, float)) and not isinstance(v, bool):
                    sums[k] = sums.get(k, 0) + v
        out = {"status": "ok", "replicas": len(self.replicas), **sums, "per_replica": blocks,
               "load": [self.affinity.load(i) for i in range(len(self.replicas))],
               "routed_by_affinity": self.affinity.routed_by_affinity, "routed_by_load": self.affinity.routed_by_load}
        return 200, out


def serve(argv: list[str], host: str, port: int, layout: list[list[int]]) -> None:
    replicas = start_replicas(argv, layout)
    try:
        wait_ready(replicas)
    except BaseException:
        stop_replicas(replicas)
        raise
    front = Front((host, port), replicas)

    def watchdog() -> None:
        while True:
            for r in replicas:
                if r.proc.poll() is not None:
                    print(f"router: replica {r.index} exited ({r.proc.returncode}); stopping", flush=True)
                    stop_replicas(replicas)
                    os._exit(1)
            time.sleep(0.5)

    threading.Thread(target=watchdog, daemon=True, name="router-watchdog").start()
    print(f"router: serving {len(replicas)} replicas on http://{host}:{port}", flush=True)
    try:
        front.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        stop_replicas(replicas)
