"""OpenAI-compatible HTTP server: ``/health``, ``/v1/models``, ``/v1/completions``,
``/v1/chat/completions`` (streaming over SSE or not).

Threads: one engine worker owns the model and runs ``Engine.step()``; every HTTP connection has
its own handler thread that parses, tokenises, answers refusals and sends the first chunk; from
then on ONE writer thread (``StreamWriter``) turns the token events of all requests into text
(incremental detokenisation, stop strings, reasoning/content split) and writes the SSE chunks,
so a decode step of 128 requests wakes one thread instead of 128 (``ENGINE_STREAM_WRITER=0``:
every handler thread consumes its own events, as before). The port opens only after the weights
are loaded, so ``/health`` 200 means ready (reference: ``engine/server.py:1-21, 488-620, 623-729``;
there, detokenisation runs on the engine thread).
"""

from __future__ import annotations

import argparse
import json
import os
import queue
import socket
import sys
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any, Iterator

from ..config import EngineConfig
from ..obs import buildlog, looptimers, reqstamps
from ..sched.request import EngineError, Generation, TokenEvent  # noqa: F401 - named in annotations
from . import protocol
from .protocol import ChatRequest, CompletionRequest, Envelope, RequestError, Usage
from .text import Detokenizer, StopMatcher


class EngineWorker(threading.Thread):
    """The only thread that touches the model."""

    def __init__(self, engine) -> None:
        super().__init__(name="engine-worker", daemon=True)
        self.engine = engine
        self.wake = threading.Event()
        self.stopping = False
        self.fatal: BaseException | None = None
        self.fatal_streak = 0  # consecutive iterations that raised: the loop is wedged when this keeps growing

    def submit(self, gen: Generation) -> None:
        self.engine.submit(gen)
        self.wake.set()

    def run(self) -> None:
        eng = self.engine
        if getattr(eng.device, "type", "cpu") == "cuda":
            # the current CUDA device is a property of the host thread and starts at 0 in every new thread: without
            # this, a replica on any other device would launch its kernels on device 0's stream
            import torch

            torch.cuda.set_device(eng.device)
        # ENGINE_STALL_DUMP_S = N: when one iteration of the loop takes longer than N seconds, the stacks of all threads
        # are written to stderr (once per stall), so that a wedged replica shows where it waits
        stall = float(os.environ.get("ENGINE_STALL_DUMP_S", "0") or 0)
        if stall > 0:
            import faulthandler
        while not self.stopping:
            try:
                if stall > 0:
                    faulthandler.dump_traceback_later(stall, repeat=False, exit=False)
                looptimers.begin()
                busy = eng.step()
                looptimers.end(len(eng.running))
                self.fatal_streak = 0
            except BaseException as e:  # noqa: BLE001 - keep the failure visible on /health
                self.fatal = e
                self.fatal_streak += 1
                import traceback

                traceback.print_exc()
                try:  # nobody may be left waiting on a request this loop can no longer advance
                    eng.fail_all(f"engine loop failed: {e!r}")
                except Exception:  # noqa: BLE001
                    traceback.print_exc()
                time.sleep(0.05)
                continue
            if not busy and not eng.has_work():
                # replicas that run their passes together agree before every pass: an idle one must come back quickly,
                # or it holds up the others' requests
                self.wake.wait(timeout=0.001 if eng.tick is not None and eng.broken is None else 0.05)
                self.wake.clear()

    def stop(self) -> None:
        self.stopping = True
        self.wake.set()


class _TextStream:
    """Token events -> (reasoning delta, content delta), with stop strings applied to content."""

    def __init__(self, codec, stops: list[str], thinking: bool) -> None:
        self.codec = codec
        self.in_reasoning = thinking
        self.detok = Detokenizer(codec.tok)
        self.matcher = StopMatcher(stops)
        self.content: list[str] = []
        self.reasoning: list[str] = []

    @property
    def stopped(self) -> bool:
        return self.matcher.stopped

    def push(self, token: int) -> tuple[str, str]:
        if self.in_reasoning and token == self.codec.think_end_id:
            tail = self.detok.flush()
            self.reasoning.append(tail)
            self.in_reasoning = False
            self.detok = Detokenizer(self.codec.tok)
            return tail, ""
        text = self.detok.push(token)
        if self.in_reasoning:
            self.reasoning.append(text)
            return text, ""
        out = self.matcher.push(text)
        self.content.append(out)
        return "", out

    def flush(self) -> tuple[str, str]:
        tail = self.detok.flush()
        if self.in_reasoning:
            self.reasoning.append(tail)
            return tail, ""
        out = self.matcher.push(tail) + self.matcher.flush()
        self.content.append(out)
        return "", out


class RequestState:
    """Token events of one request -> response objects: chunks (and an optional usage chunk) when streaming, else
    one body at the end. Push style, so that either the request's own thread or the shared writer can drive it."""

    def __init__(self, service, request: CompletionRequest | ChatRequest, prompt_len: int, gen: Generation) -> None:
        self.service, self.request, self.gen = service, request, gen
        self.chat = isinstance(request, ChatRequest)
        self.env = Envelope(service.model_name, "chat.completion" if self.chat else "text_completion")
        self.text = _TextStream(service.codec, request.sampling.stop, self.chat and request.thinking)
        self.usage = Usage(prompt_len)
        self.ids: list[int] = []
        self.first = True

    def feed(self, ev: TokenEvent) -> tuple[list[dict[str, Any]], bool]:
        """Returns ``(objects to send now, the request is finished)``; raises ``RequestError`` for an error event."""
        request, chat, env, text, usage = self.request, self.chat, self.env, self.text, self.usage
        if ev.error is not None:
            raise RequestError(str(ev.error), ev.error.status)
        out: list[dict[str, Any]] = []
        if self.first:
            self.first = False
            usage.cached_tokens = self.gen.cached_tokens
            if request.stream and chat:
                out.append(protocol.chat_chunk(env, {"role": "assistant", "content": ""}, None, None,
                                               request.return_token_ids))
        reasoning = content = ""
        if ev.token is not None:
            self.ids.append(ev.token)
            usage.completion_tokens += 1
            reasoning, content = text.push(ev.token)
        done = ev.finish_reason
        if text.stopped:
            done = "stop"
            self.gen.cancelled.set()
            self.service.worker.wake.set()
        elif done is not None:
            r2, c2 = text.flush()
            reasoning, content = reasoning + r2, content + c2
            if text.stopped:
                done = "stop"
        if done == "cancelled":
            done = "stop"
        if request.stream:
            if chat:
                delta: dict[str, Any] = {"content": content}
                if reasoning:
                    delta = {"reasoning_content": reasoning, **({"content": content} if content else {})}
                out.append(protocol.chat_chunk(env, delta, ev.token, done, request.return_token_ids))
            else:
                out.append(protocol.completion_chunk(env, content, ev.token, done, request.return_token_ids))
        if done is None:
            return out, False
        if request.stream:
            if request.include_usage:
                out.append(protocol.usage_chunk(env, usage))
        elif chat:
            out.append(protocol.chat_response(env, "".join(text.content),
                                              "".join(text.reasoning) if request.thinking else None, self.ids, done,
                                              usage, request.return_token_ids))
        else:
            out.append(protocol.completion_response(env, "".join(text.content), self.ids, done, usage,
                                                    request.return_token_ids))
        return out, True


def sse(objects: list[dict[str, Any]]) -> bytes:
    return b"".join(b"data: " + json.dumps(o).encode() + b"\n\n" for o in objects)


class Stream:
    """One request between its handler thread and the shared writer. Events first queue up for the handler thread
    (``next_direct``: refusals must become HTTP statuses, and the first chunk follows the headers), then
    ``hand_over`` redirects them, in order, to the writer thread, and the handler sleeps until ``finished``."""

    def __init__(self, service, request: CompletionRequest | ChatRequest, prompt: list[int]) -> None:
        self.service = service
        self.q: "queue.SimpleQueue[TokenEvent]" = queue.SimpleQueue()
        self.lock = threading.Lock()
        self.to_writer = False
        self.gen = Generation(prompt, request.sampling, on_event=self._sink)
        self.state = RequestState(service, request, len(prompt), self.gen)
        self.sock: socket.socket | None = None  # set for SSE responses: the writer sends on it
        self.backlog = bytearray()  # bytes the socket did not take yet
        self.objects: list[dict[str, Any]] = []  # non-streaming: the body, once finished
        self.error: RequestError | None = None
        self.dead = False  # the client went away
        self.finished = threading.Event()

    def _sink(self, gen: Generation, ev: TokenEvent) -> None:  # engine thread
        with self.lock:
            if self.to_writer:
                self.service.writer.inbox.put((self, ev))
            else:
                self.q.put(ev)

    def next_direct(self) -> tuple[list[dict[str, Any]], bool]:
        """Handler thread, before the hand-over: wait for the next event and run it through the state machine."""
        return self.state.feed(self.q.get())

    def hand_over(self, sock: socket.socket | None) -> None:
        """From here on the writer thread consumes this request's events (those already queued go first)."""
        with self.lock:
            self.sock = sock
            while True:
                try:
                    self.service.writer.inbox.put((self, self.q.get_nowait()))
                except queue.Empty:
                    break
            self.to_writer = True

    def cancel(self) -> None:
        if not self.gen.done:
            self.gen.cancelled.set()
            self.service.worker.wake.set()


class StreamWriter(threading.Thread):
    """The one thread that turns token events of all handed-over requests into response bytes. SSE chunks go out
    with non-blocking sends; what a socket does not take is kept per request and retried (a client that stops
    reading cannot stall the others; past ``MAX_BACKLOG`` bytes it is treated as gone). When a request finishes,
    its handler thread wakes once, sends any remainder with a blocking write and closes the connection."""

    MAX_BACKLOG = 8 << 20

    def __init__(self) -> None:
        super().__init__(daemon=True, name="stream-writer")
        self.inbox: "queue.SimpleQueue[tuple[Stream, TokenEvent] | None]" = queue.SimpleQueue()
        self.backlogged: set[Stream] = set()
        self.stats = {"writer_batches": 0, "writer_events": 0, "writer_partial_sends": 0}

    def run(self) -> None:
        while True:
            try:
                item = self.inbox.get(timeout=0.01 if self.backlogged else None)
            except queue.Empty:
                item = False
            if item is None:
                return
            batch = [item] if item else []
            while True:
                try:
                    nxt = self.inbox.get_nowait()
                except queue.Empty:
                    break
                if nxt is None:
                    return
                batch.append(nxt)
            self.stats["writer_batches"] += 1
            self.stats["writer_events"] += len(batch)
            for stream, ev in batch:
                try:
                    self._handle(stream, ev)
                except Exception as e:  # noqa: BLE001 - one request's failure must not end the thread
                    stream.error = stream.error or RequestError(f"internal error: {e}", 500)
                    stream.cancel()
                    self._finish(stream)
            for stream in list(self.backlogged):
                try:
                    self._send(stream, b"")
                except Exception:  # noqa: BLE001
                    stream.dead = True
                    stream.cancel()
                    self._finish(stream)

    def stop(self) -> None:
        self.inbox.put(None)

    def _handle(self, stream: Stream, ev: TokenEvent) -> None:
        if stream.finished.is_set():
            return  # events after the end (a cancelled request's last event)
        try:
            out, done = stream.state.feed(ev)
        except RequestError as e:
            stream.error = e
            self._finish(stream)
            return
        if stream.sock is None:
            stream.objects.extend(out)
        else:
            self._send(stream, sse(out) + (b"data: [DONE]\n\n" if done else b""))
        if done and not stream.finished.is_set():
            self._finish(stream)

    def _send(self, stream: Stream, data: bytes) -> None:
        if stream.dead:
            return
        buf = stream.backlog
        if buf:
            buf += data
            data = bytes(buf)
        if not data:
            return
        try:
            n = stream.sock.send(data, socket.MSG_DONTWAIT)  # type: ignore[union-attr]
        except (BlockingIOError, InterruptedError):
            n = 0
        except OSError:  # the client went away: stop generating for it
            stream.dead = True
            stream.cancel()
            self._finish(stream)
            return
        if n == len(data):
            buf.clear()
            self.backlogged.discard(stream)
            return
        self.stats["writer_partial_sends"] += 1
        del buf[:]
        buf += data[n:]
        self.backlogged.add(stream)
        if len(buf) > self.MAX_BACKLOG:
            stream.dead = True
            stream.cancel()
            self._finish(stream)

    def _finish(self, stream: Stream) -> None:
        self.backlogged.discard(stream)
        stream.finished.set()


class Service:
    """Everything the handlers need: engine worker, tokenizer, served model name."""

    def __init__(self, engine, codec, model_name: str) -> None:
        self.engine = engine
        self.codec = codec
        self.model_name = model_name
        self.worker = EngineWorker(engine)
        self.worker.start()
        self.writer: StreamWriter | None = None
        if os.environ.get("ENGINE_STREAM_WRITER", "1") == "1":
            self.writer = StreamWriter()
            self.writer.start()

    # ------------------------------------------------------------------ request -> events
    def _events(self, prompt: list[int], sampling) -> tuple[Generation, "queue.Queue[TokenEvent]"]:
        q: "queue.Queue[TokenEvent]" = queue.Queue()
        gen = Generation(prompt, sampling, on_event=lambda g, e: q.put(e))
        self.worker.submit(gen)
        return gen, q

    def run(self, request: CompletionRequest | ChatRequest, prompt: list[int]) -> Iterator[dict[str, Any]]:
        """Yield response objects: chunks (and an optional usage chunk) when streaming, else one body.

        Raises ``RequestError`` before the first yield when the engine refuses the request.
        """
        gen, q = self._events(prompt, request.sampling)
        state = RequestState(self, request, len(prompt), gen)
        try:
            while True:
                out, done = state.feed(q.get())
                yield from out
                if done:
                    break
        finally:
            if not gen.done:
                gen.cancelled.set()  # client went away or the consumer stopped early
                self.worker.wake.set()

    def open(self, request: CompletionRequest | ChatRequest, prompt: list[int]) -> "Stream":
        """Submit the request; its events are consumed through the returned ``Stream`` (first by the caller, then by
        the shared writer thread)."""
        stream = Stream(self, request, prompt)
        self.worker.submit(stream.gen)
        return stream

    def tokenize(self, request: CompletionRequest | ChatRequest) -> list[int]:
        if isinstance(request, ChatRequest):
            try:
                return self.codec.encode_chat(request.messages, request.tools, **request.template_kwargs)
            except RequestError:
                raise
            except Exception as e:  # jinja raises many kinds
                raise RequestError(f"the chat template rejected the messages: {e}") from e
        if isinstance(request.prompt, str):
            return self.codec.encode(request.prompt)
        return list(request.prompt)

    def health(self) -> dict[str, Any]:
        # "ok": serving. "degraded": the engine loop raised at some point but recovered. "unavailable": the rank group
        # was torn down or the loop keeps raising; /health then answers 503 so that a front takes the replica out.
        if self.engine.broken is not None or self.worker.fatal_streak >= 3:
            status = "unavailable"
        else:
            status = "ok" if self.worker.fatal is None else "degraded"
        body: dict[str, Any] = {"status": status}
        if self.worker.fatal is not None:
            body["last_loop_error"] = repr(self.worker.fatal)
        body.update(self.engine.health())
        if self.codec is not None:
            body.update(self.codec.encoder.stats)
        if self.writer is not None:
            body.update(self.writer.stats)
        if looptimers.ENABLED:
            body["loop_timers"] = looptimers.summary()
        if reqstamps.ENABLED:
            body["request_stamps"] = reqstamps.summary()
        body["native_loads"] = len(buildlog.events())
        body["native_loads_while_serving"] = len(buildlog.events(serving_only=True))
        return body


def metrics_text(health: dict[str, Any]) -> str:
    """The numeric fields of ``/health`` in the Prometheus text exposition format (one gauge each, prefix
    ``engine_``), plus ``engine_up`` (1 while the status is ``ok`` or ``degraded``). The reference reports its
    counters on ``/health`` only (``engine/server.py:498-512``); this is the same data for a scraper."""
    lines = ["# TYPE engine_up gauge", f"engine_up {0 if health.get('status') == 'unavailable' else 1}"]
    for key in sorted(health):
        v = health[key]
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            continue
        name = "engine_" + "".join(c if c.isalnum() else "_" for c in key)
        lines += [f"# TYPE {name} gauge", f"{name} {v}"]
    return "\n".join(lines) + "\n"


class Handler(BaseHTTPRequestHandler):
    protocol_version = "HTTP/1.1"
    service: Service  # set on the server class

    def log_message(self, fmt: str, *args: Any) -> None:  # quiet
        return

    # ------------------------------------------------------------------ helpers
    def _json(self, status: int, body: dict[str, Any]) -> None:
        data = json.dumps(body).encode()
        self.send_response(status)
        self.send_header("Content-Type", "application/json")
        self.send_header("Content-Length", str(len(data)))
        self.end_headers()
        self.wfile.write(data)

    def _error(self, message: str, status: int) -> None:
        self._json(status, protocol.error_body(message, status))

    # ------------------------------------------------------------------ routes
    def do_GET(self) -> None:
        svc = self.server.service  # type: ignore[attr-defined]
        if self.path == "/health":
            body = svc.health()
            self._json(503 if body["status"] == "unavailable" else 200, body)
        elif self.path == "/v1/models":
            self._json(200, protocol.models_body(svc.model_name, svc.engine.max_model_len))
        elif self.path == "/metrics":
            data = metrics_text(svc.health()).encode()
            self.send_response(200)
            self.send_header("Content-Type", "text/plain; version=0.0.4; charset=utf-8")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)
        else:
            self._error(f"no route {self.path}", 404)

    def do_POST(self) -> None:
        svc: Service = self.server.service  # type: ignore[attr-defined]
        stamp = reqstamps.start(self.headers.get("X-Engine-Sent"))
        try:
            length = int(self.headers.get("Content-Length") or 0)
            raw = self.rfile.read(length)
            try:
                body = json.loads(raw or b"{}")
            except json.JSONDecodeError:
                raise RequestError("the request body is not valid JSON") from None
            if self.path == "/v1/completions":
                request = protocol.parse_completion(body)
            elif self.path == "/v1/chat/completions":
                request = protocol.parse_chat(body)
            else:
                raise RequestError(f"no route {self.path}", 404)
            if request.model is not None and request.model != svc.model_name:
                raise RequestError(f"model {request.model!r} is not served here (serving {svc.model_name!r})", 404)
            reqstamps.mark(stamp, "parsed")
            prompt = svc.tokenize(request)
            svc.engine.validate(prompt, request.sampling)
            reqstamps.mark(stamp, "tokenized")
            if svc.writer is not None:
                self._respond_shared(svc, request, prompt, stamp)
                return
            events = svc.run(request, prompt)
            first = next(events)  # engine refusals surface here, before any header is sent
        except RequestError as e:
            self._error(str(e), e.status)
            return
        except EngineError as e:
            self._error(str(e), e.status)
            return
        except StopIteration:
            self._error("the request produced no response", 500)
            return
        except Exception as e:  # noqa: BLE001
            self._error(f"internal error: {e}", 500)
            return
        reqstamps.mark(stamp, "first_event")
        if not request.stream:
            self._json(200, first)
            reqstamps.finish(stamp)
            return
        try:
            self.send_response(200)
            self.send_header("Content-Type", "text/event-stream")
            self.send_header("Cache-Control", "no-cache")
            self.send_header("Connection", "close")
            self.end_headers()
            self.wfile.write(b"data: " + json.dumps(first).encode() + b"\n\n")
            self.wfile.flush()
            reqstamps.mark(stamp, "first_byte")
            for ev in events:
                self.wfile.write(b"data: " + json.dumps(ev).encode() + b"\n\n")
                self.wfile.flush()
            self.wfile.write(b"data: [DONE]\n\n")
            self.wfile.flush()
        except (BrokenPipeError, ConnectionResetError, OSError):
            events.close()  # runs the generator's finally: cancels the generation
        finally:
            self.close_connection = True
            reqstamps.finish(stamp)

    @staticmethod
    def _await(svc: "Service", stream: "Stream") -> None:
        """Sleep until the writer thread has finished the request (and notice if that thread is gone)."""
        while not stream.finished.wait(2.0):
            if not svc.writer.is_alive():
                stream.error = stream.error or RequestError("the response writer stopped", 500)
                stream.cancel()
                return

    def _respond_shared(self, svc: "Service", request, prompt: list[int], stamp) -> None:
        """Answer through the shared writer thread: this thread handles refusals, the headers and the first chunk,
        then sleeps until the request is finished."""
        stream = svc.open(request, prompt)
        try:
            if not request.stream:
                stream.hand_over(None)
                self._await(svc, stream)
                reqstamps.mark(stamp, "first_event")
                if stream.error is not None:
                    self._error(str(stream.error), stream.error.status)
                elif not stream.objects:
                    self._error("the request produced no response", 500)
                else:
                    self._json(200, stream.objects[-1])
                return
            try:
                out, done = stream.next_direct()  # engine refusals surface here, before any header is sent
            except RequestError as e:
                self._error(str(e), e.status)
                return
            reqstamps.mark(stamp, "first_event")
            self.send_response(200)
            self.send_header("Content-Type", "text/event-stream")
            self.send_header("Cache-Control", "no-cache")
            self.send_header("Connection", "close")
            self.end_headers()
            self.wfile.write(sse(out) + (b"data: [DONE]\n\n" if done else b""))
            self.wfile.flush()
            reqstamps.mark(stamp, "first_byte")
            if not done:
                stream.hand_over(self.connection)
                self._await(svc, stream)
                if stream.backlog and not stream.dead:
                    self.wfile.write(bytes(stream.backlog))  # what the socket had not taken yet: a blocking write now
                    self.wfile.flush()
        except (BrokenPipeError, ConnectionResetError, OSError):
            pass
        except Exception as e:  # noqa: BLE001
            try:
                self._error(f"internal error: {e}", 500)
            except OSError:
                pass
        finally:
            stream.cancel()  # no-op when the generation is done: the client went away or this thread stopped early
            if request.stream:
                self.close_connection = True
            reqstamps.finish(stamp)


class Server(ThreadingHTTPServer):
    daemon_threads = True
    allow_reuse_address = True
    request_queue_size = 256

    def __init__(self, addr: tuple[str, int], service: Service) -> None:
        super().__init__(addr, Handler)
        self.service = service


# --------------------------------------------------------------------------- process entry
def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="b200serve", description="B200-native Qwen3.6-35B-A3B serving engine")
    env = os.environ.get
    ap.add_argument("--model", required=True, help="checkpoint directory (HF layout)")
    ap.add_argument("--revision", default=None)
    ap.add_argument("--served-model-name", default=None)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--max-model-len", type=int, default=262144)
    ap.add_argument("--prefill-chunk-tokens", type=int, default=2048)
    ap.add_argument("--prefix-cache-tokens", type=int, default=4194304)
    ap.add_argument("--prefix-cache-entries", type=int, default=128)
    ap.add_argument("--prefix-cache-gib", type=float, default=16.0)
    ap.add_argument("--experts-implementation", default=None, help="accepted for compatibility; one implementation exists")
    ap.add_argument("--replicas", type=int, default=int(env("ENGINE_REPLICAS", "0")) or None)
    ap.add_argument("--gpus-per-replica", type=int, default=int(env("ENGINE_GPUS_PER_REPLICA", "0")) or None)
    ap.add_argument("--replica-devices", default=env("ENGINE_REPLICA_DEVICES"))
    ap.add_argument("--device", default=env("ENGINE_DEVICE", "auto"), choices=["auto", "cpu", "cuda"])
    ap.add_argument("--max-seqs", type=int, default=int(env("ENGINE_SLOTS", "128")))
    ap.add_argument("--replica-split", default=env("ENGINE_REPLICA_SPLIT", "tensor"), choices=["tensor", "layers"],
                    help="how a replica of several GPUs (--gpus-per-replica) divides the model: every layer sharded "
                         "across them, or a run of whole layers on each (a capacity measure: one GPU computes at a time)")
    ap.add_argument("--expert-parallel", action="store_true", default=env("ENGINE_EP", "0") not in ("", "0"),
                    help="the replicas of this server form one expert-parallel group: each holds all dense weights and "
                         "1/N of the routed experts (one GPU per replica)")
    return ap


def load_service(args: argparse.Namespace) -> Service:
    import torch

    from ..models.checkpoint import load_checkpoint
    from ..sched.engine import Engine
    from .tokenizer import TextCodec

    use_cuda = args.device == "cuda" or (args.device == "auto" and torch.cuda.is_available())
    t0 = time.time()
    cfg = EngineConfig.from_env(
        model=args.model, max_model_len=args.max_model_len, prefill_chunk_tokens=args.prefill_chunk_tokens,
        prefix_cache_tokens=args.prefix_cache_tokens, prefix_cache_entries=args.prefix_cache_entries,
        prefix_cache_gib=args.prefix_cache_gib, max_seqs=args.max_seqs,
    )
    if os.environ.get("ENGINE_PACK_WEIGHTS") is None:
        cfg.pack_weights = True  # the server owns the weights it loads: stream them tile-packed
    tp = int(args.gpus_per_replica or os.environ.get("ENGINE_TP", "1") or 1)
    followers = []
    from ..parallel import dpep

    if dpep.env_group() is not None:
        # one of N replicas that share their MoE blocks (data-parallel attention, expert-parallel experts)
        tp = 1
        weights = None
        if args.model.startswith("random:"):
            import tempfile

            from ..config import ModelConfig
            from ..models.checkpoint import random_weights
            from ..models.tiny import build_tokenizer

            device = torch.device("cuda", dpep.env_group()[3]) if use_cuda else torch.device("cpu")
            mcfg = ModelConfig.tiny() if args.model == "random:tiny" else ModelConfig.qwen36_35b_a3b()
            weights = random_weights(mcfg, seed=0, device=device, dtype=torch.bfloat16 if use_cuda else torch.float32)
            tok_dir = tempfile.mkdtemp(prefix="b200serve-tok-")
            build_tokenizer(512).save_pretrained(tok_dir)
            args.model_dir_for_tokenizer = tok_dir
        engine = dpep.build_engine(args.model, cfg, use_cuda, weights=weights)
        device = engine.device
    elif tp > 1:  # a tensor-parallel replica: this process is rank 0, the other ranks are child processes
        from ..parallel import replica

        passthrough = ["--max-model-len", str(args.max_model_len), "--prefill-chunk-tokens",
                       str(args.prefill_chunk_tokens), "--prefix-cache-tokens", str(args.prefix_cache_tokens),
                       "--prefix-cache-entries", str(args.prefix_cache_entries), "--prefix-cache-gib",
                       str(args.prefix_cache_gib), "--max-seqs", str(args.max_seqs)]
        engine, followers = replica.leader_engine(args.model, tp, use_cuda, cfg, passthrough, split=args.replica_split)
        device = engine.device
    elif args.model.startswith("random:"):
        # benchmark mode: random-init weights of a named architecture created on the device, no checkpoint on disk
        import tempfile

        from ..config import ModelConfig
        from ..models.checkpoint import random_weights
        from ..models.tiny import build_tokenizer

        device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
        dtype = torch.bfloat16 if use_cuda else torch.float32
        mcfg = ModelConfig.tiny() if args.model == "random:tiny" else ModelConfig.qwen36_35b_a3b()
        engine = Engine(random_weights(mcfg, seed=0, device=device, dtype=dtype), cfg)
        tok_dir = tempfile.mkdtemp(prefix="b200serve-tok-")
        build_tokenizer(512).save_pretrained(tok_dir)
        args.model_dir_for_tokenizer = tok_dir
    else:
        device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
        dtype = torch.bfloat16 if use_cuda else torch.float32
        engine = Engine(load_checkpoint(args.model, device=device, dtype=dtype), cfg)
    if tp == 1 and os.environ.get("ENGINE_WARMUP", "1") == "1":
        engine.warmup()
    codec = TextCodec(getattr(args, "model_dir_for_tokenizer", args.model))
    name = args.served_model_name or args.model
    print(f"engine: loaded {args.model} on {device} tp={tp} ({engine.model.w.nbytes() / 1e9:.2f} GB per rank) in "
          f"{time.time() - t0:.1f} s; kv_pages={engine.pages.num_pages} slots={engine.slots.num_slots} "
          f"mtp={engine.spec is not None}", flush=True)
    service = Service(engine, codec, name)
    service.followers = followers
    return service


def main(argv: list[str] | None = None) -> None:
    args = build_parser().parse_args(argv)
    from ..router import router

    if args.expert_parallel:
        os.environ["ENGINE_EP"] = "1"
    layout = router.resolve_layout(args.replicas, args.gpus_per_replica, args.replica_devices)
    if layout is not None and len(layout) > 1:
        router.serve(sys.argv[1:] if argv is None else argv, args.host, args.port, layout)
        return
    service = load_service(args)
    server = Server((args.host, args.port), service)
    buildlog.mark_serving()  # any native load from here on is a stall a request can see
    print(f"engine: serving {service.model_name} on http://{args.host}:{args.port}", flush=True)
    try:
        server.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        service.worker.stop()
        if service.engine.tick is not None:
            service.worker.join(timeout=5)
            service.engine.tick.stop(service.engine)
        if service.engine.coordinator is not None:
            service.worker.join(timeout=5)
            service.engine.coordinator.stop(service.engine)
        for p in getattr(service, "followers", []):
            p.terminate()


if __name__ == "__main__":
    main()
