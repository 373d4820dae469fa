"""OpenAI-compatible wire format: request parsing/validation and response builders.

Pure functions, no engine state. Accepted and rejected fields follow the reference
(``engine/protocol.py:22-44, 149-269``): completions take a string, a token-id list or a
one-element list of either; ``n`` must be 1; ``logprobs``, ``echo``, ``best_of``, ``suffix``
and ``logit_bias`` are refused; chat takes ``max_completion_tokens`` before ``max_tokens``
and defaults to the rest of the context; usage reports ``cached_tokens``.
"""

from __future__ import annotations

import json
import time
import uuid
from dataclasses import dataclass, field
from typing import Any

from ..sched.request import Sampling

REFUSED_FIELDS = ("logprobs", "top_logprobs", "echo", "best_of", "suffix", "logit_bias")


class RequestError(Exception):
    def __init__(self, message: str, status: int = 400) -> None:
        super().__init__(message)
        self.status = status


@dataclass
class CompletionRequest:
    prompt: str | list[int]
    sampling: Sampling
    stream: bool = False
    include_usage: bool = False
    return_token_ids: bool = False
    model: str | None = None


@dataclass
class ChatRequest:
    messages: list[dict[str, Any]]
    sampling: Sampling
    tools: list[dict[str, Any]] | None = None
    template_kwargs: dict[str, Any] = field(default_factory=dict)
    stream: bool = False
    include_usage: bool = False
    return_token_ids: bool = False
    model: str | None = None

    @property
    def thinking(self) -> bool:
        return self.template_kwargs.get("enable_thinking") is True


# --------------------------------------------------------------------------- parsing
def _obj(body: Any) -> dict[str, Any]:
    if not isinstance(body, dict):
        raise RequestError("the request body must be a JSON object")
    for key in REFUSED_FIELDS:
        if body.get(key) not in (None, False, 0):
            raise RequestError(f"'{key}' is not supported")
    if body.get("n", 1) != 1:
        raise RequestError("'n' must be 1")
    return body


def _num(body: dict, key: str, default: float, lo: float, hi: float) -> float:
    v = body.get(key)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not (lo <= v <= hi):
        raise RequestError(f"'{key}' must be a number between {lo} and {hi}")
    return float(v)


def _int(body: dict, key: str, default: int | None, lo: int) -> int | None:
    v = body.get(key)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, int) or v < lo:
        raise RequestError(f"'{key}' must be an integer >= {lo}")
    return v


def _stops(body: dict) -> list[str]:
    v = body.get("stop")
    if v is None:
        return []
    if isinstance(v, str):
        v = [v]
    if not isinstance(v, list) or not all(isinstance(s, str) and s for s in v):
        raise RequestError("'stop' must be a non-empty string or a list of them")
    return list(v)


def _sampling(body: dict, default_max: int | None, max_keys: tuple[str, ...]) -> Sampling:
    max_tokens = default_max
    for key in max_keys:
        if body.get(key) is not None:
            max_tokens = _int(body, key, default_max, 0)
            break
    seed = body.get("seed")
    if seed is not None and (isinstance(seed, bool) or not isinstance(seed, int)):
        raise RequestError("'seed' must be an integer")
    top_k = _int(body, "top_k", 0, -1) or 0
    return Sampling(
        max_tokens=max_tokens,
        temperature=_num(body, "temperature", 1.0, 0.0, 100.0),
        top_p=_num(body, "top_p", 1.0, 0.0, 1.0) or 1.0,
        top_k=max(top_k, 0),
        seed=seed,
        stop=_stops(body),
        ignore_eos=bool(body.get("ignore_eos", False)),
        min_tokens=_int(body, "min_tokens", 0, 0) or 0,
    )


def _stream_flags(body: dict) -> tuple[bool, bool, bool]:
    stream = bool(body.get("stream", False))
    opts = body.get("stream_options") or {}
    if not isinstance(opts, dict):
        raise RequestError("'stream_options' must be an object")
    return stream, bool(opts.get("include_usage", False)), bool(body.get("return_token_ids", False))


def _token_list(v: Any) -> list[int] | None:
    if isinstance(v, list) and v and all(isinstance(t, int) and not isinstance(t, bool) for t in v):
        return list(v)
    return None


def parse_completion(body: Any) -> CompletionRequest:
    body = _obj(body)
    prompt = body.get("prompt")
    if isinstance(prompt, list) and len(prompt) == 1 and isinstance(prompt[0], (str, list)):
        prompt = prompt[0]  # a one-element batch
    ids = _token_list(prompt)
    if ids is not None:
        prompt = ids
    elif not isinstance(prompt, str) or not prompt:
        raise RequestError("'prompt' must be a non-empty string or a list of token ids")
    stream, usage, with_ids = _stream_flags(body)
    return CompletionRequest(prompt, _sampling(body, 16, ("max_tokens",)), stream, usage, with_ids, body.get("model"))


def parse_chat(body: Any) -> ChatRequest:
    body = _obj(body)
    messages = body.get("messages")
    if not isinstance(messages, list) or not messages or not all(isinstance(m, dict) and "role" in m for m in messages):
        raise RequestError("'messages' must be a non-empty list of {role, content} objects")
    messages = [_normalise_message(m) for m in messages]
    tools = body.get("tools")
    if tools is not None and (not isinstance(tools, list) or not all(isinstance(t, dict) for t in tools)):
        raise RequestError("'tools' must be a list of objects")
    kwargs = body.get("chat_template_kwargs") or {}
    if not isinstance(kwargs, dict):
        raise RequestError("'chat_template_kwargs' must be an object")
    stream, usage, with_ids = _stream_flags(body)
    sampling = _sampling(body, None, ("max_completion_tokens", "max_tokens"))
    return ChatRequest(messages, sampling, tools or None, dict(kwargs), stream, usage, with_ids, body.get("model"))


def _normalise_message(m: dict[str, Any]) -> dict[str, Any]:
    """Tool-call arguments arrive as JSON strings; templates iterate them as mappings."""
    calls = m.get("tool_calls")
    if not calls:
        return m
    out = dict(m)
    fixed = []
    for call in calls:
        call = dict(call)
        fn = dict(call.get("function") or {})
        args = fn.get("arguments")
        if isinstance(args, str):
            try:
                fn["arguments"] = json.loads(args)
            except json.JSONDecodeError:
                raise RequestError("tool call arguments must be a JSON object") from None
        if fn:
            call["function"] = fn
        fixed.append(call)
    out["tool_calls"] = fixed
    return out


# --------------------------------------------------------------------------- responses
@dataclass
class Usage:
    prompt_tokens: int
    cached_tokens: int = 0
    completion_tokens: int = 0

    def body(self) -> dict[str, Any]:
        return {
            "prompt_tokens": self.prompt_tokens,
            "completion_tokens": self.completion_tokens,
            "total_tokens": self.prompt_tokens + self.completion_tokens,
            "prompt_tokens_details": {"cached_tokens": self.cached_tokens},
        }


@dataclass
class Envelope:
    model: str
    kind: str  # "text_completion" | "chat.completion"
    id: str = field(default_factory=lambda: "cmpl-" + uuid.uuid4().hex)
    created: int = field(default_factory=lambda: int(time.time()))

    def head(self, chunk: bool = False) -> dict[str, Any]:
        obj = self.kind + (".chunk" if chunk and self.kind == "chat.completion" else "")
        return {"id": self.id, "object": obj, "created": self.created, "model": self.model}


def _choice(payload: dict[str, Any], finish: str | None, token_ids: list[int] | None) -> dict[str, Any]:
    c = {"index": 0, **payload, "logprobs": None, "finish_reason": finish}
    if token_ids is not None:
        c["token_ids"] = token_ids
    return c


def completion_chunk(env: Envelope, text: str, token: int | None, finish: str | None, with_ids: bool) -> dict:
    ids = ([] if token is None else [token]) if with_ids else None
    return {**env.head(True), "choices": [_choice({"text": text}, finish, ids)]}


def chat_chunk(env: Envelope, delta: dict[str, Any], token: int | None, finish: str | None, with_ids: bool) -> dict:
    ids = ([] if token is None else [token]) if with_ids else None
    return {**env.head(True), "choices": [_choice({"delta": delta}, finish, ids)]}


def usage_chunk(env: Envelope, usage: Usage) -> dict:
    return {**env.head(True), "choices": [], "usage": usage.body()}


def completion_response(env: Envelope, text: str, ids: list[int], finish: str, usage: Usage, with_ids: bool) -> dict:
    return {**env.head(), "choices": [_choice({"text": text}, finish, ids if with_ids else None)], "usage": usage.body()}


def chat_response(env: Envelope, content: str, reasoning: str | None, ids: list[int], finish: str, usage: Usage,
                  with_ids: bool) -> dict:
    msg: dict[str, Any] = {"role": "assistant", "content": content}
    if reasoning is not None:
        msg["reasoning_content"] = reasoning
    return {**env.head(), "choices": [_choice({"message": msg}, finish, ids if with_ids else None)], "usage": usage.body()}


def error_body(message: str, status: int) -> dict:
    kinds = {404: "NotFoundError", 503: "ServiceUnavailableError", 500: "InternalServerError"}
    return {"error": {"message": message, "type": kinds.get(status, "BadRequestError"), "code": status}}


def models_body(model: str, max_model_len: int) -> dict:
    return {"object": "list", "data": [{"id": model, "object": "model", "owned_by": "b200serve",
                                        "max_model_len": max_model_len}]}
