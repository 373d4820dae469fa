"""HTTP contract of the server on a tiny random checkpoint served on the CPU in fp32.

The list of behaviours follows the reference's contract tests
(``.vibesys/shared/cpu_check/test_engine_contract.py:63-297``): exact lengths under ``ignore_eos``,
one SSE event per token, usage with cached tokens, cache reuse that never changes outputs, EOS and
``min_tokens``, stop strings, chat thinking switches, refusals, and batching that leaves every
request's tokens equal to the same request served alone.
"""

from concurrent.futures import ThreadPoolExecutor

import pytest
import requests

from http_util import CHUNK, ServerProc, ids_of


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    from b200serve.models.tiny import write_tiny_checkpoint

    path = tmp_path_factory.mktemp("tiny-ckpt")
    write_tiny_checkpoint(path, lm_head_std=0.5)
    return path


@pytest.fixture(scope="module")
def server(model_dir):
    s = ServerProc(model_dir)
    yield s
    s.stop()


@pytest.fixture(scope="module")
def cold_server(model_dir):
    s = ServerProc(model_dir, extra=["--prefix-cache-entries", "0"])
    yield s
    s.stop()


def test_health_and_models(server):
    assert requests.get(server.url + "/health").status_code == 200
    models = requests.get(server.url + "/v1/models").json()
    assert [m["id"] for m in models["data"]] == [server.model]
    assert models["data"][0]["max_model_len"] == 2048


@pytest.mark.parametrize("max_tokens", [1, 2, 7, 33])
def test_ignore_eos_streams_exactly_the_requested_tokens(server, max_tokens):
    prompt = list(range(40, 40 + 11 + max_tokens))
    chunks, usage = server.completion(prompt, max_tokens)
    assert len(chunks) == max_tokens
    assert all(len(c["choices"][0]["token_ids"]) == 1 for c in chunks)
    assert [c["choices"][0]["finish_reason"] for c in chunks] == [None] * (max_tokens - 1) + ["length"]
    assert usage["prompt_tokens"] == len(prompt)
    assert usage["completion_tokens"] == max_tokens
    assert usage["total_tokens"] == len(prompt) + max_tokens


def test_repeated_prompt_reports_cache_hit_and_repeats_tokens(server):
    prompt = list(range(100, 100 + 3 * CHUNK + 5))
    first, u1 = server.completion(prompt, 12)
    second, u2 = server.completion(prompt, 12)
    assert u1["prompt_tokens_details"]["cached_tokens"] == 0
    cached = u2["prompt_tokens_details"]["cached_tokens"]
    assert 0 < cached <= len(prompt) - 1
    assert ids_of(second) == ids_of(first)


@pytest.mark.parametrize("extra", [1, CHUNK - 1, CHUNK, 3 * CHUNK + 2])
def test_reusing_a_prefix_never_changes_the_output(server, cold_server, extra):
    base = [7 + (i * 13) % 250 + extra for i in range(2 * CHUNK + 3 + extra)]
    server.completion(base, 2)
    grown = base + [9 + (i * 7) % 250 for i in range(extra + 4)]
    warm, wu = server.completion(grown, 16)
    cold, cu = cold_server.completion(grown, 16)
    cached = wu["prompt_tokens_details"]["cached_tokens"]
    assert cached == (len(base) - 1) // CHUNK * CHUNK  # the last chunk boundary inside the shared prefix
    assert cu["prompt_tokens_details"]["cached_tokens"] == 0
    assert ids_of(warm) == ids_of(cold)


def test_session_round_reuses_the_tail(server):
    prompt = [11 + (i * 5) % 300 for i in range(90)]
    first, _ = server.completion(prompt, 10)
    nxt = prompt + ids_of(first) + [21, 22, 23]
    _, usage = server.completion(nxt, 4)
    assert usage["prompt_tokens_details"]["cached_tokens"] == len(prompt) + 10 - 1


@pytest.fixture(scope="module")
def eos_case(cold_server):
    """A greedy continuation and a position in it whose token is then declared end-of-sequence."""
    prompt = list(range(5, 40))
    chunks, _ = cold_server.completion(prompt, 24)
    return prompt, ids_of(chunks)


def test_end_of_sequence_stops_unless_ignored(model_dir, eos_case):
    import json

    prompt, ids = eos_case
    index = next(i for i in range(3, len(ids)) if ids[i] not in ids[:i])
    gen = model_dir / "generation_config.json"
    old = gen.read_text()
    gen.write_text(json.dumps({"eos_token_id": [ids[index]]}))
    s = ServerProc(model_dir, extra=["--prefix-cache-entries", "0"])
    try:
        stopped, usage = s.completion(prompt, 24, ignore_eos=False)
        assert ids_of(stopped) == ids[:index]
        assert stopped[-1]["choices"][0]["finish_reason"] == "stop"
        assert usage["completion_tokens"] == index
        ignored, usage = s.completion(prompt, 24)
        assert ids_of(ignored) == ids and usage["completion_tokens"] == 24
        held, usage = s.completion(prompt, 24, ignore_eos=False, min_tokens=index + 1)
        assert ids[index] not in ids_of(held)[: index + 1]
        assert usage["completion_tokens"] >= index + 1
    finally:
        s.stop()
        gen.write_text(old)


def test_streaming_and_non_streaming_agree(server):
    body = {"prompt": "def schedule(requests):\n    for", "max_tokens": 10, "temperature": 0, "ignore_eos": True,
            "return_token_ids": True}
    whole = server.post("/v1/completions", body).json()
    chunks = server.stream("/v1/completions", body)
    assert whole["object"] == "text_completion"
    assert whole["choices"][0]["token_ids"] == ids_of(chunks)
    assert whole["choices"][0]["text"] == "".join(c["choices"][0]["text"] for c in chunks)
    assert whole["choices"][0]["finish_reason"] == "length"
    assert whole["usage"]["completion_tokens"] == 10


def test_default_max_tokens_is_16(server):
    r = server.post("/v1/completions", {"prompt": [50, 51, 52, 53], "temperature": 0, "ignore_eos": True}).json()
    assert r["usage"]["completion_tokens"] == 16


def test_stop_string_cuts_before_the_match(server):
    body = {"prompt": "Question: what is", "max_tokens": 30, "temperature": 0, "ignore_eos": True}
    text = server.post("/v1/completions", body).json()["choices"][0]["text"]
    assert len(text) > 6
    stop = text[4:7]
    cut = server.post("/v1/completions", {**body, "stop": [stop]}).json()
    assert cut["choices"][0]["text"] == text[: text.find(stop)]
    assert cut["choices"][0]["finish_reason"] == "stop"


def test_chat_thinking_switch_and_reasoning_content(server):
    msgs = [{"role": "user", "content": "hello world"}]
    base = {"model": server.model, "messages": msgs, "max_tokens": 12, "temperature": 0, "ignore_eos": True}
    plain = server.post("/v1/chat/completions", base).json()
    assert plain["object"] == "chat.completion"
    assert "reasoning_content" not in plain["choices"][0]["message"]
    off = server.post("/v1/chat/completions", {**base, "chat_template_kwargs": {"enable_thinking": False}}).json()
    assert off["choices"][0]["message"]["content"] == plain["choices"][0]["message"]["content"]
    think = server.post("/v1/chat/completions", {**base, "chat_template_kwargs": {"enable_thinking": True}}).json()
    assert "reasoning_content" in think["choices"][0]["message"]
    assert think["usage"]["prompt_tokens"] < plain["usage"]["prompt_tokens"]  # the "off" template appends an empty block
    events = server.stream("/v1/chat/completions", {**base, "chat_template_kwargs": {"enable_thinking": True}})
    assert events[0]["choices"][0]["delta"] == {"role": "assistant", "content": ""}
    assert events[0]["object"] == "chat.completion.chunk"
    streamed = "".join(e["choices"][0]["delta"].get("reasoning_content", "") for e in events[1:])
    assert streamed == think["choices"][0]["message"]["reasoning_content"]


def test_chat_accepts_tool_call_history(server):
    msgs = [
        {"role": "user", "content": "add"},
        {"role": "assistant", "content": "", "tool_calls": [
            {"id": "1", "type": "function", "function": {"name": "add", "arguments": "{\"a\": 1, \"b\": 2}"}}]},
        {"role": "tool", "content": "3"},
    ]
    r = server.post("/v1/chat/completions", {"messages": msgs, "max_tokens": 4, "temperature": 0,
                                             "tools": [{"type": "function", "function": {"name": "add"}}]})
    assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] <= 4


@pytest.mark.parametrize("body,status", [
    ({"model": "other", "prompt": [1, 2, 3]}, 404),
    ({"prompt": list(range(3, 300)) * 8}, 400),
    ({"prompt": [5, 10 ** 9]}, 400),
    ({"prompt": [5, 6], "n": 2}, 400),
    ({"prompt": [5, 6], "logprobs": 3}, 400),
    ({"prompt": {"a": 1}}, 400),
    ({"prompt": [5, 6], "max_tokens": 5000}, 400),
])
def test_refusals(server, body, status):
    r = server.post("/v1/completions", body)
    assert r.status_code == status
    err = r.json()["error"]
    assert err["code"] == status and err["message"]


def test_concurrent_requests_equal_solo_and_share_decode_steps(server, cold_server):
    prompts = [[3 + (i * (7 + j)) % 400 for i in range(16 + 23 * j)] for j in range(8)]
    solo = [ids_of(cold_server.completion(p, 32)[0]) for p in prompts[:3]]
    before = server.health()
    with ThreadPoolExecutor(8) as pool:
        outs = list(pool.map(lambda p: server.completion(p, 32), prompts))
    after = server.health()
    assert [ids_of(c) for c, _ in outs[:3]] == solo
    assert all(u["completion_tokens"] == 32 for _, u in outs)
    steps = after["decode_steps"] - before["decode_steps"]
    tokens = after["decoded_tokens"] - before["decoded_tokens"]
    assert tokens > steps  # several requests advanced in one step
    assert after["largest_batch"] > 1
    # chat route, streamed, under concurrency
    body = {"messages": [{"role": "user", "content": "hi there"}], "max_tokens": 8, "temperature": 0,
            "ignore_eos": True, "return_token_ids": True}
    one = ids_of(cold_server.stream("/v1/chat/completions", body)[1:])
    with ThreadPoolExecutor(4) as pool:
        many = list(pool.map(lambda _: ids_of(server.stream("/v1/chat/completions", body)[1:]), range(4)))
    assert all(m == one for m in many)
