"""Property-based checks (hypothesis) of the host-side pieces whose inputs are arbitrary: request bodies, streamed
text, growing prompts, chunk spans."""

import json

import pytest
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from b200serve.api import protocol
from b200serve.api.protocol import RequestError
from b200serve.api.text import Detokenizer, StopMatcher

json_values = st.recursive(
    st.none() | st.booleans() | st.integers(-10**6, 10**6) | st.floats(allow_nan=False, allow_infinity=False) | st.text(max_size=12),
    lambda inner: st.lists(inner, max_size=4) | st.dictionaries(st.text(max_size=8), inner, max_size=4), max_leaves=12)
KEYS = ["prompt", "messages", "max_tokens", "max_completion_tokens", "temperature", "top_p", "top_k", "seed", "stop", "stream",
        "stream_options", "n", "logprobs", "echo", "ignore_eos", "min_tokens", "model", "tools", "chat_template_kwargs",
        "return_token_ids", "best_of", "suffix", "logit_bias"]


@settings(max_examples=300, deadline=None)
@given(st.dictionaries(st.sampled_from(KEYS), json_values, max_size=8) | json_values)
def test_any_json_body_is_parsed_or_refused_with_a_request_error(body):
    """Whatever JSON arrives, the parsers either build a request or raise ``RequestError`` with a 4xx status."""
    for parse in (protocol.parse_completion, protocol.parse_chat):
        try:
            req = parse(json.loads(json.dumps(body)))
        except RequestError as e:
            assert 400 <= e.status < 500
        else:
            s = req.sampling
            assert s.max_tokens is None or s.max_tokens >= 0
            assert s.temperature >= 0 and 0 < s.top_p <= 1 and s.min_tokens >= 0
            assert all(isinstance(x, str) and x for x in s.stop)


@settings(max_examples=300, deadline=None)
@given(st.text(alphabet="abcx#\n ", max_size=60), st.lists(st.text(alphabet="abcx#\n", min_size=1, max_size=4), max_size=3),
       st.lists(st.integers(1, 7), max_size=30))
def test_stop_matcher_output_does_not_depend_on_how_the_text_arrives(text, stops, cuts):
    """Streaming in any chunking gives the text cut right before the stop string that is complete first (of two
    that end together, the one that starts earlier), or all of it."""
    ends = [(i + len(s), i) for s, i in ((s, text.find(s)) for s in stops) if i >= 0]
    first = min(ends)[1] if ends else None
    want = text if first is None else text[:first]
    m = StopMatcher(stops)
    out, pos = [], 0
    for c in cuts + [len(text)]:
        out.append(m.push(text[pos : pos + c]))
        pos += c
        if pos >= len(text):
            break
    out.append(m.flush())
    assert "".join(out) == want and m.stopped == (first is not None)
    released = "".join(out[:-1])
    assert want.startswith(released)  # nothing that was sent early ever has to be taken back


@pytest.fixture(scope="module")
def tok(tmp_path_factory):
    from b200serve.api.tokenizer import TextCodec
    from b200serve.models.tiny import write_tiny_checkpoint

    d = tmp_path_factory.mktemp("tok")
    write_tiny_checkpoint(d)
    return TextCodec(d)


@settings(max_examples=120, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture])
@given(st.text(alphabet=st.characters(codec="utf-8", categories=["L", "N", "P", "Zs", "So"]), max_size=40))
def test_streamed_detokenisation_equals_the_whole_decode(tok, text):
    """Any text, multi-byte characters and emoji included: the deltas never contain half a character and add up to
    the decode of the whole sequence."""
    ids = tok.tok.encode(text, add_special_tokens=False)
    det = Detokenizer(tok.tok)
    parts = [det.push(t) for t in ids] + [det.flush()]
    assert all("\ufffd" not in p for p in parts[:-1]) or "\ufffd" in text
    assert "".join(parts) == tok.tok.decode(ids, skip_special_tokens=True)


@settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture])
@given(st.lists(st.text(alphabet="abc def,.\n\u00e9\u4e16", min_size=1, max_size=80), min_size=2, max_size=6))
def test_incremental_encoding_of_a_growing_prompt_equals_a_full_encode(tok, turns):
    from b200serve.api.tokenizer import PromptEncoder

    enc = PromptEncoder(tok.tok.backend_tokenizer, capacity=8)
    text = "x" * 70  # long enough for the cache to be consulted
    for t in turns:
        text += t
        assert enc.encode(text) == tok.tok.backend_tokenizer.encode(text, add_special_tokens=False).ids
    assert enc.stats["tokenize_calls"] == len(turns)


@settings(max_examples=200, deadline=None)
@given(st.integers(0, 5000), st.integers(1, 3000), st.sampled_from([8, 64, 256, 2048]))
def test_chunk_spans_cover_the_range_exactly_once(start, length, chunk):
    from b200serve.sched.engine import Engine

    eng = Engine.__new__(Engine)
    eng.chunk = chunk
    spans = Engine._spans(eng, start, start + length)
    assert spans[0][0] == start and spans[-1][1] == start + length
    assert all(a < b and b - a <= chunk for a, b in spans)
    assert all(x[1] == y[0] for x, y in zip(spans, spans[1:]))
    assert all(b % chunk == 0 for _, b in spans[:-1])  # every span but the last ends on a chunk boundary
