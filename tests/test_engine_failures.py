"""What the engine does when a pass fails: a device-side error word, an exception outside the per-pass handlers,
and the once-per-step delivery of tokens. All on the CPU path; the device error word is a host tensor here."""

import types

import pytest
import torch

from b200serve.config import EngineConfig, ModelConfig
from b200serve.models.checkpoint import random_weights
from b200serve.ops import torch_ops
from b200serve.sched.engine import Engine
from b200serve.sched.request import Generation, Sampling


@pytest.fixture(scope="module")
def weights():
    return random_weights(ModelConfig.tiny(), seed=0, dtype=torch.float32, std=0.02, lm_head_std=0.5)


class _KernelError(RuntimeError):
    pass


def _ops_with_error_word():
    """The CPU op set plus the two things ``Engine.check_device`` uses from the CUDA op set."""
    ops = types.SimpleNamespace(**{k: getattr(torch_ops, k) for k in dir(torch_ops) if not k.startswith("__")})
    word = torch.zeros(1, dtype=torch.int32)
    ops.err_word = lambda device: word
    ops.KernelError = _KernelError
    return ops, word


def _engine(weights, ops=None):
    return Engine(weights, EngineConfig(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=8, mtp=False), ops=ops)


def _submit(eng, n, max_tokens=20):
    events = []
    g = eng.submit(Generation([3 + (i * 7) % 900 for i in range(n)], Sampling(max_tokens=max_tokens, ignore_eos=True),
                              on_event=lambda gen, ev: events.append(ev)))
    return g, events


def test_a_set_error_word_fails_the_requests_of_that_pass_and_is_cleared(weights):
    ops, word = _ops_with_error_word()
    eng = _engine(weights, ops)
    a, ev_a = _submit(eng, 40)
    b, ev_b = _submit(eng, 70)
    for _ in range(4):
        eng.step()
    assert len(a.output) >= 2 and not a.done
    word[0] = 4  # what a peer wait that ran out leaves behind
    eng.step()
    eng.flush_events()
    # nothing sampled from that pass reached the clients: both requests ended with an error event instead
    assert a.finish_reason == "error" and b.finish_reason == "error"
    assert ev_a[-1].error is not None and ev_a[-1].error.status == 500 and ev_a[-1].token is None
    assert int(word[0]) == 0 and eng.stats["device_errors"] == 1
    assert eng.slots.free + len(eng.cache) == eng.slots.num_slots - 1  # the failed requests gave their slots back
    # the engine keeps serving, with the same tokens as an engine that never saw the failure
    c, _ = _submit(eng, 40)
    while not c.done:
        eng.step()
    ref = _engine(weights).generate([c.prompt], Sampling(max_tokens=20, ignore_eos=True))[0]
    assert c.output == ref.output and eng.broken is None


def test_in_a_rank_group_a_device_failure_tears_the_engine_down(weights):
    ops, word = _ops_with_error_word()
    eng = _engine(weights, ops)
    eng.multi_rank = True  # as with tp= / ep=: peers may have taken a different path through the failed pass
    a, ev_a = _submit(eng, 40, max_tokens=50)
    for _ in range(3):
        eng.step()
    word[0] = 4
    eng.step()   # the pass fails its requests and latches the failure
    eng.step()   # no agreement channel here: the rank gives up on the group at once
    assert eng.broken is not None and a.finish_reason == "error"
    late, ev = _submit(eng, 10)
    eng.step()
    assert late.finish_reason == "error" and ev[-1].error.status == 503
    assert eng.health()["broken"]


def test_an_exception_outside_the_pass_handlers_fails_everything_once_and_the_engine_recovers(weights):
    eng = _engine(weights)
    a, ev_a = _submit(eng, 40)
    b, ev_b = _submit(eng, 130)  # still prefilling when the failure comes
    eng.step()
    orig, calls = eng._sample_and_emit, []

    def boom(*args, **kw):
        calls.append(1)
        raise IndexError("bookkeeping bug")

    eng._sample_and_emit = boom
    eng.step()
    eng._sample_and_emit = orig
    assert calls and a.finish_reason == "error" and b.finish_reason == "error"
    assert ev_a[-1].error.status == 500 and ev_b[-1].error.status == 500
    assert not eng.running and not eng.prefilling and not eng.waiting and eng.stats["step_errors"] == 1
    for _ in range(3):
        eng.step()  # must not raise again on leftovers of the failed iteration
    c = eng.generate([[9, 8, 7, 6, 5]], Sampling(max_tokens=6, ignore_eos=True))[0]
    assert len(c.output) == 6
    # no slot leaked: every slot is free, the scratch slot 0, or held by a prefix-cache entry
    assert eng.slots.free + len(eng.cache) == eng.slots.num_slots - 1


def test_tokens_are_delivered_every_step_when_the_graph_path_is_not_taken(weights):
    """With decode graphs configured, tokens are normally handed over right after the next graph launch. A step that
    falls back to kernel-by-kernel launches (failed capture, batch outside the buckets) must deliver them itself."""
    eng = _engine(weights)
    eng._graphs = types.SimpleNamespace(usable=lambda gens: False, buckets={})  # graphs "exist" but never apply
    g, events = _submit(eng, 30, max_tokens=12)
    while not eng.running:
        eng.step()
    assert len(events) == len(g.output) >= 1  # the iteration that finished the prefill delivered its tokens too
    seen = len(events)
    for _ in range(5):
        eng.step()
        assert len(events) == seen + 1  # one token per step, delivered within that step
        seen = len(events)


# --------------------------------------------------------------------------- run-ahead (decode-graph scheduling on CPU)
def _graph_engine(weights, run_ahead, **kw):
    cfg = EngineConfig(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=8, mtp=False, graphs_on_cpu=True,
                       run_ahead=run_ahead, decode_buckets=(1, 2, 4, 8), **kw)
    return Engine(weights, cfg)


def test_run_ahead_keeps_tokens_lengths_and_cache_identical(weights):
    """Step n + 1 is launched from device-built inputs before step n is read: same tokens as without it, exact
    lengths, page growth across the 64-token boundary, and session tails that later requests can resume from."""
    prompts = [[3 + (i * (7 + s)) % 900 for i in range(n)] for s, n in enumerate((40, 61, 130))]
    samp = [Sampling(max_tokens=m, ignore_eos=True) for m in (90, 33, 7)]
    outs, stats = [], []
    for ahead in (False, True):
        eng = _graph_engine(weights, ahead)
        assert eng._graphs is not None
        gens = eng.generate(prompts, samp)
        outs.append([g.output for g in gens])
        stats.append(dict(eng.stats))
        assert [len(g.output) for g in gens] == [90, 33, 7]
        # a second round on top of the first: resumes from the tail that a run-ahead engine parked
        again = eng.generate([prompts[0] + gens[0].output + [5, 6, 7]], Sampling(max_tokens=9, ignore_eos=True))[0]
        outs[-1].append(again.output)
        assert again.cached_tokens == len(prompts[0]) + 90 - 1
    assert outs[0] == outs[1]
    assert stats[0]["ahead_steps"] == 0 and stats[1]["ahead_steps"] > 50
    ref = _engine(weights).generate(prompts, samp)
    assert [g.output for g in ref] == outs[1][:3]


def test_run_ahead_stops_for_requests_that_can_end_on_a_token_and_for_new_arrivals(weights):
    eng = _graph_engine(weights, True)
    a, _ = _submit(eng, 40, max_tokens=60)
    for _ in range(8):
        eng.step()
    ahead0 = eng.stats["ahead_steps"]
    assert ahead0 > 0 and eng._pending is not None
    b = eng.submit(Generation([9, 8, 7, 6, 5, 4], Sampling(max_tokens=50, ignore_eos=False)))  # may stop on EOS
    for _ in range(3):
        eng.step()
    assert b in eng.running and eng._pending is None  # the pipeline drained and did not restart: b can end any time
    mid = eng.stats["ahead_steps"]
    while not (a.done and b.done):
        eng.step()
    assert eng.stats["ahead_steps"] <= mid + 60  # only once b is gone may a run ahead again
    solo = _engine(weights).generate([a.prompt, b.prompt], [a.sampling, b.sampling])
    assert a.output == solo[0].output and b.output == solo[1].output


def test_a_cancelled_request_keeps_the_token_of_the_step_in_flight(weights):
    """The step launched ahead already advanced the request's state: its token is booked before the cancellation, so
    the parked tail matches the state."""
    eng = _graph_engine(weights, True)
    a, ev = _submit(eng, 40, max_tokens=200)
    for _ in range(6):
        eng.step()
    assert eng._pending is not None
    a.cancelled.set()
    n0 = len(a.output)
    for _ in range(3):
        eng.step()
    assert a.finish_reason == "cancelled" and len(a.output) == n0 + 1 and eng._pending is None
    nxt = eng.generate([a.prompt + a.output + [4, 4]], Sampling(max_tokens=5, ignore_eos=True))[0]
    cold = _engine(weights).generate([a.prompt + a.output + [4, 4]], Sampling(max_tokens=5, ignore_eos=True))[0]
    assert nxt.cached_tokens > 0 and nxt.output == cold.output
