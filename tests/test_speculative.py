"""MTP speculative decoding on the CPU oracle path: outputs never change, states stay consistent."""

import pytest
import torch

from b200serve.config import EngineConfig, ModelConfig
from b200serve.models.checkpoint import random_weights
from b200serve.sched.engine import Engine
from b200serve.sched.request import Sampling
from b200serve.spec.controller import DepthPolicy


@pytest.fixture(scope="module")
def weights():
    cfg = ModelConfig.tiny()
    cfg.eos_token_ids = [2]
    return random_weights(cfg, seed=0, dtype=torch.float32, std=0.02, lm_head_std=0.5)


def _engine(weights, mtp, k=0, kmax=3):
    return Engine(weights, EngineConfig(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=8, mtp=mtp, spec_k=k,
                                        spec_kmax=kmax))


def _prompts(n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(3, 1024, (int(torch.randint(16, 150, (1,), generator=g)),), generator=g).tolist() for _ in range(n)]


@pytest.fixture(scope="module")
def plain(weights):
    prompts = _prompts(4)
    outs = [g.output for g in _engine(weights, False).generate(prompts, Sampling(max_tokens=20, ignore_eos=True))]
    return prompts, outs


@pytest.mark.parametrize("k", [1, 3])
def test_served_outputs_with_mtp_equal_plain(weights, plain, k):
    prompts, outs = plain
    eng = _engine(weights, True, k=k)
    got = [g.output for g in eng.generate(prompts, Sampling(max_tokens=20, ignore_eos=True))]
    assert got == outs
    assert eng.stats["mtp_verify_steps"] > 0 and eng.stats["mtp_proposed"] > 0


@pytest.mark.parametrize("mode", ["right", "wrong", "half"])
def test_forced_drafts_accept_or_reject_without_changing_outputs(weights, plain, mode):
    prompts, outs = plain
    truth = {tuple(p): o for p, o in zip(prompts, outs)}
    eng = _engine(weights, True, k=3)

    def override(g, k):
        full = truth[tuple(g.prompt)]
        nxt = full[len(g.output):len(g.output) + k]
        if mode == "right":
            return nxt
        if mode == "wrong":
            return [(t + 1) % 1000 + 3 for t in nxt]
        return nxt[:1] + [(t + 1) % 1000 + 3 for t in nxt[1:]]

    eng.spec.draft_override = override
    gens = eng.generate(prompts, Sampling(max_tokens=20, ignore_eos=True))
    assert [g.output for g in gens] == outs
    st = eng.stats
    if mode == "right":
        assert st["mtp_accepted"] == st["mtp_proposed"] > 0
        assert st["decode_steps"] < 4 * 20 / 2  # several tokens per step
    elif mode == "wrong":
        assert st["mtp_accepted"] == 0
    else:
        assert 0 < st["mtp_accepted"] < st["mtp_proposed"]
    # the parked state after speculation continues exactly like a plain engine's
    eng.spec.draft_override = None
    nxt = prompts[0] + outs[0] + [7, 8, 9]
    cont = eng.generate([nxt], Sampling(max_tokens=6, ignore_eos=True))[0]
    ref = _engine(weights, False).generate([nxt], Sampling(max_tokens=6, ignore_eos=True))[0]
    assert cont.cached_tokens >= len(prompts[0]) and cont.output == ref.output


def test_eos_inside_an_accepted_run_stops_exactly_there(weights, plain):
    prompts, outs = plain
    truth = {tuple(p): o for p, o in zip(prompts, outs)}
    eos_tok = outs[0][5]
    eng = _engine(weights, True, k=3)
    eng.eos = {eos_tok}
    eng.spec.draft_override = lambda g, k: truth[tuple(g.prompt)][len(g.output):len(g.output) + k]
    g = eng.generate([prompts[0]], Sampling(max_tokens=20))[0]
    cut = outs[0].index(eos_tok)
    assert g.finish_reason == "stop" and g.output == outs[0][:cut]
    ref = _engine(weights, False)
    ref.eos = {eos_tok}
    r = ref.generate([prompts[0]], Sampling(max_tokens=20))[0]
    assert r.output == g.output
    # a follow-up that reuses the parked tail matches a cold engine
    eng.spec.draft_override = None
    nxt = prompts[0] + g.output + [eos_tok, 11, 12]
    a = eng.generate([nxt], Sampling(max_tokens=5, ignore_eos=True))[0]
    b = _engine(weights, False).generate([nxt], Sampling(max_tokens=5, ignore_eos=True))[0]
    assert a.cached_tokens > 0 and a.output == b.output


def test_sampling_rows_ride_along_without_drafts(weights):
    eng = _engine(weights, True, k=2)
    p = _prompts(2, seed=9)
    s = [Sampling(max_tokens=10, ignore_eos=True), Sampling(max_tokens=10, temperature=0.7, seed=3, ignore_eos=True)]
    a = eng.generate(p, s)
    b = _engine(weights, False).generate(p, s)
    assert a[0].output == b[0].output  # greedy row unchanged
    assert len(a[1].output) == 10


def test_depth_policy_host_logic():
    pol = DepthPolicy(kmax=3)
    pol.accept = [0.9, 0.9, 0.9]
    assert pol.choose(1, 3) == 3
    assert pol.choose(1, 1) == 1  # no more drafts than available
    pol.accept = [0.05, 0.05, 0.05]
    assert pol.choose(1, 3) == 0
    pol.table = {(1, 0): 7.0, (1, 1): 7.1, (1, 3): 8.9, (8, 0): 10.0, (8, 1): 30.0, (8, 3): 60.0}
    pol.accept = [0.6, 0.5, 0.4]
    assert pol.choose(1, 3) >= 1 and pol.choose(8, 3) == 0
    fixed = DepthPolicy(kmax=3, fixed=2)
    assert fixed.choose(4, 3) == 2 and fixed.choose(4, 1) == 1 and fixed.choose(200, 3) == 0
    before = list(pol.accept)
    pol.observe(3, 1)  # draft 1 accepted, draft 2 rejected, draft 3 untested
    assert pol.accept[0] > before[0] and pol.accept[1] < before[1] and pol.accept[2] == before[2]


def test_depth_policy_reads_a_measured_cost_table_and_extends_it_to_deeper_chains(tmp_path):
    import json
    from pathlib import Path

    from b200serve.spec.controller import DepthPolicy

    shipped = Path(__import__("b200serve").__file__).resolve().parent.parent / "qwen36-mi250-tracelab-20261107_b200/spec/cost_table_b200.json"
    p = DepthPolicy(kmax=7)
    p.load_table(shipped)
    assert p.cost(1, 0) < p.cost(1, 1) < p.cost(1, 3) and p.cost(5, 2) == p.cost(8, 2)  # bucket of the next larger batch
    assert p.cost(1, 5) == pytest.approx(7.63) and p.cost(1, 4) == pytest.approx((p.cost(1, 3) + p.cost(1, 5)) / 2)  # measured; between
    assert p.cost(64, 5) == pytest.approx(p.cost(64, 3) + 2 * (p.cost(64, 3) - p.cost(64, 2)))  # beyond the measured depths
    assert p.cost(200, 1) == p.cost(64, 1)  # beyond the largest measured bucket
    # high acceptance at batch 1 pays for deep chains, low acceptance or a big batch does not
    p.accept = [0.9] * 7
    assert p.choose(1, 7) >= 4
    p.accept = [0.2] * 7
    assert p.choose(64, 7) == 0
    custom = tmp_path / "t.json"
    custom.write_text(json.dumps({"ms": {"4": {"0": 1.0, "1": 1.1}}}))
    q = DepthPolicy(kmax=2)
    q.load_table(custom)
    q.accept = [0.8, 0.8]
    assert q.choose(2, 2) == 2


def test_shortlist_index_is_deterministic_and_exact_when_every_cluster_is_probed():
    from b200serve.ops import torch_ops
    from b200serve.spec.ivf import IvfIndex

    g = torch.Generator().manual_seed(4)
    head = torch.randn(1000, 64, generator=g)
    a = IvfIndex.build(head, n_clusters=32, probes=32)
    b = IvfIndex.build(head, n_clusters=32, probes=32)
    assert torch.equal(a.order, b.order) and torch.equal(a.offsets, b.offsets) and torch.equal(a.centroids, b.centroids)
    # a partition of the vocabulary
    assert sorted(a.order.tolist()) == list(range(1000)) and int(a.offsets[-1]) == 1000
    h = torch.randn(9, 64, generator=g)
    full = (h @ head.t()).argmax(-1)
    assert torch.equal(a.pick(torch_ops, h, head), full)  # all clusters probed: the shortlist is the vocabulary
    # a few probes: the pick is the best member of the probed clusters, and it is the full argmax whenever the
    # argmax row's cluster was probed
    few = IvfIndex(a.centroids, a.order, a.offsets, probes=4)
    picks = few.pick(torch_ops, h, head)
    scores = h @ a.centroids.float().t()
    probed = scores.topk(4, dim=-1).indices
    cluster_of = torch.empty(1000, dtype=torch.long)
    off = a.offsets.tolist()
    for c in range(32):
        cluster_of[a.order[off[c]:off[c + 1]].long()] = c
    for r in range(9):
        members = torch.cat([a.order[off[c]:off[c + 1]] for c in probed[r].tolist()]).long()
        assert int(picks[r]) in members.tolist()
        assert float(h[r] @ head[picks[r]]) == pytest.approx(float((head[members] @ h[r]).max()))
        if int(cluster_of[full[r]]) in probed[r].tolist():
            assert int(picks[r]) == int(full[r])


def test_shortlist_drafts_never_change_outputs(weights, plain):
    """Drafts from the vocabulary shortlist are only guesses: served outputs stay those of plain decoding."""
    prompts, outs = plain
    eng = Engine(weights, EngineConfig(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=8, mtp=True, spec_k=2,
                                       spec_kmax=3, draft_ivf=16, draft_ivf_probes=4))
    assert eng.model.draft_index is not None and eng.model.draft_index.n_clusters == 16
    got = [g.output for g in eng.generate(prompts, Sampling(max_tokens=20, ignore_eos=True))]
    assert got == outs
    assert eng.stats["mtp_verify_steps"] > 0 and eng.stats["mtp_proposed"] > 0
