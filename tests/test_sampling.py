"""The batched, device-side sampler: filters, tie rule, seeds, and agreement with the written-out definition."""

import torch

from b200serve.sched.request import Sampling
from b200serve.sched.sampling import pick_token, pick_tokens


def _gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


def test_greedy_rows_take_the_first_maximum_and_honour_masks():
    logits = torch.tensor([[1.0, 5.0, 5.0, 2.0], [3.0, 0.0, 3.0, 3.0], [0.1, 0.2, 0.3, 0.9]])
    s = Sampling(temperature=0.0)
    assert pick_tokens(logits, [s, s, s], [None] * 3, [None, None, None]) == [1, 0, 3]
    assert pick_tokens(logits, [s, s, s], [None] * 3, [{1}, {0, 2}, {3}]) == [2, 3, 2]
    assert pick_token(logits[0], s, None, {1, 2}) == 3


def test_top_k_one_and_tiny_top_p_are_greedy():
    torch.manual_seed(0)
    logits = torch.randn(6, 500)
    want = logits.argmax(-1).tolist()
    k1 = Sampling(temperature=0.9, top_k=1, seed=1)
    p0 = Sampling(temperature=1.3, top_p=1e-6, seed=2)
    assert pick_tokens(logits, [k1] * 6, [_gen(i) for i in range(6)], [None] * 6) == want
    assert pick_tokens(logits, [p0] * 6, [_gen(i) for i in range(6)], [None] * 6) == want


def test_draws_stay_inside_the_filtered_support():
    torch.manual_seed(1)
    logits = torch.randn(1, 300) * 2
    probs = torch.softmax(logits[0] / 0.7, -1)
    order = probs.argsort(descending=True)
    top20 = set(order[:20].tolist())
    cum = probs[order].cumsum(0)
    nucleus = set(order[: int((cum - probs[order] <= 0.6).sum())].tolist())  # smallest set whose mass reaches 0.6
    sk = Sampling(temperature=0.7, top_k=20, seed=0)
    sp = Sampling(temperature=0.7, top_p=0.6, seed=0)
    both = Sampling(temperature=0.7, top_k=20, top_p=0.6, seed=0)
    g = _gen(3)
    for _ in range(300):
        assert pick_tokens(logits, [sk], [g], [None])[0] in top20
        assert pick_tokens(logits, [sp], [g], [None])[0] in nucleus
        assert pick_tokens(logits, [both], [g], [None])[0] in (top20 & nucleus)
    banned = set(order[:5].tolist())
    for _ in range(100):
        assert pick_tokens(logits, [sk], [g], [banned])[0] not in banned


def test_frequencies_follow_the_distribution():
    logits = torch.log(torch.tensor([[0.5, 0.25, 0.125, 0.125]]))
    s = Sampling(temperature=1.0, seed=0)
    g = _gen(5)
    n = 4000
    counts = torch.zeros(4)
    for _ in range(n):
        counts[pick_tokens(logits, [s], [g], [None])[0]] += 1
    assert torch.allclose(counts / n, torch.tensor([0.5, 0.25, 0.125, 0.125]), atol=0.03)
    hot = Sampling(temperature=2.0, seed=0)  # temperature 2 flattens: p ~ sqrt of the above, renormalised
    want = torch.tensor([0.5, 0.25, 0.125, 0.125]).sqrt()
    want = want / want.sum()
    counts = torch.zeros(4)
    for _ in range(n):
        counts[pick_tokens(logits, [hot], [g], [None])[0]] += 1
    assert torch.allclose(counts / n, want, atol=0.03)


def test_a_seed_fixes_the_tokens_whatever_shares_the_batch():
    torch.manual_seed(2)
    logits = torch.randn(5, 2000)
    mixed = [Sampling(temperature=0.8, top_p=0.9, seed=7), Sampling(temperature=0.0), Sampling(temperature=1.1, top_k=40, seed=8),
             Sampling(temperature=0.6, top_k=3000, seed=9), Sampling(temperature=0.0)]
    seeds = [7, None, 8, 9, None]

    def run(rows):
        gens = {i: (_gen(seeds[i]) if seeds[i] is not None else None) for i in rows}
        outs = {i: [] for i in rows}
        for _ in range(8):
            got = pick_tokens(logits[rows], [mixed[i] for i in rows], [gens[i] for i in rows], [None] * len(rows))
            for i, t in zip(rows, got):
                outs[i].append(t)
        return outs

    together, alone0, pair = run([0, 1, 2, 3, 4]), run([0]), run([3, 2])
    assert together[0] == alone0[0] and together[2] == pair[2] and together[3] == pair[3]
    assert together[1] == [int(logits[1].argmax())] * 8 and len(set(together[0])) > 1


import pytest  # noqa: E402


@pytest.mark.gpu
def test_device_and_host_sampler_agree():
    """The same rows, seeds and filters on the GPU and on the CPU: same tokens (full sort and partial selection)."""
    torch.manual_seed(3)
    logits = (torch.randn(6, 5000) * 3).round(decimals=3)  # coarse values: no near-ties that float order could flip
    logits += torch.arange(5000) * 1e-7
    mixed = [Sampling(temperature=0.8, top_p=0.9, seed=1), Sampling(temperature=0.0), Sampling(temperature=1.2, top_k=50, seed=2),
             Sampling(temperature=0.7, top_k=4000, top_p=0.95, seed=3), Sampling(temperature=0.0), Sampling(temperature=1.0, seed=4)]
    seeds = [1, None, 2, 3, None, 4]
    masks = [None, {int(logits[1].argmax())}, {5, 6}, None, None, None]
    for rows in ([0, 1, 2, 3, 4, 5], [2], [1, 4], [2, 0]):
        def run(dev):
            gens = [(_gen(seeds[i]) if seeds[i] is not None else None) for i in rows]
            out = []
            for _ in range(6):
                out.append(pick_tokens(logits[rows].to(dev), [mixed[i] for i in rows], gens, [masks[i] for i in rows]))
            return out

        assert run("cuda") == run("cpu")
