"""Token selection from rows of logits, on the device that holds them.

Greedy at temperature 0 (ties to the lower id); otherwise temperature, top-k, top-p and a seeded draw. ``masks``
remove the end-of-sequence ids while ``min_tokens`` has not been reached (reference: ``Generator.pick``,
``engine/generator.py:1091-1110``).

All rows of a step are handled together and only the picked ids leave the device: a step with 128 sampled requests
moves 128 integers to the host, not 128 rows of 248,320 logits. The draw is an inverse-CDF lookup over the filtered
distribution in descending order of probability, with ONE uniform number per request and step taken from the
request's own seeded generator on the host: the same seed gives the same tokens on any device and in any batch.
"""

from __future__ import annotations

import torch

from .request import Sampling

# with every row asking for top-k <= this, a partial selection replaces the full sort over the vocabulary
TOPK_LIMIT = 2048


def pick_tokens(logits: torch.Tensor, samplings: list[Sampling], rngs: list, masks: list) -> list[int]:
    """Next token of each row of ``logits [n, V]``. ``rngs[i]``: the request's CPU generator (unused for greedy
    rows); ``masks[i]``: ids to exclude for this row, or None."""
    n, V = logits.shape
    dev = logits.device
    x = logits.float()
    rows = [i for i, m in enumerate(masks) if m for _ in m]
    if rows:
        cols = [t for m in masks if m for t in m]
        x = x.clone()
        x[torch.tensor(rows, device=dev), torch.tensor(cols, device=dev)] = float("-inf")
    out = [0] * n
    greedy = [i for i, s in enumerate(samplings) if s.greedy]
    sampled = [i for i, s in enumerate(samplings) if not s.greedy]
    picked_g = torch.argmax(x[torch.tensor(greedy, device=dev)], dim=-1) if greedy else None  # first maximum: lower id
    picked_s = None
    if sampled:
        ss = [samplings[i] for i in sampled]
        xs = x[torch.tensor(sampled, device=dev)] if greedy else x
        temp = torch.tensor([max(s.temperature, 1e-6) for s in ss], dtype=torch.float32, device=dev)
        xs = xs / temp[:, None]
        ks = [s.top_k if s.top_k and 0 < s.top_k < V else V for s in ss]
        width = max(ks)
        if width <= TOPK_LIMIT:
            vals, idx = torch.topk(xs, width, dim=-1, sorted=True)
        else:
            vals, idx = torch.sort(xs, dim=-1, descending=True, stable=True)
        rank = torch.arange(vals.shape[1], device=dev)
        k_t = torch.tensor(ks, device=dev)
        vals = vals.masked_fill(rank[None, :] >= k_t[:, None], float("-inf"))  # the k most likely tokens of each row
        probs = torch.softmax(vals, dim=-1)
        top_p = torch.tensor([s.top_p for s in ss], dtype=torch.float32, device=dev)
        cum = torch.cumsum(probs, dim=-1)
        probs = torch.where(cum - probs > top_p[:, None], torch.zeros_like(probs), probs)  # smallest set reaching top_p
        cdf = torch.cumsum(probs, dim=-1)
        u = torch.stack([torch.rand(1, generator=rngs[i]) for i in sampled]).to(dev).view(-1) * cdf[:, -1]
        pos = torch.searchsorted(cdf, u[:, None], right=True).clamp_(max=cdf.shape[1] - 1)  # first entry with cdf > u
        picked_s = idx.gather(1, pos).view(-1)
    if picked_g is not None and picked_s is not None:
        both = torch.cat([picked_g, picked_s]).tolist()  # one copy to the host
        g_h, s_h = both[: len(greedy)], both[len(greedy):]
    else:
        g_h = picked_g.tolist() if picked_g is not None else []
        s_h = picked_s.tolist() if picked_s is not None else []
    for i, t in zip(greedy, g_h):
        out[i] = int(t)
    for i, t in zip(sampled, s_h):
        out[i] = int(t)
    return out


def pick_token(logits: torch.Tensor, s: Sampling, rng: torch.Generator | None, mask: set[int] | None = None) -> int:
    """One row (``logits [V]``): see ``pick_tokens``."""
    return pick_tokens(logits[None, :], [s], [rng], [mask])[0]
