"""Token selection from one row of logits.

Greedy at temperature 0 (ties to the lower id); otherwise temperature, top-k, top-p and a
seeded multinomial draw. ``mask`` removes the end-of-sequence ids while ``min_tokens`` has
not been reached (reference: ``Generator.pick``, ``engine/generator.py:1091-1110``).
"""

from __future__ import annotations

import torch

from .request import Sampling


def pick_token(logits: torch.Tensor, s: Sampling, rng: torch.Generator | None, mask: set[int] | None = None) -> int:
    logits = logits.float()
    if mask:
        logits = logits.clone()
        logits[list(mask)] = float("-inf")
    if s.greedy:
        return int(torch.argmax(logits))
    logits = logits / max(s.temperature, 1e-6)
    if s.top_k and s.top_k > 0 and s.top_k < logits.numel():
        kth = torch.topk(logits, s.top_k).values[-1]
        logits = torch.where(logits < kth, torch.full_like(logits, float("-inf")), logits)
    probs = torch.softmax(logits, dim=-1)
    if s.top_p < 1.0:
        sp, si = torch.sort(probs, descending=True)
        cum = torch.cumsum(sp, dim=-1)
        drop = cum - sp > s.top_p  # keep the smallest set whose mass reaches top_p
        sp = torch.where(drop, torch.zeros_like(sp), sp)
        probs = torch.zeros_like(probs).scatter_(0, si, sp)
        probs = probs / probs.sum()
    return int(torch.multinomial(probs, 1, generator=rng))
