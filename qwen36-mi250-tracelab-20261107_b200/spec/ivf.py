"""Shortlist drafts: an inverted-file index over the LM head for the speculative draft picks.

The MTP chain asks the LM head for a token once per draft link. That token only has to be a good guess: the verify
pass accepts it only if it equals the base model's own greedy pick. At the small batches where speculation pays,
reading the whole 1 GB head per link is most of the link's time, so the draft pick can come from a shortlist
instead: the vocabulary rows are clustered once (spherical k-means on the row directions), a row's hidden state is
scored against the cluster centroids (one small GEMM), and only the members of the best ``probes`` clusters are
scored exactly (reference: ``engine/fast/draft_ivf.py:159`` index build, ``:508-644`` draft path; its predicated
full-vocabulary fallback is not reproduced, a weak draft simply costs a rejected token).

The index build is deterministic (seeded initial centroids, fixed iteration count, ties to the lower id), so all
ranks of a replica and every restart of a server hold the same index. ``pick`` runs on the device without host
synchronisation and can be captured in a CUDA graph.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class IvfIndex:
    centroids: torch.Tensor  # [C, H] in the weights' dtype
    order: torch.Tensor      # [V] int32: vocabulary rows grouped by cluster
    offsets: torch.Tensor    # [C + 1] int32: cluster c owns order[offsets[c] : offsets[c + 1]]
    probes: int

    @property
    def n_clusters(self) -> int:
        return self.centroids.shape[0]

    @classmethod
    def build(cls, lm_head: torch.Tensor, n_clusters: int = 4096, probes: int = 64, iters: int = 6, seed: int = 0,
              chunk: int = 16384) -> "IvfIndex":
        """Cluster the rows of a plain (not tile-packed) LM head ``[V, H]``."""
        V, H = lm_head.shape
        C = max(1, min(n_clusters, V))
        dev = lm_head.device
        g = torch.Generator(device="cpu").manual_seed(seed)
        first = torch.randperm(V, generator=g)[:C].sort().values.to(dev)

        def unit(x: torch.Tensor) -> torch.Tensor:
            return x / x.norm(dim=-1, keepdim=True).clamp_min(1e-12)

        cent = unit(lm_head[first].float())
        assign = torch.empty(V, dtype=torch.int64, device=dev)
        for it in range(iters + 1):
            for a in range(0, V, chunk):
                rows = unit(lm_head[a:a + chunk].float())
                assign[a:a + chunk] = (rows @ cent.t()).argmax(dim=-1)  # first maximum: ties to the lower cluster id
            if it == iters:
                break
            sums = torch.zeros(C, H, dtype=torch.float32, device=dev)
            for a in range(0, V, chunk):
                sums.index_add_(0, assign[a:a + chunk], unit(lm_head[a:a + chunk].float()))
            keep = sums.norm(dim=-1) > 0  # an emptied cluster keeps its old centroid
            cent = torch.where(keep[:, None], unit(sums), cent)
        order = torch.sort(assign, stable=True).indices.to(torch.int32)
        counts = torch.bincount(assign, minlength=C)
        offsets = torch.zeros(C + 1, dtype=torch.int32, device=dev)
        offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
        # probe with the mean row of each cluster (not its direction): the score that is compared is an inner product
        means = torch.zeros(C, H, dtype=torch.float32, device=dev)
        for a in range(0, V, chunk):
            means.index_add_(0, assign[a:a + chunk], lm_head[a:a + chunk].float())
        means = means / counts.clamp_min(1)[:, None].float()
        return cls(means.to(lm_head.dtype).contiguous(), order.contiguous(), offsets.contiguous(), min(probes, C))

    # ------------------------------------------------------------------ draft pick
    def pick(self, ops, hidden: torch.Tensor, lm_head: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Best shortlist token of every row of ``hidden [R, H]`` (int64 ``[R]``)."""
        R = hidden.shape[0]
        scores = ops.linear(hidden, self.centroids, out_dtype=torch.float32)[:, : self.n_clusters]
        probes = torch.topk(scores, self.probes, dim=-1).indices.to(torch.int32)
        if hidden.device.type == "cuda" and hasattr(ops, "ivf_pick"):
            return ops.ivf_pick(hidden, lm_head, probes, self.offsets, self.order, out=out)
        picks = self.pick_reference(hidden, lm_head, probes)
        if out is not None:
            out.copy_(picks)
            return out
        return picks

    def pick_reference(self, hidden: torch.Tensor, lm_head: torch.Tensor, probes: torch.Tensor) -> torch.Tensor:
        """Plain PyTorch form of the gathered scoring (the oracle of the kernel test; the CPU path)."""
        picks = []
        off = self.offsets.tolist()
        for r in range(hidden.shape[0]):
            ids = torch.cat([self.order[off[c]:off[c + 1]] for c in probes[r].tolist()]).long()
            if ids.numel() == 0:
                picks.append(0)
                continue
            ids = ids.sort().values  # first maximum of ascending ids = ties to the lower id
            logit = lm_head[ids].float() @ hidden[r].float()
            picks.append(int(ids[int(logit.argmax())]))
        return torch.tensor(picks, dtype=torch.int64, device=hidden.device)
