"""Layer-split (pipeline) placement of one replica over several GPUs.

Each rank of the group holds a contiguous run of the 40 layers with their KV pages and Gated DeltaNet states; the
first rank also embeds, the last one also holds the final norm, the LM head and the sampler's input. A forward pass
walks the ranks in order: a rank receives the residual stream and the normed hidden state of the rows from its
predecessor, runs its layers and hands both on. There is no micro-batching: like the reference's layer split over two
devices (``engine/fast/model.py:187-200``, a capacity measure for GPUs that cannot hold the model) only one rank
computes at a time, so this mode buys memory, not speed; a B200 holds the whole model and the served modes are the
data-parallel replicas, the tensor-parallel replica and data-parallel attention with expert-parallel MoE.

All ranks run the same scheduler on the same requests in lockstep (``parallel/lockstep.py``), as a tensor-parallel
replica does: page and slot bookkeeping is identical everywhere, each rank fills only its own layers' caches. The
tokens picked on the last rank are broadcast to the others, which need them as the next step's inputs.
Point-to-point transfers are ``torch.distributed`` send/recv (NCCL over NVLink between GPUs, gloo between CPU ranks in
the tests); they are not captured in CUDA graphs, so a layer-split engine launches eagerly.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass

import torch

from ..models.checkpoint import Weights


@dataclass
class PPContext:
    rank: int
    world: int
    group: object = None

    @property
    def is_first(self) -> bool:
        return self.rank == 0

    @property
    def is_last(self) -> bool:
        return self.rank == self.world - 1

    def _dist(self):
        import torch.distributed as dist

        return dist

    def _global(self, group_rank: int) -> int:
        dist = self._dist()
        return dist.get_global_rank(self.group, group_rank) if self.group is not None else group_rank

    def send(self, res: torch.Tensor, h: torch.Tensor) -> None:
        """Hand the residual stream and the normed hidden state of every row to the next rank."""
        self._dist().send(torch.stack([res, h]).contiguous(), self._global(self.rank + 1), group=self.group)

    def recv(self, rows: int, hidden: int, dtype: torch.dtype, device: torch.device):
        buf = torch.empty(2, rows, hidden, dtype=dtype, device=device)
        self._dist().recv(buf, self._global(self.rank - 1), group=self.group)
        return buf[0], buf[1]

    def share(self, value: torch.Tensor | None, shape, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        """Broadcast a result of the last rank (picked tokens, logits) to every rank of the group."""
        t = value.contiguous() if self.is_last else torch.empty(shape, dtype=dtype, device=device)
        self._dist().broadcast(t, self._global(self.world - 1), group=self.group)
        return t


def layer_range(n_layers: int, rank: int, world: int) -> tuple[int, int]:
    """Layers [first, end) of ``rank``: equal runs, the earlier ranks one longer when the count does not divide."""
    base, extra = divmod(n_layers, world)
    first = rank * base + min(rank, extra)
    return first, first + base + (1 if rank < extra else 0)


def split_layers(w: Weights, rank: int, world: int) -> Weights:
    """This rank's part of full weights: its run of layers under a config that lists only them, the embedding on the
    first rank's path and the head on the last one's (both tensors are kept where tied). The norm that follows a rank's
    last layer is the next rank's first input norm, so it travels in the ``final_norm`` field: the receiving rank gets
    a hidden state that is already normed for its first layer."""
    if not 1 <= world <= len(w.layers):
        raise ValueError(f"cannot split {len(w.layers)} layers over {world} ranks")
    first, end = layer_range(len(w.layers), rank, world)
    cfg = copy.deepcopy(w.config)
    cfg.layer_types = list(w.config.layer_types[first:end])
    cfg.num_hidden_layers = end - first
    cfg.mtp_num_hidden_layers = 0  # the draft head needs the whole stack's hidden state and embedding on one rank
    boundary = w.layers[end].input_norm if end < len(w.layers) else w.final_norm
    return Weights(cfg, w.embed, w.lm_head, boundary, list(w.layers[first:end]), None, w.vocab_start, w.full_vocab)
