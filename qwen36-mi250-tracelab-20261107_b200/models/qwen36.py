"""The hybrid Gated-DeltaNet / gated-attention MoE forward over packed rows.

One ``Model`` owns the weights, the paged KV pool and the GDN state slots of one
device and exposes three passes, all over *packed rows* (no padding between
sequences):

* ``prefill``  — one span per sequence (chunked prefill), any start position;
* ``decode``   — one row per sequence;
* ``verify``   — ``G`` rows per sequence (speculative chain), GDN states of every
  row kept so that the accepted prefix can be committed afterwards.

The reference's equivalent is ``FastModel`` (``engine/fast/model.py:296-472,
1220-1256, 1516-1670``). Which kernels run is decided by the ``ops`` object:
``ops.torch_ops`` (oracle, any device) or ``ops.cuda_ops`` (sm_100a kernels).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..config import PAGE_SIZE, ModelConfig
from ..ops import torch_ops
from .checkpoint import LayerWeights, Weights


@dataclass
class PackedBatch:
    """Host description of one pass. Lists are per sequence (segment)."""

    tokens: torch.Tensor  # [T] int64 on the model device
    seg_starts: list[int]  # len nseg+1, row offsets
    seg_slots: list[int]  # state slot of each sequence
    seg_pos0: list[int]  # position of each segment's first row
    block_tables: torch.Tensor  # [nseg, max_pages] int32 (device)

    @property
    def nseg(self) -> int:
        return len(self.seg_slots)

    def positions(self, device) -> torch.Tensor:
        pos = [
            torch.arange(p, p + (self.seg_starts[i + 1] - self.seg_starts[i]), dtype=torch.int64)
            for i, p in enumerate(self.seg_pos0)
        ]
        return torch.cat(pos).to(device) if pos else torch.zeros(0, dtype=torch.int64, device=device)


class Model:
    def __init__(
        self,
        weights: Weights,
        num_pages: int,
        state_slots: int,
        ops=None,
        kv_dtype: torch.dtype | None = None,
    ) -> None:
        self.w = weights
        self.cfg: ModelConfig = weights.config
        self.ops = ops or torch_ops
        cfg, dev, dt = self.cfg, weights.device, weights.dtype
        self.device, self.dtype = dev, dt
        self.num_pages, self.state_slots = num_pages, state_slots
        # page 0 and slot 0 are scratch targets for padding rows of fixed-size graph buckets
        self.kv = torch.zeros(
            cfg.num_kv_layers, num_pages, 2, cfg.num_key_value_heads, PAGE_SIZE, cfg.head_dim,
            dtype=kv_dtype or dt, device=dev,
        )
        n_gdn = len(cfg.gdn_layers)
        self.conv_state = torch.zeros(
            n_gdn, state_slots, cfg.gdn_conv_dim, cfg.linear_conv_kernel_dim - 1, dtype=dt, device=dev
        )
        self.rec_state = torch.zeros(
            n_gdn, state_slots, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim,
            dtype=torch.float32, device=dev,
        )
        self._kv_index = {layer: i for i, layer in enumerate(cfg.attention_layers)}
        self._gdn_index = {layer: i for i, layer in enumerate(cfg.gdn_layers)}
        self.mtp_kv_index = len(cfg.attention_layers)

    # ------------------------------------------------------------------ state management
    def reset_slot(self, slot: int) -> None:
        self.conv_state[:, slot].zero_()
        self.rec_state[:, slot].zero_()

    def copy_slot(self, src: int, dst: int) -> None:
        self.conv_state[:, dst].copy_(self.conv_state[:, src])
        self.rec_state[:, dst].copy_(self.rec_state[:, src])

    def copy_page(self, src: int, dst: int) -> None:
        self.kv[:, dst].copy_(self.kv[:, src])

    # ------------------------------------------------------------------ blocks
    def _moe(self, lw: LayerWeights, x: torch.Tensor) -> torch.Tensor:
        cfg, ops = self.cfg, self.ops
        E, k = cfg.num_experts, cfg.num_experts_per_tok
        logits = ops.linear(x, lw.router, out_dtype=torch.float32)
        wts, idx = ops.router_topk(logits[:, :E], k)
        if lw.shared_merged:
            sg = torch.sigmoid(logits[:, E : E + 1])
            wts = torch.cat([wts, sg], dim=1)
            idx = torch.cat([idx, torch.full_like(idx[:, :1], E)], dim=1)
            return ops.moe_experts(x, wts.to(x.dtype), idx, lw.w_gate_up, lw.w_down)
        routed = ops.moe_experts(x, wts.to(x.dtype), idx, lw.w_gate_up, lw.w_down)
        Is = lw.shared_gate_up.shape[0] // 2
        gu = ops.linear(x, lw.shared_gate_up)
        act = torch.nn.functional.silu(gu[:, :Is].float()).to(x.dtype) * gu[:, Is:]
        shared = ops.linear(act, lw.shared_down)
        sg = torch.sigmoid(ops.linear(x, lw.shared_gate, out_dtype=torch.float32))
        return routed + (sg * shared.float()).to(x.dtype)

    def _attention(self, lw, kv_layer, h, positions, batch: PackedBatch) -> torch.Tensor:
        cfg, ops = self.cfg, self.ops
        qkv = ops.linear(h, lw.in_proj)
        q, gate, k, v = ops.attn_prep(
            qkv, positions, lw.q_norm, lw.k_norm, cfg.num_attention_heads, cfg.num_key_value_heads,
            cfg.head_dim, cfg.rotary_dim, cfg.rope_theta, cfg.rms_norm_eps,
        )
        seg_of_row = torch.repeat_interleave(
            torch.arange(batch.nseg, device=h.device),
            torch.tensor([batch.seg_starts[i + 1] - batch.seg_starts[i] for i in range(batch.nseg)], device=h.device),
        )
        page_ids = batch.block_tables[seg_of_row, positions // PAGE_SIZE].long()
        ops.kv_write(kv_layer, k, v, page_ids, positions % PAGE_SIZE)
        core = ops.paged_attention(q, gate, kv_layer, batch.block_tables, batch.seg_starts, batch.seg_pos0)
        return ops.linear(core, lw.out_proj)

    def _gdn(self, lw, gi: int, h: torch.Tensor, batch: PackedBatch, mode: str, ring=None) -> torch.Tensor:
        cfg, ops = self.cfg, self.ops
        mixed = ops.linear(h, lw.in_proj)
        args = (
            lw.conv_w, lw.A_log, lw.dt_bias, lw.gnorm_w, cfg.linear_num_key_heads, cfg.linear_num_value_heads,
            cfg.linear_key_head_dim, cfg.linear_value_head_dim, cfg.rms_norm_eps,
        )
        conv, rec = self.conv_state[gi], self.rec_state[gi]
        if mode == "prefill":
            core = ops.gdn_prefill(mixed, batch.seg_starts, batch.seg_slots, conv, rec, *args)
        elif mode == "decode":
            slots = torch.tensor(batch.seg_slots, device=h.device)
            core = ops.gdn_decode(mixed, slots, conv, rec, *args)
        else:  # verify: G rows per sequence, one recurrent step per row, states after each row kept
            G = batch.seg_starts[1] - batch.seg_starts[0]
            B = batch.nseg
            slots = torch.tensor(batch.seg_slots, device=h.device)
            core = torch.empty(B * G, cfg.gdn_value_dim, dtype=h.dtype, device=h.device)
            rows = torch.arange(B, device=h.device) * G
            for j in range(G):
                core[rows + j] = ops.gdn_decode(mixed[rows + j], slots, conv, rec, *args)
                ring[0][gi, :, j] = conv[slots.long()]
                ring[1][gi, :, j] = rec[slots.long()]
        return ops.linear(core, lw.out_proj)

    def _layer(self, lw, x, res, positions, batch, mode, kv_layer=None, gi=None, ring=None):
        cfg, ops = self.cfg, self.ops
        res, h = ops.add_rmsnorm(x, res, lw.input_norm, cfg.rms_norm_eps)
        if lw.kind == "linear_attention":
            mix = self._gdn(lw, gi, h, batch, mode, ring)
        else:
            mix = self._attention(lw, kv_layer, h, positions, batch)
        res, h = ops.add_rmsnorm(mix, res, lw.post_norm, cfg.rms_norm_eps)
        return self._moe(lw, h), res

    # ------------------------------------------------------------------ passes
    def forward(self, batch: PackedBatch, mode: str, ring=None) -> torch.Tensor:
        """Run the layer stack; returns the final-normed hidden state of every row ``[T, H]``."""
        cfg, ops = self.cfg, self.ops
        positions = batch.positions(self.device)
        x = self.w.embed[batch.tokens]
        res = None
        for i, lw in enumerate(self.w.layers):
            if lw.kind == "linear_attention":
                x, res = self._layer(lw, x, res, positions, batch, mode, gi=self._gdn_index[i], ring=ring)
            else:
                x, res = self._layer(lw, x, res, positions, batch, mode, kv_layer=self.kv[self._kv_index[i]])
        _, h = ops.add_rmsnorm(x, res, self.w.final_norm, cfg.rms_norm_eps)
        return h

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.ops.linear(hidden, self.w.lm_head, out_dtype=torch.float32)

    def mtp_forward(self, hidden: torch.Tensor, next_tokens: torch.Tensor, batch: PackedBatch) -> torch.Tensor:
        """The MTP block over packed rows: row ``t`` pairs base hidden ``H[t]`` with token ``x[t+1]``.

        Writes the block's own KV (layer index ``mtp_kv_index``) at the rows' positions and
        returns the block's normed output ``[T, H]`` (feed to ``logits`` for token ``t+2``;
        reference: ``engine/mtp.py:7-12, 112-151``).
        """
        cfg, ops, m = self.cfg, self.ops, self.w.mtp
        e = ops.rmsnorm(self.w.embed[next_tokens], m.pre_fc_norm_embedding, cfg.rms_norm_eps)
        h = ops.rmsnorm(hidden, m.pre_fc_norm_hidden, cfg.rms_norm_eps)
        x = ops.linear(torch.cat([e, h], dim=-1), m.fc)
        positions = batch.positions(self.device)
        x, res = self._layer(m.layer, x, None, positions, batch, "prefill", kv_layer=self.kv[self.mtp_kv_index])
        _, y = ops.add_rmsnorm(x, res, m.norm, cfg.rms_norm_eps)
        return y

    # ------------------------------------------------------------------ verify ring (oracle path)
    def new_ring(self, B: int, G: int):
        cfg = self.cfg
        n_gdn = len(cfg.gdn_layers)
        conv = torch.empty(n_gdn, B, G, *self.conv_state.shape[2:], dtype=self.dtype, device=self.device)
        rec = torch.empty(n_gdn, B, G, *self.rec_state.shape[2:], dtype=torch.float32, device=self.device)
        return conv, rec

    def commit_ring(self, ring, slots: list[int], accepted_rows: list[int]) -> None:
        """Set each slot's GDN state to the state after row ``accepted_rows[i]`` of its verify rows."""
        for i, (slot, j) in enumerate(zip(slots, accepted_rows)):
            self.conv_state[:, slot] = ring[0][:, i, j]
            self.rec_state[:, slot] = ring[1][:, i, j]
