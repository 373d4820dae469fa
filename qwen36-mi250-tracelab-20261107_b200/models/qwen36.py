"""The hybrid Gated-DeltaNet / gated-attention MoE forward over packed rows.

One ``Model`` owns the weights, the paged KV pool and the GDN state slots of one
device and runs three kinds of pass, all over *packed rows* (no padding between
sequences):

* prefill — one span per sequence (chunked prefill), any start position (``G = 0``);
* decode  — one row per sequence (``G = 1``);
* verify  — ``G = k + 1`` rows per sequence (speculative chain); the GDN state after
  every row is kept in a ring so that the accepted prefix can be committed.

The reference's equivalent is ``FastModel`` (``engine/fast/model.py:296-472,
1220-1256, 1516-1670``). Which kernels run is decided by ``ops``:
``ops.torch_ops`` (oracle, any device) or ``ops.cuda_ops`` (sm_100a kernels).
Decode and verify passes touch only device tensors of fixed shape, so a pass can be
captured in a CUDA graph and replayed on refreshed input buffers.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..config import PAGE_SIZE, ModelConfig
from ..ops import torch_ops
from .checkpoint import LayerWeights, Weights


@dataclass
class PackedBatch:
    """One pass. Device tensors drive the kernels; the host lists exist for ragged prefill only."""

    tokens: torch.Tensor  # [T] int64
    positions: torch.Tensor  # [T] int64
    seq_of_row: torch.Tensor  # [T] int32, row -> sequence index
    slots: torch.Tensor  # [nseg] int32 state slot of each sequence
    block_tables: torch.Tensor  # [nseg, max_pages] int32
    G: int  # rows per sequence (decode 1, verify k+1); 0 = ragged prefill
    seg_starts: list[int] | None = None
    seg_slots: list[int] | None = None
    seg_pos0: list[int] | None = None
    meta: object | None = None  # ragged prefill from fixed-shape device tables (``sched/graphs.py`` ``PrefillTables``)

    @classmethod
    def prefill(cls, token_lists, slots, pos0, block_tables, device) -> "PackedBatch":
        lens = [len(t) for t in token_lists]
        starts = [0]
        for n in lens:
            starts.append(starts[-1] + n)
        tokens = torch.tensor([t for ts in token_lists for t in ts], dtype=torch.int64)
        positions = torch.cat([torch.arange(p, p + n, dtype=torch.int64) for p, n in zip(pos0, lens)])
        seq = torch.repeat_interleave(torch.arange(len(lens), dtype=torch.int32), torch.tensor(lens))
        return cls(
            tokens.to(device), positions.to(device), seq.to(device),
            torch.tensor(slots, dtype=torch.int32, device=device), block_tables.to(device), 0,
            starts, list(slots), list(pos0),
        )

    @classmethod
    def uniform(cls, tokens, positions, slots, block_tables, G: int, device) -> "PackedBatch":
        """Decode (``G = 1``) or verify batch from host lists: ``tokens``/``positions`` hold ``B*G`` entries."""
        B = len(slots)
        seq = torch.repeat_interleave(torch.arange(B, dtype=torch.int32), G)
        return cls(
            torch.as_tensor(tokens, dtype=torch.int64).to(device),
            torch.as_tensor(positions, dtype=torch.int64).to(device),
            seq.to(device), torch.as_tensor(slots, dtype=torch.int32).to(device), block_tables.to(device), G,
        )


class Model:
    def __init__(self, weights: Weights, num_pages: int, state_slots: int, ops=None,
                 kv_dtype: torch.dtype | None = None, tp=None, ep=None, pp=None) -> None:
        """``weights`` may be one rank's shard (``parallel.tp.shard_weights``); then ``tp`` names the rank
        group and every mixer / MoE output is summed across it. ``ep`` (a ``parallel.ep.EpMoE``) selects data-parallel
        attention with expert-parallel MoE instead: this rank serves its own rows with full dense weights, holds only
        its share of the routed experts (``parallel.ep.shard_experts``) and exchanges rows with the other ranks inside
        every MoE block, so all ranks must run their forward passes in step. ``pp`` (a ``parallel.pp.PPContext``) marks
        ``weights`` as one rank's run of layers (``parallel.pp.split_layers``): the pass receives its input rows from the
        rank before and hands its output to the rank after."""
        self.tp = tp
        self.ep = ep
        self.pp = pp
        self.draft_index = None  # spec.ivf.IvfIndex: draft picks from a vocabulary shortlist instead of the full head
        self.w = weights
        self.cfg: ModelConfig = weights.config
        self.ops = ops or torch_ops
        cfg, dev, dt = self.cfg, weights.device, weights.dtype
        self.device, self.dtype = dev, dt
        self.num_pages, self.state_slots = num_pages, state_slots
        # page 0 and slot 0 are scratch targets for the padding rows of fixed-size graph buckets
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

    def new_ring(self, B: int, G: int):
        """Per-layer state-after-row buffers of one verify pass."""
        n_gdn = len(self.cfg.gdn_layers)
        conv = torch.empty(n_gdn, B, G, *self.conv_state.shape[2:], dtype=self.dtype, device=self.device)
        rec = torch.empty(n_gdn, B, G, *self.rec_state.shape[2:], dtype=torch.float32, device=self.device)
        return conv, rec

    def commit_ring(self, ring, slots: torch.Tensor, keep_rows: torch.Tensor) -> None:
        """Set each slot's GDN state to the state after row ``keep_rows[i]`` of its verify rows."""
        if hasattr(self.ops, "ring_commit") and self.device.type == "cuda" \
                and ring[0][0, 0, 0].numel() * ring[0].element_size() % 16 == 0:
            self.ops.ring_commit(self.conv_state, self.rec_state, ring, slots, keep_rows)
            return
        b = torch.arange(slots.shape[0], device=self.device)
        sl, kr = slots.long(), keep_rows.long()
        self.conv_state[:, sl] = ring[0][:, b, kr]
        self.rec_state[:, sl] = ring[1][:, b, kr]

    # ------------------------------------------------------------------ blocks
    def _moe(self, lw: LayerWeights, x: torch.Tensor) -> torch.Tensor:
        cfg, ops = self.cfg, self.ops
        if self.ep is not None:  # token-sharded expert parallelism: all-to-all dispatch / combine over peer memory
            return self.ep.forward(x, lw.router, lw.w_gate_up, lw.w_down)
        if self.tp is not None:  # expert parallel: local experts only, partial sums meet in the all-reduce
            part = ops.moe_block(x, lw.router, lw.w_gate_up, lw.w_down, cfg.num_experts, cfg.num_experts_per_tok,
                                 True, expert_map=lw.expert_map, partial_f32=True)
            return self.tp.comm.allreduce(part, None, x.dtype)
        out = ops.moe_block(x, lw.router, lw.w_gate_up, lw.w_down, cfg.num_experts, cfg.num_experts_per_tok,
                            lw.shared_merged)
        if lw.shared_merged:
            return out
        act = ops.linear_silu_mul(x, lw.shared_gate_up)
        shared = ops.linear(act, lw.shared_down)
        sg = torch.sigmoid(ops.linear(x, lw.shared_gate, out_dtype=torch.float32))
        return out + (sg * shared.float()).to(x.dtype)

    def _attention(self, lw, kv_layer, h, batch: PackedBatch) -> torch.Tensor:
        cfg, ops = self.cfg, self.ops
        qkv = ops.linear(h, lw.in_proj)
        core = ops.attention(
            qkv, batch.positions, batch.seq_of_row, batch.block_tables, kv_layer, lw.q_norm, lw.k_norm,
            cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rotary_dim, cfg.rope_theta,
            cfg.rms_norm_eps, batch.G, batch.seg_starts, batch.seg_pos0,
            **({} if batch.meta is None else {"meta": batch.meta.flash}),
        )
        return self._out_proj(core, lw.out_proj)

    def _gdn(self, lw, gi: int, h: torch.Tensor, batch: PackedBatch, ring) -> torch.Tensor:
        cfg, ops = self.cfg, self.ops
        mixed = ops.linear(h, lw.in_proj)
        args = (
            lw.conv_w, lw.A_log, lw.dt_bias, lw.gnorm_w, cfg.linear_num_key_heads, cfg.linear_num_value_heads,
            cfg.linear_key_head_dim, cfg.linear_value_head_dim, cfg.rms_norm_eps,
        )
        conv, rec = self.conv_state[gi], self.rec_state[gi]
        if batch.G == 0:
            core = ops.gdn_prefill(mixed, batch.seg_starts, batch.seg_slots, conv, rec, *args,
                                   **({} if batch.meta is None else {"meta": batch.meta.gdn}))
        else:
            r = None if ring is None else (ring[0][gi], ring[1][gi])
            core = ops.gdn_decode(mixed, batch.slots, conv, rec, *args, G=batch.G, ring=r)
        return self._out_proj(core, lw.out_proj)

    def _out_proj(self, core: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """Mixer output projection; under tensor parallelism the GEMM's epilogue is the all-reduce."""
        if self.tp is None:
            return self.ops.linear(core, w)
        return self.tp.comm.gemm_allreduce(self.ops, core, w)

    def _moe_norm(self, lw: LayerWeights, h: torch.Tensor, res: torch.Tensor, norm_w: torch.Tensor):
        """MoE block, residual add and the RMSNorm that follows it (the next layer's input norm or the final norm);
        returns ``(new residual, normed)``. On the CUDA path of one GPU the three are one kernel behind the grouped
        GEMMs (reference: ``engine/fast/fused.py:635-692`` folds combine + shared expert + residual into its down
        kernel); elsewhere the norm is its own op, with identical rounding points."""
        cfg, ops = self.cfg, self.ops
        if self.ep is not None:  # the combine kernel of the expert-parallel block carries the residual add and the norm
            return self.ep.forward(h, lw.router, lw.w_gate_up, lw.w_down, residual=res, norm_w=norm_w,
                                   eps=cfg.rms_norm_eps)
        if self.tp is not None and hasattr(self.tp.comm, "allreduce_norm"):
            # tensor + expert parallel: the partial sums of the local experts meet in an all-reduce whose kernel also
            # adds the residual and applies the next norm (one launch instead of three)
            part = ops.moe_block(h, lw.router, lw.w_gate_up, lw.w_down, cfg.num_experts, cfg.num_experts_per_tok,
                                 True, expert_map=lw.expert_map, partial_f32=True)
            fused = self.tp.comm.allreduce_norm(part, res, norm_w, cfg.rms_norm_eps)
            if fused is not None:
                return fused
            return ops.add_rmsnorm(self.tp.comm.allreduce(part, None, h.dtype), res, norm_w, cfg.rms_norm_eps)
        if self.tp is None and lw.shared_merged and getattr(ops, "FUSED_MOE_NORM", False):
            return ops.moe_block(h, lw.router, lw.w_gate_up, lw.w_down, cfg.num_experts, cfg.num_experts_per_tok, True,
                                 residual=res, norm_w=norm_w, eps=cfg.rms_norm_eps)
        return ops.add_rmsnorm(self._moe(lw, h), res, norm_w, cfg.rms_norm_eps)

    def _layer(self, lw, h, res, batch, next_norm, kv_layer=None, gi=None, ring=None):
        """One decoder layer from its normed input ``h`` and the residual stream ``res``; returns the new residual
        and the input of the next layer, already normed with ``next_norm``."""
        cfg, ops = self.cfg, self.ops
        if lw.kind == "linear_attention":
            mix = self._gdn(lw, gi, h, batch, ring)
        else:
            mix = self._attention(lw, kv_layer, h, batch)
        res, h = ops.add_rmsnorm(mix, res, lw.post_norm, cfg.rms_norm_eps)
        return self._moe_norm(lw, h, res, next_norm)

    # ------------------------------------------------------------------ passes
    SP_MIN_ROWS = 512  # prefill passes at least this long take the sequence-parallel collectives under TP

    def _sp(self, T: int):
        """The rank group's sequence-parallel kernels when this prefill pass should use them, else None."""
        tp = self.tp
        if tp is None or not getattr(tp.comm, "fused", False) or T < self.SP_MIN_ROWS or not self.device.type == "cuda":
            return None
        sp = getattr(tp, "sp", None)
        if sp is None:
            from ..parallel.sp import SeqParallel

            sp = tp.sp = SeqParallel(self.device, tp.comm.group, max_rows=self.SP_MAX_ROWS, hidden=self.cfg.hidden_size)
        unit = tp.world * 128
        return sp if (T + unit - 1) // unit * unit <= sp.max_rows else None

    SP_MAX_ROWS = 16384

    def _forward_sp(self, batch: PackedBatch, sp) -> torch.Tensor:
        """Prefill pass under tensor parallelism with a row-sharded residual stream: every all-reduce becomes a
        reduce-scatter into the owner's rows, RMSNorm runs on the owned rows only, and the all-gather is the
        norm kernel's stores into every rank's activation buffer, which the next GEMM consumes shard by shard
        (``parallel/sp.py``). Rows are padded to a multiple of ``world * 128``; padding rows belong to no
        sequence, feed only the GEMMs, and are dropped at the end."""
        cfg, ops, R = self.cfg, self.ops, self.tp.world
        ops.DECODE_MODE = False
        T = batch.tokens.shape[0]
        unit = R * 128
        Tp = (T + unit - 1) // unit * unit
        rpr = Tp // R
        eps = cfg.rms_norm_eps
        x = ops.embed(batch.tokens, self.w.embed)
        if Tp != T:
            x = torch.cat([x, x.new_zeros(Tp - T, x.shape[1])])
        res = x[self.tp.rank * rpr:(self.tp.rank + 1) * rpr].contiguous()      # this rank's rows of the residual
        sp.barrier()  # no peer is still reading its activation buffer from an earlier pass
        full = sp.norm_allgather(res, self.w.layers[0].input_norm, eps)         # first norm: no reduction yet

        def pad(t: torch.Tensor) -> torch.Tensor:
            return t if Tp == T else torch.cat([t, t.new_zeros(Tp - T, t.shape[1])])

        for i, lw in enumerate(self.w.layers):
            mixed = sp.gemm_gathered(full, lw.in_proj)
            if lw.kind == "linear_attention":
                gi = self._gdn_index[i]
                core = ops.gdn_prefill(mixed[:T], batch.seg_starts, batch.seg_slots, self.conv_state[gi], self.rec_state[gi],
                                       lw.conv_w, lw.A_log, lw.dt_bias, lw.gnorm_w, cfg.linear_num_key_heads,
                                       cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim, eps)
            else:
                core = ops.attention(mixed[:T], batch.positions, batch.seq_of_row, batch.block_tables,
                                     self.kv[self._kv_index[i]], lw.q_norm, lw.k_norm, cfg.num_attention_heads,
                                     cfg.num_key_value_heads, cfg.head_dim, cfg.rotary_dim, cfg.rope_theta, eps, 0,
                                     batch.seg_starts, batch.seg_pos0)
            sp.gemm_reduce_scatter(pad(core), lw.out_proj)
            res, full = sp.reduce_norm_allgather(rpr, res, lw.post_norm, eps)
            logits = sp.gemm_gathered(full, lw.router, out_dtype=torch.float32)
            part = ops.moe_block(full, lw.router, lw.w_gate_up, lw.w_down, cfg.num_experts, cfg.num_experts_per_tok,
                                 True, expert_map=lw.expert_map, partial_f32=True, logits=logits)
            sp.push_reduce_scatter(part)
            nxt = self.w.layers[i + 1].input_norm if i + 1 < len(self.w.layers) else self.w.final_norm
            res, full = sp.reduce_norm_allgather(rpr, res, nxt, eps)
        # the last all-gather has no GEMM behind it to wait for the shards: a one-row gathered GEMM would do, but the
        # final hidden state is consumed by the LM head on the host's schedule, so wait for every shard here
        sp.wait_all(full)
        return full[:T].clone()

    def forward(self, batch: PackedBatch, ring=None) -> torch.Tensor:
        """Run the layer stack; returns the final-normed hidden state of every row ``[T, H]``."""
        cfg, ops = self.cfg, self.ops
        if batch.G == 0:
            sp = self._sp(batch.tokens.shape[0])
            if sp is not None:
                return self._forward_sp(batch, sp)
        ops.DECODE_MODE = batch.G > 0  # decode / verify passes may split K across clusters; prefill never does
        layers = self.w.layers
        pp = self.pp
        if pp is not None and not pp.is_first:
            res, h = pp.recv(batch.tokens.shape[0], cfg.hidden_size, self.dtype, self.device)
        else:
            x = ops.embed(batch.tokens, self.w.embed)
            res, h = ops.add_rmsnorm(x, None, layers[0].input_norm, cfg.rms_norm_eps)
        for i, lw in enumerate(layers):
            nxt = layers[i + 1].input_norm if i + 1 < len(layers) else self.w.final_norm
            if lw.kind == "linear_attention":
                res, h = self._layer(lw, h, res, batch, nxt, gi=self._gdn_index[i], ring=ring)
            else:
                res, h = self._layer(lw, h, res, batch, nxt, kv_layer=self.kv[self._kv_index[i]])
        if pp is not None and not pp.is_last:
            pp.send(res, h)  # normed with the next rank's first input norm (carried in final_norm)
        return h

    def forward_empty(self) -> None:
        """This rank's share of a pass in which it has no rows (data-parallel attention with expert-parallel MoE): it
        still hosts experts for the other ranks' rows, so it takes part in every layer's dispatch and combine."""
        assert self.ep is not None
        x = torch.empty(0, self.cfg.hidden_size, dtype=self.dtype, device=self.device)
        for lw in self.w.layers:
            self.ep.forward(x, lw.router, lw.w_gate_up, lw.w_down, residual=None, norm_w=lw.post_norm,
                            eps=self.cfg.rms_norm_eps)

    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        if self.pp is not None:  # only the last rank's hidden state is the stack's output
            out = self.ops.linear(hidden, self.w.lm_head, out_dtype=torch.float32) if self.pp.is_last else None
            return self.pp.share(out, (hidden.shape[0], self.w.lm_head.shape[0]), torch.float32, self.device)
        out = self.ops.linear(hidden, self.w.lm_head, out_dtype=torch.float32)
        if self.tp is None:
            return out
        import torch.distributed as dist

        V = self.w.full_vocab
        per = (V + self.tp.world - 1) // self.tp.world
        pad = torch.full((out.shape[0], per), float("-inf"), dtype=out.dtype, device=out.device)
        pad[:, : out.shape[1]] = out
        parts = [torch.empty_like(pad) for _ in range(self.tp.world)]
        dist.all_gather(parts, pad, group=self.tp.comm.group)
        return torch.cat(parts, dim=1)[:, :V]

    def greedy(self, hidden: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Greedy next token of each row (LM head with fused argmax on the CUDA path). ``out``: int64 ``[rows]``
        tensor that receives the picks (the captured speculative step assembles its result vector in place)."""
        if self.pp is not None:
            picks = self.ops.lm_head_argmax(hidden, self.w.lm_head) if self.pp.is_last else None
            picks = self.pp.share(picks, (hidden.shape[0],), torch.int64, self.device)
            if out is not None:
                out.copy_(picks)
                return out
            return picks
        if self.tp is None:
            if out is not None and self.ops is not torch_ops:
                return self.ops.lm_head_argmax(hidden, self.w.lm_head, out=out)
            picks = self.ops.lm_head_argmax(hidden, self.w.lm_head)
        else:
            idx, val = self.ops.lm_head_argmax(hidden, self.w.lm_head, return_value=True)
            picks = self.tp.comm.argmax(val, idx + self.w.vocab_start)
        if out is not None:
            out.copy_(picks)
            return out
        return picks

    def draft_pick(self, hidden: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Draft token of each row of the MTP block's output: the full greedy head, or the best token of a
        vocabulary shortlist when a draft index is attached (only a guess is needed: the verify pass decides)."""
        if self.draft_index is None or self.tp is not None:
            return self.greedy(hidden, out=out)
        return self.draft_index.pick(self.ops, hidden, self.w.lm_head, out=out)

    def mtp_forward(self, hidden: torch.Tensor, next_tokens: torch.Tensor, batch: PackedBatch) -> torch.Tensor:
        """The MTP block over packed rows: row ``t`` pairs base hidden ``H[t]`` with token ``x[t+1]``.

        Writes the block's own KV (layer index ``mtp_kv_index``) at the rows' positions and
        returns the block's normed output ``[T, H]`` (feed to ``logits``/``greedy`` for token
        ``t+2``; reference: ``engine/mtp.py:7-12, 112-151``).
        """
        cfg, ops, m = self.cfg, self.ops, self.w.mtp
        if hasattr(ops, "mtp_in") and hidden.is_contiguous():  # embedding gather, both pre-norms and the concat: one kernel
            x_in = ops.mtp_in(next_tokens, self.w.embed, hidden, m.pre_fc_norm_embedding, m.pre_fc_norm_hidden,
                              cfg.rms_norm_eps)
        else:
            e = ops.rmsnorm(ops.embed(next_tokens, self.w.embed), m.pre_fc_norm_embedding, cfg.rms_norm_eps)
            h = ops.rmsnorm(hidden, m.pre_fc_norm_hidden, cfg.rms_norm_eps)
            x_in = torch.cat([e, h], dim=-1)
        x = ops.linear(x_in, m.fc)
        res, h = ops.add_rmsnorm(x, None, m.layer.input_norm, cfg.rms_norm_eps)
        _, y = self._layer(m.layer, h, res, batch, m.norm, kv_layer=self.kv[self.mtp_kv_index])
        return y
