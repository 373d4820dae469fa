"""Tensor + expert parallel sharding of the model inside one replica.

Layout for a group of ``R`` ranks (one process per GPU):

* Gated DeltaNet: key heads and value heads split ``R`` ways together with their conv
  channels, ``in_proj`` rows, ``A_log`` / ``dt_bias``; ``out_proj`` split along its input
  (each rank produces a partial ``[T, H]``).
* Gated attention: query heads (with their gates) split; KV heads split while ``R`` divides
  them, else each rank keeps the one KV head its query heads use; ``o_proj`` split along its
  input.
* MoE: router replicated; the routed experts are distributed ``E / R`` per rank (expert
  parallelism) and the shared expert lives whole on rank ``layer % R``. Activations are
  replicated after every all-reduce, so each rank serves the (row, expert) pairs of its own
  experts for all rows and the partial sums meet in the block's all-reduce.
* Embedding, norms, MTP ``fc`` replicated; ``lm_head`` split by vocabulary rows with a
  cross-rank ``(max, index)`` pick.

Two all-reduces per layer, as in the reference's TP=2 (``engine/fast/tp.py:1-24, 670-800``), which
halves every expert instead of distributing them and supports exactly two ranks. ``Comm``
implementations: ``SymmComm`` kernels over NVLink peer memory (fused into the projection GEMM's
epilogue) and ``DistComm`` over ``torch.distributed`` (NCCL on GPUs as the baseline path, gloo
for CPU ranks in tests).
"""

from __future__ import annotations

import copy
import ctypes
from dataclasses import dataclass

import torch

from ..config import ModelConfig
from ..models.checkpoint import LayerWeights, MTPWeights, Weights


# --------------------------------------------------------------------------- communication
class DistComm:
    """Collectives through ``torch.distributed`` (the library baseline; also CPU ranks over gloo)."""

    fused = False

    def __init__(self, group=None) -> None:
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    def allreduce(self, partial: torch.Tensor, residual: torch.Tensor | None = None,
                  out_dtype: torch.dtype | None = None) -> torch.Tensor:
        out_dtype = out_dtype or (residual.dtype if residual is not None else torch.bfloat16)
        acc = partial.float().contiguous()
        self.dist.all_reduce(acc, group=self.group)
        out = acc.to(out_dtype)
        if residual is not None:
            out = (out.float() + residual.float()).to(out_dtype)
        return out

    def gemm_allreduce(self, ops, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        return self.allreduce(ops.linear(x, w, out_dtype=torch.float32), residual, x.dtype)

    def argmax(self, val: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        """Global greedy pick from per-rank (max, index): larger value wins, ties to the lower index."""
        vals = [torch.empty_like(val) for _ in range(self.world)]
        idxs = [torch.empty_like(idx) for _ in range(self.world)]
        self.dist.all_gather(vals, val.contiguous(), group=self.group)
        self.dist.all_gather(idxs, idx.contiguous(), group=self.group)
        best_v, best_i = vals[0], idxs[0]
        for v, i in zip(vals[1:], idxs[1:]):
            take = (v > best_v) | ((v == best_v) & (i < best_i))
            best_v, best_i = torch.where(take, v, best_v), torch.where(take, i, best_i)
        return best_i


class FusedComm(DistComm):
    """NVLink peer-memory kernels for decode-sized messages; larger ones fall back to the library."""

    fused = True

    def __init__(self, device: torch.device, group=None, slot_elems: int = 1 << 21, max_blocks: int = 4096) -> None:
        super().__init__(group)
        from .symm import SymmComm

        self.symm = SymmComm(device, group, slot_elems, max_blocks)

    def allreduce(self, partial, residual=None, out_dtype=None):
        out_dtype = out_dtype or torch.bfloat16
        if partial.is_cuda and self.symm.fits(partial.numel()) and partial.numel() % 4 == 0 and out_dtype == torch.bfloat16:
            return self.symm.allreduce(partial.contiguous(), residual)
        return super().allreduce(partial, residual, out_dtype)

    def allreduce_norm(self, partial, residual, norm_w, eps):
        """All-reduce + residual add + the next RMSNorm in one kernel when the rows fit a block of the push
        all-reduce; ``None`` otherwise (the caller then runs the separate ops)."""
        if partial.is_cuda and partial.dim() == 2 and self.symm.norm_fits(*partial.shape) and norm_w.dtype == torch.bfloat16:
            return self.symm.allreduce_norm(partial.contiguous(), residual, norm_w, eps)
        return None

    def argmax(self, val: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        """Cross-rank greedy pick without a library collective (so that it can live inside a CUDA graph):
        every rank fills its own row of a ``[world, T, 2]`` fp32 table (value, index; indices below 2^24
        are exact in fp32), the one-shot all-reduce adds the disjoint rows, then each rank picks."""
        if not val.is_cuda:
            return super().argmax(val, idx)
        T = val.shape[0]
        table = torch.zeros(self.world, T, 2, dtype=torch.float32, device=val.device)
        table[self.rank, :, 0] = val
        table[self.rank, :, 1] = idx.float()
        table = self.symm.allreduce(table, out_dtype=torch.float32)
        best_v, best_i = table[0, :, 0], table[0, :, 1]
        for r in range(1, self.world):
            v, i = table[r, :, 0], table[r, :, 1]
            take = (v > best_v) | ((v == best_v) & (i < best_i))
            best_v, best_i = torch.where(take, v, best_v), torch.where(take, i, best_i)
        return best_i.long()

    def gemm_allreduce(self, ops, x, w, residual=None):
        from ..ops import cuda_ops
        from .symm import _lib

        T, K = x.shape
        N = w.shape[0]
        bt = cuda_ops.lib().b200_pick_bt(T)
        blocks = ((N + 127) // 128) * ((T + bt - 1) // bt)
        if not (x.is_cuda and T * N <= self.symm.slot_elems and blocks <= self.symm.max_blocks):
            return super().gemm_allreduce(ops, x, w, residual)
        L = _lib()
        if not getattr(L, "_gar_ready", False):
            P, I = ctypes.c_void_p, ctypes.c_int
            L.b200_gemm_allreduce.argtypes = [ctypes.c_void_p, P, P, P, P, I, I, I, I, I, I, P]
            L.b200_gemm_allreduce.restype = I
            L._gar_ready = True
        out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
        rc = L.b200_gemm_allreduce(
            ctypes.byref(self.symm.ctx), x.data_ptr(), w.data_ptr(), None if residual is None else residual.data_ptr(),
            out.data_ptr(), T, N, K, x.stride(0), w.stride(0), bt, torch.cuda.current_stream().cuda_stream,
        )
        if rc:
            raise cuda_ops.KernelError(f"gemm_allreduce failed with code {rc}")
        return out


# --------------------------------------------------------------------------- sharding
@dataclass
class TPContext:
    rank: int
    world: int
    comm: DistComm
    vocab_start: int = 0  # first vocabulary row of this rank's lm_head shard


def local_config(cfg: ModelConfig, world: int) -> ModelConfig:
    """The per-rank view of the architecture: local head counts, everything else unchanged."""
    if cfg.linear_num_key_heads % world or cfg.linear_num_value_heads % world or cfg.num_attention_heads % world:
        raise ValueError(f"tensor parallel size {world} does not divide the head counts")
    if cfg.num_experts % world:
        raise ValueError(f"expert parallel size {world} does not divide {cfg.num_experts} experts")
    lc = copy.deepcopy(cfg)
    lc.linear_num_key_heads //= world
    lc.linear_num_value_heads //= world
    lc.num_attention_heads //= world
    lc.num_key_value_heads = max(1, cfg.num_key_value_heads // world)
    return lc


def _rows(t: torch.Tensor, start: int, n: int) -> torch.Tensor:
    return t[start : start + n].contiguous()


def shard_layer(lw: LayerWeights, cfg: ModelConfig, rank: int, world: int, layer_index: int) -> LayerWeights:
    out = copy.copy(lw)
    if lw.kind == "linear_attention":
        hk, hv = cfg.linear_num_key_heads // world, cfg.linear_num_value_heads // world
        dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        kd, vd = cfg.gdn_key_dim, cfg.gdn_value_dim
        q0, k0, v0 = rank * hk * dk, kd + rank * hk * dk, 2 * kd + rank * hv * dv
        z0 = cfg.gdn_conv_dim + rank * hv * dv
        b0 = cfg.gdn_conv_dim + vd + rank * hv
        a0 = b0 + cfg.linear_num_value_heads
        w = lw.in_proj
        out.in_proj = torch.cat([_rows(w, q0, hk * dk), _rows(w, k0, hk * dk), _rows(w, v0, hv * dv),
                                 _rows(w, z0, hv * dv), _rows(w, b0, hv), _rows(w, a0, hv)], 0)
        c = lw.conv_w
        out.conv_w = torch.cat([_rows(c, q0, hk * dk), _rows(c, k0, hk * dk), _rows(c, v0, hv * dv)], 0)
        out.A_log = _rows(lw.A_log, rank * hv, hv)
        out.dt_bias = _rows(lw.dt_bias, rank * hv, hv)
        out.out_proj = lw.out_proj[:, rank * hv * dv : (rank + 1) * hv * dv].contiguous()
    else:
        nq, D = cfg.num_attention_heads // world, cfg.head_dim
        nkv_l = max(1, cfg.num_key_value_heads // world)
        q_rows = cfg.attn_q_rows
        kv_head0 = (rank * nq) // (cfg.num_attention_heads // cfg.num_key_value_heads)  # KV head of this rank's first Q head
        w = lw.in_proj
        out.in_proj = torch.cat([
            _rows(w, rank * nq * 2 * D, nq * 2 * D),
            _rows(w, q_rows + kv_head0 * D, nkv_l * D),
            _rows(w, q_rows + cfg.attn_kv_rows + kv_head0 * D, nkv_l * D),
        ], 0)
        out.out_proj = lw.out_proj[:, rank * nq * D : (rank + 1) * nq * D].contiguous()
    E = cfg.num_experts
    per = E // world
    e0 = rank * per
    if not lw.shared_merged:
        raise ValueError("expert parallelism expects the shared expert stored as expert E")
    host_shared = (layer_index % world) == rank
    ids = list(range(e0, e0 + per)) + ([E] if host_shared else [])
    sel = torch.tensor(ids, device=lw.w_gate_up.device)
    out.w_gate_up = lw.w_gate_up[sel].contiguous()
    out.w_down = lw.w_down[sel].contiguous()
    emap = torch.full((E + 1,), -1, dtype=torch.int32)
    emap[torch.tensor(ids)] = torch.arange(len(ids), dtype=torch.int32)
    out.expert_map = emap.to(lw.w_gate_up.device)
    return out


def shard_weights(w: Weights, rank: int, world: int) -> Weights:
    """This rank's shard of full weights (tests and small models; big models shard layer by layer at load)."""
    cfg = w.config
    lc = local_config(cfg, world)
    layers = [shard_layer(lw, cfg, rank, world, i) for i, lw in enumerate(w.layers)]
    V = cfg.vocab_size
    per = (V + world - 1) // world
    v0, v1 = rank * per, min(V, (rank + 1) * per)
    mtp = None
    if w.mtp is not None:
        m = w.mtp
        mtp = MTPWeights(m.fc, m.pre_fc_norm_embedding, m.pre_fc_norm_hidden, m.norm,
                         shard_layer(m.layer, cfg, rank, world, len(w.layers)))
    return Weights(lc, w.embed, w.lm_head[v0:v1].contiguous(), w.final_norm, layers, mtp, vocab_start=v0, full_vocab=V)
