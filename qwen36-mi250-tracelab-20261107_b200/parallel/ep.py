"""Expert-parallel MoE block for token-sharded activations (each rank owns different rows).

``EpMoE.forward`` runs, on every rank of the group and in the same order: router GEMM + top-k on the
rank's own rows, the dispatch all-to-all (rows stored straight into the hosting rank's receive region
for this source over NVLink, no count exchange first), a plan kernel that waits for every source and
sorts the received rows by expert without moving them, the grouped gate/up GEMM whose producer fetches
those rows by index, the grouped down GEMM whose epilogue scatters every output row back to its owner
(the combine all-to-all), and the top-k weighted sum (with the residual add and next RMSNorm). Kernels: ``ops/cuda/ep_moe.cu`` and the ``EPI_SCATTER`` epilogue of
``ops/cuda/gemm_tcgen05.cu``; buffers are CUDA IPC symmetric memory as in ``parallel/symm.py``.
The reference has no expert parallelism (``engine/fast/tp.py:19-21``: tensor parallelism over two devices only);
this block is what lets the experts of the 35B model be spread over 2, 4 or 8 GPUs with data-parallel attention.
"""

from __future__ import annotations

import ctypes

import torch

from ..ops import cuda_ops
from .symm import MAX_RANKS, _lib as _symm_lib


class EpCtx(ctypes.Structure):
    _fields_ = [
        ("xs", ctypes.c_void_p * MAX_RANKS),
        ("meta", ctypes.c_void_p * MAX_RANKS),
        ("pair_out", ctypes.c_void_p * MAX_RANKS),
        ("arrive", ctypes.c_void_p * MAX_RANKS),
        ("flags", ctypes.c_void_p * MAX_RANKS),
        ("epoch", ctypes.c_void_p),
        ("cursors", ctypes.c_void_p),
        ("err", ctypes.c_void_p),
        ("rank", ctypes.c_int),
        ("world", ctypes.c_int),
        ("E", ctypes.c_int),
        ("per", ctypes.c_int),
        ("cap_src", ctypes.c_int),
        ("max_pairs", ctypes.c_int),
        ("wait_cycles", ctypes.c_longlong),
    ]


def _lib():
    L = _symm_lib()
    if not getattr(L, "_ep_ready", False):
        P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        C = ctypes.POINTER(EpCtx)
        L.b200_ep_route_send.argtypes = [C, P, P, I, I, I, I, I, P, P, P]
        L.b200_ep_plan.argtypes = [C, I, P, P, I, P, P, P, P]
        L.b200_ep_compact.argtypes = [P, P, P, I, I, P, P]
        L.b200_ep_combine.argtypes = [C, P, I, I, I, P, P, P, P, P, F, P]
        L.b200_gemm_grouped_scatter.argtypes = [P, P, I, I, I, I, I, P, P, I, P, P, I, P, I, P]
        for n in ("b200_ep_route_send", "b200_ep_plan", "b200_ep_compact", "b200_ep_combine", "b200_gemm_grouped_scatter",
                  "b200_ep_ctx_size"):
            getattr(L, n).restype = I
        assert L.b200_ep_ctx_size() == ctypes.sizeof(EpCtx), "EpCtx layout mismatch"
        L._ep_ready = True
    return L


class EpMoE:
    # widest token tile whose rows the gate/up GEMM fetches by index from the receive buffer; wider tiles (prefill-size
    # blocks) are compacted into expert order first. The local block gathers up to 64 rows; here the 32-row form is the
    # one measured on 2 and 4 GPUs.
    GATHER_MAX_BT = 32

    def __init__(self, device: torch.device, group, n_experts: int, hidden: int, top_k: int, max_rows: int,
                 capacity_factor: float | None = None, wait_s: float = 1.0) -> None:
        """``max_rows``: most rows any rank brings to one call. Every rank keeps one receive region per source rank;
        a region holds ``cap_src`` rows. By default that is the worst case (every pair of a source lands on one
        host); ``capacity_factor`` f sizes it for f times the uniform share instead (plus the shared expert's rows),
        and a call that needs more sets the error word rather than dropping rows silently. ``wait_s``: how long a
        kernel waits for a peer's rows or results before it gives up with a status (about a second when the ranks are
        driven in step by one program; replicas that launch from separate server processes need more slack)."""
        import torch.distributed as dist

        self.device, self.group = device, group
        self.rank = dist.get_rank(group) if group is not None else 0
        self.world = dist.get_world_size(group) if group is not None else 1
        self.E, self.H, self.top_k = n_experts, hidden, top_k
        self.P = top_k + 1
        self.per = n_experts // self.world
        self.max_rows = max_rows
        self.max_pairs = max_rows * self.P
        worst = self.max_pairs
        if capacity_factor is None:
            self.cap_src = worst
        else:
            share = -(-max_rows * top_k // self.world)
            self.cap_src = min(worst, max(256, int(capacity_factor * share)) + max_rows)
        self.cap_rows = self.cap_src * self.world
        L = _lib()
        sizes = {
            "xs": self.cap_rows * hidden * 2,
            "meta": self.cap_rows * 8,
            "pair_out": self.max_pairs * hidden * 2,
            "arrive": MAX_RANKS * 8,
            "flags": 2 * MAX_RANKS * 4,
            "epoch": 16,
            "cursors": (MAX_RANKS + 1) * 4,
        }
        self._own, self._opened = {}, []
        self._work: dict = {}

        def agree(ok: bool, what: str) -> None:
            """Every rank raises if any rank failed, so that nobody is left waiting in the next collective."""
            if self.world > 1:
                t = torch.tensor([0 if ok else 1], device=device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
                ok = t.item() == 0
            if not ok:
                self.close()
                raise RuntimeError(f"expert-parallel set-up failed on some rank: {what}")

        shared = ("xs", "meta", "pair_out", "arrive", "flags")
        with torch.cuda.device(device):
            ok = True
            for name, nbytes in sizes.items():
                p = ctypes.c_void_p()
                if L.b200_symm_alloc(ctypes.byref(p), nbytes):
                    ok = False
                    break
                self._own[name] = p.value
            torch.cuda.synchronize(device)
            agree(ok, "symmetric allocation")
            peers = {k: [self._own[k]] * 1 for k in shared}
            if self.world > 1:
                handles, ok = {}, True
                for name in peers:
                    buf = ctypes.create_string_buffer(64)
                    if L.b200_symm_export(self._own[name], buf):
                        ok = False
                    handles[name] = buf.raw
                agree(ok, "cudaIpcGetMemHandle")
                gathered: list = [None] * self.world
                dist.all_gather_object(gathered, handles, group=group)
                peers = {k: [] for k in peers}
                ok = True
                for r in range(self.world):
                    for name in peers:
                        if r == self.rank:
                            peers[name].append(self._own[name])
                            continue
                        p = ctypes.c_void_p()
                        if L.b200_symm_import(gathered[r][name], ctypes.byref(p)):
                            ok = False
                            peers[name].append(None)
                            continue
                        peers[name].append(p.value)
                        self._opened.append(p.value)
                agree(ok, "cudaIpcOpenMemHandle")
        ctx = EpCtx()
        for r in range(self.world):
            for name in peers:
                getattr(ctx, name)[r] = peers[name][r]
        ctx.epoch = self._own["epoch"]
        ctx.cursors = self._own["cursors"]
        ctx.err = cuda_ops.err_word(device).data_ptr()
        ctx.rank, ctx.world, ctx.E, ctx.per = self.rank, self.world, n_experts, self.per
        ctx.cap_src, ctx.max_pairs = self.cap_src, self.max_pairs
        ctx.wait_cycles = int(max(0.05, wait_s) * 2.0e9)  # clock64 ticks at about 2 GHz
        self.ctx = ctx
        self._pair_out_ptrs = (ctypes.c_void_p * MAX_RANKS)(*[peers["pair_out"][r] if r < self.world else None
                                                             for r in range(MAX_RANKS)])

    def local_experts(self, w_gate_up: torch.Tensor, w_down: torch.Tensor):
        """This rank's slice of full stacked expert weights ``[E + 1, ...]``: its routed experts, then the shared one."""
        ids = list(range(self.rank * self.per, (self.rank + 1) * self.per)) + [self.E]
        sel = torch.tensor(ids, device=w_gate_up.device)
        return w_gate_up[sel].contiguous(), w_down[sel].contiguous()

    def _buffers(self, inter: int, dtype: torch.dtype):
        """Host-side work buffers of the received rows (activations, tile table, sort indices), made once per expert
        width: their size depends on the receive capacity only, never on a call's row count."""
        w = self._work.get(inter)
        if w is None:
            dev = self.device
            max_tiles = self.per + 1 + self.cap_rows // 16 + 1  # enough for the narrowest token tile
            w = self._work[inter] = dict(
                act=torch.empty(self.cap_rows, inter, dtype=dtype, device=dev),
                tiles=torch.empty(max_tiles, 4, dtype=torch.int32, device=dev),
                gather_rows=torch.zeros(self.cap_rows, dtype=torch.int32, device=dev),
                ret_meta=torch.zeros(self.cap_rows, 2, dtype=torch.int32, device=dev),
                ints=torch.zeros(2, dtype=torch.int32, device=dev),
                sorted=None, max_tiles=max_tiles,
            )
        return w

    def reserve(self, inter: int, dtype: torch.dtype) -> None:
        """Allocate every work buffer a call can need for experts of width ``inter`` now (a server does this before it
        sizes its KV pool, so that the first long prefill pass does not find the memory gone)."""
        w = self._buffers(inter, dtype)
        if w["sorted"] is None:
            w["sorted"] = torch.empty(self.cap_rows, self.H, dtype=dtype, device=self.device)

    def forward(self, x: torch.Tensor, router: torch.Tensor, w_gate_up_local: torch.Tensor,
                w_down_local: torch.Tensor, residual: torch.Tensor | None = None, norm_w: torch.Tensor | None = None,
                eps: float = 1e-6):
        """The MoE block of this rank's rows. With ``norm_w`` the combine kernel also adds ``residual`` and applies
        the next RMSNorm, and the call returns ``(new residual, normed)``; otherwise it returns the block's output."""
        T, H = x.shape
        assert T * self.P <= self.max_pairs and H == self.H and x.is_contiguous()
        dev, L, st = x.device, _lib(), torch.cuda.current_stream().cuda_stream
        K = cuda_ops.lib()
        E, Pn = self.E, self.P
        inter = w_down_local.shape[2]
        n_pairs = T * Pn
        logits = cuda_ops.linear(x, router, out_dtype=torch.float32)
        wts = torch.empty(T, Pn, dtype=torch.float32, device=dev)
        idx = torch.empty(T, Pn, dtype=torch.int32, device=dev)
        codes: list = []  # every launcher's return code: a failure names the call
        C = ctypes.byref(self.ctx)
        # routing and dispatch in one launch: a CTA per row routes it, then sends its pairs to their hosts
        codes.append(("route_send", L.b200_ep_route_send(C, x.data_ptr(), logits.data_ptr(), logits.stride(0), T, self.top_k, Pn, H,
                                  wts.data_ptr(), idx.data_ptr(), st)))
        # token tile of this host's GEMMs from the rows it can expect (its own count times the ranks); a row's bits
        # do not depend on it, so ranks with different batches need not agree
        bt = cuda_ops.moe_bt(max(T, 1) * self.world, Pn, E)
        w = self._buffers(inter, x.dtype)
        n_tiles, n_rows = w["ints"][:1], w["ints"][1:]
        codes.append(("plan", L.b200_ep_plan(C, bt, w["tiles"].data_ptr(), n_tiles.data_ptr(), w["max_tiles"],
                             w["gather_rows"].data_ptr(), w["ret_meta"].data_ptr(), n_rows.data_ptr(), st)))
        err = cuda_ops.err_word(dev)
        if bt <= min(cuda_ops.GATHER_MAX_BT, self.GATHER_MAX_BT):
            codes.append(("gate_up(gather)", K.b200_gemm_grouped(self._own["xs"], w_gate_up_local.data_ptr(), w["act"].data_ptr(), self.cap_rows,
                                      self.per + 1, inter, 2 * inter, H, inter, cuda_ops.EPI_SILU_MUL, inter, bt,
                                      w["tiles"].data_ptr(), n_tiles.data_ptr(), w["max_tiles"], err.data_ptr(), 1,
                                      cuda_ops.is_packed(w_gate_up_local), w["gather_rows"].data_ptr(), H, st)))
        else:
            if w["sorted"] is None:
                w["sorted"] = torch.empty(self.cap_rows, H, dtype=x.dtype, device=dev)
            codes.append(("compact", L.b200_ep_compact(self._own["xs"], w["gather_rows"].data_ptr(), n_rows.data_ptr(), self.cap_rows, H,
                                    w["sorted"].data_ptr(), st)))
            codes.append(("gate_up", K.b200_gemm_grouped(w["sorted"].data_ptr(), w_gate_up_local.data_ptr(), w["act"].data_ptr(),
                                      self.cap_rows, self.per + 1, inter, 2 * inter, H, inter, cuda_ops.EPI_SILU_MUL,
                                      inter, bt, w["tiles"].data_ptr(), n_tiles.data_ptr(), w["max_tiles"],
                                      err.data_ptr(), 1, cuda_ops.is_packed(w_gate_up_local), None, 0, st)))
        codes.append(("down(scatter)", L.b200_gemm_grouped_scatter(w["act"].data_ptr(), w_down_local.data_ptr(), self.cap_rows, self.per + 1, H,
                                          inter, bt, w["tiles"].data_ptr(), n_tiles.data_ptr(), w["max_tiles"],
                                          w["ret_meta"].data_ptr(), self._pair_out_ptrs, self.world, err.data_ptr(),
                                          cuda_ops.is_packed(w_down_local), st)))
        if norm_w is not None:
            new_res, y = torch.empty_like(x), torch.empty_like(x)
            codes.append(("combine", L.b200_ep_combine(C, wts.data_ptr(), T, Pn, H, None,
                                                     None if residual is None else residual.data_ptr(), norm_w.data_ptr(),
                                                     new_res.data_ptr(), y.data_ptr(), eps, st)))
            out = (new_res, y)
        else:
            out = torch.empty_like(x)
            codes.append(("combine", L.b200_ep_combine(C, wts.data_ptr(), T, Pn, H, out.data_ptr(), None, None, None, None, 0.0, st)))
        bad = [(n, c) for n, c in codes if c]
        if bad:
            raise cuda_ops.KernelError(f"expert-parallel MoE failed: {bad} (rows {T}, token tile {bt})")
        return out

    def close(self) -> None:
        L = _lib()
        torch.cuda.synchronize(self.device)
        for p in getattr(self, "_opened", []):
            L.b200_symm_close(p)
        for p in getattr(self, "_own", {}).values():
            L.b200_symm_free(p)
        self._opened, self._own = [], {}


def shard_layer_experts(lw, n_experts: int, rank: int, world: int):
    """One layer with only this rank's ``E / world`` routed experts and the shared expert (stacked last)."""
    import copy

    if n_experts % world:
        raise ValueError(f"{n_experts} experts do not split over {world} ranks")
    if not lw.shared_merged:
        raise ValueError("expert parallelism needs the shared expert merged into the expert stack")
    per = n_experts // world
    out = copy.copy(lw)
    sel = torch.tensor(list(range(rank * per, (rank + 1) * per)) + [n_experts], device=lw.w_gate_up.device)
    out.w_gate_up = lw.w_gate_up[sel].contiguous()
    out.w_down = lw.w_down[sel].contiguous()
    return out


def shard_experts(weights, rank: int, world: int):
    """This rank's weights for data-parallel attention + expert-parallel MoE: everything dense stays whole, every
    layer keeps only its ``E / world`` routed experts and a replica of the shared expert (stacked last), in the order
    ``EpMoE`` expects. The MTP block is dropped (drafting would make the ranks' pass sequences differ)."""
    from ..models.checkpoint import Weights

    cfg = weights.config
    layers = [shard_layer_experts(lw, cfg.num_experts, rank, world) for lw in weights.layers]
    return Weights(cfg, weights.embed, weights.lm_head, weights.final_norm, layers, None)
