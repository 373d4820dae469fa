"""Sequence-parallel tensor parallelism for prefill-size passes: fused GEMM -> reduce-scatter and
all-gather -> GEMM over NVLink peer memory.

With T token rows replicated on R ranks, a one-shot all-reduce after every row-parallel projection moves
``T * N * 4 * (R - 1)`` bytes out of each GPU. For large T this class keeps the residual stream row-sharded
instead (rank r owns rows ``[r * T / R, (r + 1) * T / R)``) and runs three kernels per half-layer:

* ``gemm_reduce_scatter``: the row-parallel GEMM (``ops/cuda/gemm_tcgen05.cu``, ``EPI_REDUCE_SCATTER``)
  stores each fp32 partial tile straight from TMEM into the owner rank's receive slot and releases the tile's
  arrival flag; it never waits. ``(R - 1) / R`` of the all-reduce bytes.
* ``reduce_norm_allgather`` (``ops/cuda/allreduce.cu``): the owner waits for the flags of a row's tiles, adds
  the partials in rank order plus the residual, stores the new residual row, and pushes the RMSNorm of the row
  into every rank's full activation buffer; the last CTA publishes one arrival epoch for the shard.
* ``gemm_gathered``: the following column-parallel GEMM reads the full buffer locally; its TMA producer
  waits only for the shard that owns the tile's rows, so tiles of early shards overlap the rest of the gather.

Calls must be made in the same order on every rank. Two ``gemm_reduce_scatter`` calls must be separated by a
``reduce_norm_allgather`` + ``gemm_gathered`` pair (as in a transformer layer): that pair is what guarantees that an
owner has finished reading a receive slot before a peer writes it again. The reference has no counterpart
(its tensor parallelism is a 2-GPU all-reduce, ``engine/fast/tp.py:132-162``).
"""

from __future__ import annotations

import ctypes

import torch

from ..ops import cuda_ops
from .symm import MAX_RANKS, CommCtx, SymmComm, _lib as _symm_lib


class AgCtx(ctypes.Structure):
    _fields_ = [
        ("xfull", ctypes.c_void_p * MAX_RANKS),
        ("flags", ctypes.c_void_p * MAX_RANKS),
        ("epoch", ctypes.c_void_p),
        ("counter", ctypes.c_void_p),
        ("rank", ctypes.c_int),
        ("world", ctypes.c_int),
    ]


def _lib():
    L = _symm_lib()
    if not getattr(L, "_sp_ready", False):
        P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.b200_gemm_reduce_scatter.argtypes = [ctypes.POINTER(CommCtx), P, P, I, I, I, I, I, I, P]
        L.b200_gemm_gathered.argtypes = [P, P, P, I, I, I, I, I, I, I, I, I, P, P, P, P]
        L.b200_reduce_norm_allgather.argtypes = [ctypes.POINTER(AgCtx), ctypes.POINTER(CommCtx), P, P, P, P, I, I, F, I, I, P]
        L.b200_rs_push.argtypes = [ctypes.POINTER(CommCtx), P, I, I, I, P]
        L.b200_ag_wait.argtypes = [ctypes.POINTER(AgCtx), P, P]
        L.b200_ag_wait.restype = I
        for n in ("b200_gemm_reduce_scatter", "b200_gemm_gathered", "b200_reduce_norm_allgather", "b200_ag_ctx_size",
                  "b200_rs_push"):
            getattr(L, n).restype = I
        assert L.b200_ag_ctx_size() == ctypes.sizeof(AgCtx), "AgCtx layout mismatch"
        L._sp_ready = True
    return L


class _DevMem:
    """A raw device allocation seen through ``__cuda_array_interface__`` so that torch can view it."""

    def __init__(self, ptr: int, n_u16: int) -> None:
        self.__cuda_array_interface__ = {"shape": (n_u16,), "typestr": "<u2", "data": (ptr, False), "version": 3,
                                         "strides": None}


class SeqParallel:
    def __init__(self, device: torch.device, group, max_rows: int, hidden: int, max_n: int | None = None) -> None:
        """``max_rows``: most token rows of one pass (all ranks together); ``max_n``: widest reduce-scattered output."""
        import torch.distributed as dist

        self.device, self.group = device, group
        self.rank = dist.get_rank(group) if group is not None else 0
        self.world = dist.get_world_size(group) if group is not None else 1
        self.max_rows, self.H = max_rows, hidden
        self.bt_cap = 256  # widest token tile of the three kernels
        n = max_n or hidden
        rpr = (max_rows + self.world - 1) // self.world
        self.comm = SymmComm(device, group, slot_elems=rpr * n, max_blocks=max(4096, ((n + 127) // 128) * (max_rows // 16 + 1)))
        L = _lib()
        sizes = {"xfull": max_rows * hidden * 2, "flags": MAX_RANKS * 4, "epoch": 16, "counter": 16}
        self._own, self._opened = {}, []
        with torch.cuda.device(device):
            for name, nbytes in sizes.items():
                p = ctypes.c_void_p()
                if L.b200_symm_alloc(ctypes.byref(p), nbytes):
                    raise RuntimeError(f"symmetric allocation of {nbytes} bytes failed")
                self._own[name] = p.value
            torch.cuda.synchronize(device)
            peers = {k: [self._own[k]] for k in ("xfull", "flags")}
            if self.world > 1:
                handles = {}
                for name in peers:
                    buf = ctypes.create_string_buffer(64)
                    if L.b200_symm_export(self._own[name], buf):
                        raise RuntimeError("cudaIpcGetMemHandle failed")
                    handles[name] = buf.raw
                gathered: list = [None] * self.world
                dist.all_gather_object(gathered, handles, group=group)
                peers = {k: [] for k in peers}
                for r in range(self.world):
                    for name in peers:
                        if r == self.rank:
                            peers[name].append(self._own[name])
                            continue
                        p = ctypes.c_void_p()
                        if L.b200_symm_import(gathered[r][name], ctypes.byref(p)):
                            raise RuntimeError(f"cudaIpcOpenMemHandle failed for rank {r}")
                        peers[name].append(p.value)
                        self._opened.append(p.value)
                dist.barrier(group=group)
        ctx = AgCtx()
        for r in range(self.world):
            ctx.xfull[r], ctx.flags[r] = peers["xfull"][r], peers["flags"][r]
        ctx.epoch, ctx.counter = self._own["epoch"], self._own["counter"]
        ctx.rank, ctx.world = self.rank, self.world
        self.ctx = ctx
        self._xfull = torch.as_tensor(_DevMem(self._own["xfull"], max_rows * hidden), device=device).view(torch.bfloat16)

    def rows_per_rank(self, T: int) -> int:
        if T % self.world:
            raise ValueError(f"{T} rows do not split over {self.world} ranks")
        return T // self.world

    def _bt(self, rpr: int) -> int:
        bt = min(cuda_ops.lib().b200_pick_bt(rpr), self.bt_cap)
        while rpr % bt:
            bt //= 2
        if bt < 16:
            raise ValueError(f"{rpr} rows per rank are not a multiple of 16")
        return bt

    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor) -> int:
        """``x [T, K/R] @ w [N, K/R]^T``: every rank's fp32 partial of rank r's rows lands in rank r's receive
        slots. Returns the rows per rank; ``reduce_norm_allgather`` must follow on every rank."""
        T, K = x.shape
        N = w.shape[0]
        assert N == self.H
        rpr = self.rows_per_rank(T)
        rc = _lib().b200_gemm_reduce_scatter(ctypes.byref(self.comm.ctx), x.data_ptr(), w.data_ptr(), T, N, K,
                                             x.stride(0), w.stride(0), self._bt(rpr),
                                             torch.cuda.current_stream().cuda_stream)
        if rc:
            raise cuda_ops.KernelError(f"gemm_reduce_scatter failed with code {rc}")
        return rpr

    def push_reduce_scatter(self, partial: torch.Tensor) -> int:
        """Reduce-scatter of an fp32 partial ``[T, H]`` that no GEMM produced (the expert-parallel MoE output):
        same receive slots and flags as ``gemm_reduce_scatter``; ``reduce_norm_allgather`` must follow."""
        T, N = partial.shape
        assert N == self.H and partial.dtype == torch.float32 and partial.is_contiguous()
        rpr = self.rows_per_rank(T)
        rc = _lib().b200_rs_push(ctypes.byref(self.comm.ctx), partial.data_ptr(), T, N, self._bt(rpr),
                                 torch.cuda.current_stream().cuda_stream)
        if rc:
            raise cuda_ops.KernelError(f"rs_push failed with code {rc}")
        return rpr

    def reduce_norm_allgather(self, rows: int, residual: torch.Tensor | None, w: torch.Tensor, eps: float,
                              zero_centred: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
        """Finish the reduce-scatter: new residual rows ``[rows, H]`` of this rank = bf16(sum of partials) +
        ``residual``; their RMSNorm is pushed into every rank's full buffer. Returns (new residual, full view)."""
        new_res = torch.empty(rows, self.H, dtype=torch.bfloat16, device=self.device)
        rc = _lib().b200_reduce_norm_allgather(ctypes.byref(self.ctx), ctypes.byref(self.comm.ctx), None,
                                               None if residual is None else residual.data_ptr(), new_res.data_ptr(),
                                               w.data_ptr(), rows, self.H, eps, int(zero_centred), self._bt(rows),
                                               torch.cuda.current_stream().cuda_stream)
        if rc:
            raise cuda_ops.KernelError(f"reduce_norm_allgather failed with code {rc}")
        return new_res, self._xfull[: rows * self.world * self.H].view(rows * self.world, self.H)

    def norm_allgather(self, x: torch.Tensor, w: torch.Tensor, eps: float, zero_centred: bool = True) -> torch.Tensor:
        """RMSNorm of this rank's rows, pushed into every rank's full buffer; returns the (not yet complete) view."""
        rows, H = x.shape
        assert H == self.H and rows * self.world <= self.max_rows and x.is_contiguous()
        rc = _lib().b200_reduce_norm_allgather(ctypes.byref(self.ctx), None, x.data_ptr(), None, None, w.data_ptr(), rows,
                                               H, eps, int(zero_centred), 0, torch.cuda.current_stream().cuda_stream)
        if rc:
            raise cuda_ops.KernelError(f"norm_allgather failed with code {rc}")
        return self._xfull[: rows * self.world * H].view(rows * self.world, H)

    def wait_all(self, xfull: torch.Tensor) -> torch.Tensor:
        """Make the stream wait until every shard of the last all-gather is in ``xfull`` (for consumers other than
        ``gemm_gathered``)."""
        rc = _lib().b200_ag_wait(ctypes.byref(self.ctx), cuda_ops.err_word(self.device).data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)
        if rc:
            raise cuda_ops.KernelError(f"ag_wait failed with code {rc}")
        return xfull

    def barrier(self) -> None:
        """Order this rank's stream after everything every rank has enqueued so far (a 4-float one-shot all-reduce):
        the first push of a pass must not land in a buffer a peer is still reading from the previous pass."""
        self.comm.allreduce(torch.zeros(4, dtype=torch.float32, device=self.device), out_dtype=torch.float32)

    def gemm_gathered(self, xfull: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """``xfull @ w^T`` where ``xfull`` is the view ``norm_allgather`` returned: tiles wait for their shard only."""
        T, K = xfull.shape
        N = w.shape[0]
        rpr = self.rows_per_rank(T)
        bt = self._bt(rpr)
        out = torch.empty(T, N, dtype=out_dtype, device=xfull.device)
        rc = _lib().b200_gemm_gathered(xfull.data_ptr(), w.data_ptr(), out.data_ptr(), T, N, K, xfull.stride(0),
                                       w.stride(0), int(out_dtype == torch.float32), bt, rpr, self.rank * (rpr // bt), self._own["flags"],
                                       self._own["epoch"], cuda_ops.err_word(xfull.device).data_ptr(),
                                       torch.cuda.current_stream().cuda_stream)
        if rc:
            raise cuda_ops.KernelError(f"gemm_gathered failed with code {rc}")
        return out

    def close(self) -> None:
        L = _lib()
        torch.cuda.synchronize(self.device)
        self._xfull = None
        for p in self._opened:
            L.b200_symm_close(p)
        for p in self._own.values():
            L.b200_symm_free(p)
        self._opened, self._own = [], {}
        self.comm.close()
