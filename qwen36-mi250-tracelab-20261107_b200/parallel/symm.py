"""Symmetric memory between the rank processes of one node, and the collectives built on it.

Each rank allocates its receive area, arrival flags and epoch counters with ``cudaMalloc`` inside
the kernel library, exports them as CUDA IPC handles, exchanges the handles through
``torch.distributed`` (plumbing only) and maps every peer's buffers, so that kernels can store
into and load from peer memory over NVLink directly (the reference maps fine-grained peer memory
between two GPUs of one process through ctypes calls into the HIP runtime,
``engine/fast/tp.py:341-420``; here ranks are processes, one per GPU).

``world == 1`` is a loopback group: the same kernels run against this rank's own buffers, which
is how single-GPU tests exercise the protocol. Multicast (NVLS) objects are not used: every
transfer is a plain peer store or load.
"""

from __future__ import annotations

import ctypes

import torch

from ..ops import cuda_ops

MAX_RANKS = 8
AR_ELEMS = 4096


class CommCtx(ctypes.Structure):
    _fields_ = [
        ("recv", ctypes.c_void_p * MAX_RANKS),
        ("flags", ctypes.c_void_p * MAX_RANKS),
        ("epoch", ctypes.c_void_p),
        ("err", ctypes.c_void_p),
        ("rank", ctypes.c_int),
        ("world", ctypes.c_int),
        ("max_blocks", ctypes.c_int),
        ("slot_elems", ctypes.c_ulonglong),
    ]


def _lib():
    L = cuda_ops.lib()
    if not getattr(L, "_comm_ready", False):
        P, I, U = ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong
        L.b200_symm_alloc.argtypes = [ctypes.POINTER(P), U]
        L.b200_symm_free.argtypes = [P]
        L.b200_symm_export.argtypes = [P, P]
        L.b200_symm_import.argtypes = [P, ctypes.POINTER(P)]
        L.b200_symm_close.argtypes = [P]
        L.b200_allreduce_push.argtypes = [ctypes.POINTER(CommCtx), P, I, P, P, P, U, P]
        for n in ("b200_symm_alloc", "b200_symm_free", "b200_symm_export", "b200_symm_import", "b200_symm_close",
                  "b200_allreduce_push", "b200_comm_ctx_size"):
            getattr(L, n).restype = I
        assert L.b200_comm_ctx_size() == ctypes.sizeof(CommCtx), "CommCtx layout mismatch"
        L._comm_ready = True
    return L


class SymmComm:
    """A rank group's symmetric buffers plus the one-shot all-reduce over them."""

    def __init__(self, device: torch.device, group=None, slot_elems: int = 1 << 20, max_blocks: int = 4096) -> None:
        import torch.distributed as dist

        self.device = device
        self.group = group
        self.rank = dist.get_rank(group) if group is not None else 0
        self.world = dist.get_world_size(group) if group is not None else 1
        if self.world > MAX_RANKS:
            raise ValueError(f"at most {MAX_RANKS} ranks per group")
        self.slot_elems = slot_elems
        self.max_blocks = max_blocks
        L = _lib()
        with torch.cuda.device(device):
            sizes = {
                "recv": 2 * self.world * slot_elems * 4,
                "flags": self.world * max_blocks * 4,
                "epoch": max_blocks * 4,
            }
            self._own: dict[str, int] = {}
            for name, nbytes in sizes.items():
                p = ctypes.c_void_p()
                if L.b200_symm_alloc(ctypes.byref(p), nbytes):
                    raise RuntimeError(f"symmetric allocation of {nbytes} bytes failed")
                self._own[name] = p.value
            torch.cuda.synchronize(device)
            self._peers: dict[str, list[int]] = {"recv": [], "flags": []}
            self._opened: list[int] = []
            if self.world == 1:
                self._peers = {"recv": [self._own["recv"]], "flags": [self._own["flags"]]}
            else:
                handles = {}
                for name in ("recv", "flags"):
                    buf = ctypes.create_string_buffer(64)
                    if L.b200_symm_export(self._own[name], buf):
                        raise RuntimeError("cudaIpcGetMemHandle failed")
                    handles[name] = buf.raw
                gathered: list = [None] * self.world
                dist.all_gather_object(gathered, handles, group=group)
                for r in range(self.world):
                    for name in ("recv", "flags"):
                        if r == self.rank:
                            self._peers[name].append(self._own[name])
                            continue
                        p = ctypes.c_void_p()
                        if L.b200_symm_import(gathered[r][name], ctypes.byref(p)):
                            raise RuntimeError(f"cudaIpcOpenMemHandle failed for rank {r}")
                        self._peers[name].append(p.value)
                        self._opened.append(p.value)
                dist.barrier(group=group)
        self.err = cuda_ops.err_word(device)
        ctx = CommCtx()
        for r in range(self.world):
            ctx.recv[r] = self._peers["recv"][r]
            ctx.flags[r] = self._peers["flags"][r]
        ctx.epoch = self._own["epoch"]
        ctx.err = self.err.data_ptr()
        ctx.rank, ctx.world, ctx.max_blocks, ctx.slot_elems = self.rank, self.world, max_blocks, slot_elems
        self.ctx = ctx

    def fits(self, n_elems: int) -> bool:
        return n_elems <= self.slot_elems and (n_elems + AR_ELEMS - 1) // AR_ELEMS <= self.max_blocks

    def allreduce(self, partial: torch.Tensor, residual: torch.Tensor | None = None,
                  out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """Sum ``partial`` (bf16 or fp32, contiguous) over the group; bf16 output may add ``residual``."""
        assert partial.is_contiguous() and partial.numel() % 4 == 0
        n = partial.numel()
        if not self.fits(n):
            raise ValueError(f"{n} elements exceed the symmetric slot ({self.slot_elems})")
        f32 = out_dtype == torch.float32
        out = torch.empty(partial.shape, dtype=out_dtype, device=partial.device)
        rc = _lib().b200_allreduce_push(
            ctypes.byref(self.ctx), partial.data_ptr(), int(partial.dtype == torch.float32),
            None if residual is None else residual.data_ptr(), None if f32 else out.data_ptr(),
            out.data_ptr() if f32 else None, n, torch.cuda.current_stream().cuda_stream,
        )
        if rc:
            raise cuda_ops.KernelError(f"allreduce_push failed with code {rc}")
        return out

    def allreduce_norm(self, partial: torch.Tensor, residual: torch.Tensor | None, norm_w: torch.Tensor, eps: float):
        """Sum rows ``partial [T, H]`` over the group, add ``residual`` and apply the zero-centred RMSNorm that follows,
        all in the all-reduce kernel; returns ``(new residual, normed)`` with the bits of the separate kernels."""
        assert partial.is_contiguous() and partial.dim() == 2
        T, H = partial.shape
        out = torch.empty(T, H, dtype=torch.bfloat16, device=partial.device)
        y = torch.empty_like(out)
        L = _lib()
        if not getattr(L, "_arn_ready", False):
            P, I = ctypes.c_void_p, ctypes.c_int
            L.b200_allreduce_push_norm.argtypes = [P, P, I, P, P, P, P, I, I, ctypes.c_float, P]
            L.b200_allreduce_push_norm.restype = I
            L._arn_ready = True
        rc = L.b200_allreduce_push_norm(
            ctypes.byref(self.ctx), partial.data_ptr(), int(partial.dtype == torch.float32),
            None if residual is None else residual.data_ptr(), out.data_ptr(), norm_w.data_ptr(), y.data_ptr(), T, H, eps,
            torch.cuda.current_stream().cuda_stream,
        )
        if rc:
            raise cuda_ops.KernelError(f"allreduce_push_norm failed with code {rc}")
        return out, y

    def norm_fits(self, T: int, H: int) -> bool:
        return H >= 64 and AR_ELEMS % H == 0 and self.fits(T * H)

    def close(self) -> None:
        L = _lib()
        torch.cuda.synchronize(self.device)
        for p in self._opened:
            L.b200_symm_close(p)
        self._opened = []
        for p in self._own.values():
            L.b200_symm_free(p)
        self._own = {}
