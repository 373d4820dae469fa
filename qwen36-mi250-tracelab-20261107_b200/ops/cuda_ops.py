"""ctypes bindings of the sm_100a kernel library, with the same call signatures as ``torch_ops``.

The library (``ops/cuda/libb200serve_kernels.so``) is built ahead of time by
``ops/build.py`` and must be present on a GPU machine: importing this module on a
machine with a CUDA device and no library raises, so a missing build can never
turn into a silent PyTorch fallback. Every launcher takes raw device pointers and
the current CUDA stream, which makes each call capturable in a CUDA graph
(the reference gets graph-capturable launches from ``hipModuleLaunchKernel`` on the
current stream, ``engine/fast/hipmega_rtc.py:150-215``).
"""

from __future__ import annotations

import ctypes
import time
from ctypes import c_float, c_int, c_void_p

import torch

from ..obs import buildlog
from . import torch_ops
from .build import lib_path

_lib = None
ATTN_Z = 32  # context lanes of the decode attention (fixed: part of the numerics contract)

EPI_BF16, EPI_F32, EPI_SILU_MUL, EPI_ARGMAX = 0, 1, 2, 3


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.PyDLL:
    global _lib
    if _lib is None:
        path = lib_path()
        if not path.exists():
            raise KernelError(f"{path} is missing: run `python -m b200serve.ops.build` (or __graft_entry__.build())")
        t0 = time.perf_counter()
        # PyDLL: the interpreter lock stays with the calling thread during a call. Every entry point is an
        # asynchronous launch of a few microseconds; giving the lock up around each one (what CDLL does) makes the
        # engine thread queue for it again behind the request threads several hundred times per pass, which under a
        # burst of requests stretched one pass to seconds.
        _lib = ctypes.PyDLL(str(path))
        buildlog.record("load", path.name, time.perf_counter() - t0)
        for name in dir(_Sig):
            if name.startswith("b200_"):
                fn = getattr(_lib, name)
                fn.restype = c_int
                fn.argtypes = getattr(_Sig, name)
    return _lib


P, I, F = c_void_p, c_int, c_float


class _Sig:
    b200_pick_bt = [I]
    b200_gemm_dense = [P, P, P, I, I, I, I, I, I, I, I, I, P, P, P, I, I, P]
    b200_gemm_grouped = [P, P, P, I, I, I, I, I, I, I, I, I, P, P, I, P, I, I, P, I, P]
    b200_argmax_finish = [P, P, I, I, P, P, P]
    b200_ivf_pick = [P, I, P, I, I, I, P, I, P, P, I, I, P, P, I, P, P]
    b200_embed = [P, P, P, I, I, I, P]
    b200_add_rmsnorm = [P, P, P, P, P, I, I, F, I, P]
    b200_moe_route = [P, I, I, I, I, I, P, P, P, I, P, P]
    b200_moe_plan = [P, I, I, I, P, P, P, I, P, P, P, I, P, P]
    b200_moe_route_plan = [P, I, I, I, I, I, P, P, P, I, I, P, P, P, I, P, P, P, P, P, P]
    b200_moe_combine_norm = [P, P, P, I, I, I, P, P, P, P, F, P]
    b200_mtp_in = [P, P, P, P, P, P, I, I, I, F, P]
    b200_chain_accept = [P, P, P, P, P, I, I, I, I, P, P, P, P]
    b200_moe_gather = [P, P, P, I, I, I, I, P, P]
    b200_moe_combine = [P, P, P, I, I, I, P, P, P]
    b200_gdn_decode = [P, I, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P, P]
    b200_attn_prep = [P, I, P, P, I, P, P, P, P, P, P, I, I, I, I, I, F, F, I, P, P]
    b200_paged_attn = [P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, P]
    b200_gdn_prefill = [P, I, P, P, P, P, P, P, P, P, P, P, P, I, P, I, P, P, P, I, I, I, I, I, F, I, P, P]
    b200_gdn_prefill_work_stride = [I]
    b200_ring_commit = [P, P, P, P, P, P, I, I, I, I, I, ctypes.c_ulonglong, ctypes.c_ulonglong, P]
    b200_flash_prefill = [P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, I, P, P, I, P, P]
    b200_attn_combine = [P, P, P, P, I, I, I, I, P]


def launch_count() -> int:
    """Kernels launched through the library so far; taken around a graph capture it is the graph's kernel count."""
    fn = lib().b200_launch_count
    fn.restype = ctypes.c_ulonglong
    fn.argtypes = []
    return int(fn())


def _ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


_err: dict[int, torch.Tensor] = {}
_tickets: dict[int, torch.Tensor] = {}


def _ticket(device: torch.device) -> torch.Tensor:
    """The counter word of kernels whose last CTA finishes the job: zero between launches (the kernel puts it back).
    One per device, like the error word: the engine issues every pass of a device on one stream, and launches that
    share the word must be ordered."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _tickets:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("first use of the ticket word inside a graph capture: run the pass once eagerly first")
        _tickets[idx] = torch.zeros(1 + 2 * 1024, dtype=torch.int32, device=device)  # ticket, expert counts, expert cursors
        torch.cuda.synchronize(device)
    return _tickets[idx]


def err_word(device: torch.device) -> torch.Tensor:
    """The per-device error word kernels write when a bounded wait or an index check fails."""
    cur = torch.cuda.current_device()
    idx = device.index if device.index is not None else cur
    if idx != cur:
        # launches go to the calling thread's current device and stream; the current device is a property of the
        # host thread (0 in every new thread), so a worker thread of a replica on another device must select it first
        raise KernelError(f"tensors on cuda:{idx} but the calling thread's current device is cuda:{cur}: "
                          f"call torch.cuda.set_device({idx}) in this thread")
    if idx not in _err:
        _err[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _err[idx]


def check_errors(device: torch.device) -> None:
    """Read the error word (synchronises) and raise if any kernel recorded a failure."""
    code = int(err_word(device).item())
    if code:
        err_word(device).zero_()
        names = {1: "TMA stage never arrived", 2: "no free pipeline stage", 3: "accumulator never completed",
                 4: "peer flag never arrived", 5: "index out of range"}
        raise KernelError(f"device-side failure {code}: {names.get(code, 'unknown')}")


# --------------------------------------------------------------------------- GEMM family
DECODE_MODE = False  # set by Model.forward: True for decode / verify passes
# Split-K over thread-block clusters for decode passes. Measured on B200 (batch 1: 4.34 -> 3.94 ms per step;
# batch 128: 18.1 -> 19.3 ms, the leader CTA's DSMEM reads of seven partial tiles cost more than the extra
# CTAs save), so it is off unless ENGINE_SPLIT_K=1; the split factor must not depend on the batch size.
SPLIT_K_ENABLED = __import__("os").environ.get("ENGINE_SPLIT_K", "0") == "1"
# Gated DeltaNet prefill with head dims of 128: tcgen05 WY transform and state pass (ENGINE_GDN_TC=0 selects the fp32
# CUDA-core kernels, which other head dims always use)
GDN_PREFILL_TC = __import__("os").environ.get("ENGINE_GDN_TC", "1") == "1"


def split_k(N: int, K: int, grouped: bool = False) -> int:
    """CTAs per cluster that share one output tile along K. A function of the weight shape and of the kind
    of pass only (never of the number of rows), so a row's bits do not depend on its batch."""
    if not (DECODE_MODE and SPLIT_K_ENABLED):  # opt-in: measured slower at batch 128 even for the 3-tile router GEMM
        return 1
    nk = K // 64
    if grouped:  # expert tiles already give hundreds of CTAs at batch sizes where the MoE dominates the step
        return 2 if nk >= 32 else 1
    tiles, s = (N + 127) // 128, 1
    while s < 8 and tiles * s * 2 <= 160 and nk // (s * 2) >= 4:
        s *= 2
    return s


# --------------------------------------------------------------------------- tile-packed weights
# A weight streamed once per decode step is best read as long sequential runs. The plain [N, K] layout makes every
# 128-row x 64-column TMA box 128 separate 128-byte pieces, K * 2 bytes apart; packed, the box of one (weight tile,
# k-block) is one contiguous 16 KB run and a tile's k-blocks follow each other, so a CTA streams 128 * K * 2
# sequential bytes. Packing is a permutation done once after loading / sharding; a packed tensor keeps its shape
# (rows padded to a multiple of 128) but only the GEMM launchers of this module can read it.
# The mark lives on the tensor object (``w.b200_packed`` = "plain": one tile per box | "gate_up": gate and up tiles back
# to back), so it cannot outlive the tensor; a view or a copy of a packed tensor is not recognised and must not be made.


def is_packed(w: torch.Tensor) -> int:
    return 1 if getattr(w, "b200_packed", None) else 0


def pack_weight(w: torch.Tensor, gate_up: bool = False) -> torch.Tensor:
    """Tile-pack ``w [..., N, K]`` (``gate_up``: ``[..., 2I, K]`` with the gate rows first) and return the packed
    tensor: the same storage when ``N`` is a multiple of 128, otherwise a new tensor with zero rows appended.
    Tensors whose ``K`` is not a multiple of 64 (or ``I`` of 128) are returned unchanged and stay plain."""
    if w.device.type != "cuda" or w.dtype != torch.bfloat16 or is_packed(w):
        return w
    *lead, N, K = w.shape
    if K % 64 or (gate_up and (N // 2) % 128):
        return w
    if not w.is_contiguous():
        w = w.contiguous()
    E = 1
    for d in lead:
        E *= d
    if gate_up:
        I_ = N // 2
        src = w.view(E, 2, I_ // 128, 128, K // 64, 64).permute(0, 2, 4, 1, 3, 5)
    else:
        Np = (N + 127) // 128 * 128
        if Np != N:
            padded = torch.zeros(*lead, Np, K, dtype=w.dtype, device=w.device)
            padded[..., :N, :] = w
            w, N = padded, Np
        src = w.view(E, N // 128, 128, K // 64, 64).permute(0, 1, 3, 2, 4)
    flat = w.view(-1)
    # expert by expert, so that the temporary stays small next to a 60 GB expert stack
    per = flat.numel() // E
    for e in range(E):
        flat[e * per:(e + 1) * per].copy_(src[e].contiguous().view(-1))
    w.b200_packed = "gate_up" if gate_up else "plain"
    return w


def pack_weights(weights) -> None:
    """Tile-pack every GEMM weight of one device's ``Weights`` in place (fields are replaced where rows had to be
    padded). Call once, after sharding; the torch oracle and the tensor-parallel launchers cannot read packed
    tensors, so this is for the single-GPU and data-/expert-parallel engines."""
    def layer(lw) -> None:
        lw.in_proj = pack_weight(lw.in_proj)
        lw.out_proj = pack_weight(lw.out_proj)
        if lw.router is not None:
            lw.router = pack_weight(lw.router)
        if lw.w_gate_up is not None:
            lw.w_gate_up = pack_weight(lw.w_gate_up, gate_up=True)
            lw.w_down = pack_weight(lw.w_down)

    for lw in weights.layers:
        layer(lw)
    if weights.lm_head.data_ptr() != weights.embed.data_ptr():
        weights.lm_head = pack_weight(weights.lm_head)
    if weights.mtp is not None:
        weights.mtp.fc = pack_weight(weights.mtp.fc)
        layer(weights.mtp.layer)


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None, bt: int = 0) -> torch.Tensor:
    """``x [T, K] @ w[N, K].T`` on tcgen05; bf16 in, bf16 (default) or fp32 out."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    T, K = x.shape
    N = w.shape[0]
    f32 = out_dtype == torch.float32
    if T == 0:
        return torch.empty(T, N, dtype=torch.float32 if f32 else torch.bfloat16, device=x.device)
    assert x.stride(1) == 1 and w.stride(1) == 1 and K % 8 == 0
    out = torch.empty(T, N, dtype=torch.float32 if f32 else torch.bfloat16, device=x.device)
    if bt == 0 and 16 < T <= 256 and N <= 32 * 128:
        # few weight tiles (out_proj: 16, router: 3): 16-row token tiles put 8x more CTAs on the K loop, which is what
        # a latency-bound decode GEMM needs (measured at 128 rows: out_proj 27.4 -> 21.4 us, router 19.4 -> 13.2 us).
        # The token tile never changes a row's bits: every output element sees the same k order.
        bt = 16
    rc = lib().b200_gemm_dense(
        _ptr(x), _ptr(w), _ptr(out), T, N, K, x.stride(0), w.stride(0), N, EPI_F32 if f32 else EPI_BF16, 0, bt,
        None, None, _ptr(err_word(x.device)), split_k(N, K), is_packed(w), _stream(),
    )
    _check(rc, "gemm_dense")
    return out


def linear_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(x @ Wg.T) * (x @ Wu.T)`` with ``w_gate_up = [Wg; Wu]``, fused in the GEMM epilogue."""
    T, K = x.shape
    inter = w_gate_up.shape[0] // 2
    out = torch.empty(T, inter, dtype=torch.bfloat16, device=x.device)
    rc = lib().b200_gemm_dense(
        _ptr(x), _ptr(w_gate_up), _ptr(out), T, inter, K, x.stride(0), w_gate_up.stride(0), inter, EPI_SILU_MUL,
        inter, 0, None, None, _ptr(err_word(x.device)), split_k(inter, K), 0, _stream(),
    )
    _check(rc, "gemm_dense(silu_mul)")
    return out


def lm_head_argmax(x: torch.Tensor, w: torch.Tensor, return_value: bool = False, out: torch.Tensor | None = None):
    """Greedy token per row: LM-head GEMM with per-tile argmax partials, then one reduce. Ties to the lower id.
    ``out`` (int64 ``[T]``, contiguous) receives the picks in place of a new tensor."""
    T, K = x.shape
    V = w.shape[0]
    n_tiles = (V + 127) // 128
    pmax = torch.empty(n_tiles, T, dtype=torch.float32, device=x.device)
    pidx = torch.empty(n_tiles, T, dtype=torch.int32, device=x.device)
    if out is None:
        out = torch.empty(T, dtype=torch.int64, device=x.device)
    assert out.dtype == torch.int64 and out.is_contiguous() and out.numel() == T
    val = torch.empty(T, dtype=torch.float32, device=x.device) if return_value else None
    rc = lib().b200_gemm_dense(
        _ptr(x), _ptr(w), None, T, V, K, x.stride(0), w.stride(0), 0, EPI_ARGMAX, 0, 0, _ptr(pmax), _ptr(pidx),
        _ptr(err_word(x.device)), 1, is_packed(w), _stream(),
    )
    _check(rc, "gemm_dense(argmax)")
    _check(lib().b200_argmax_finish(_ptr(pmax), _ptr(pidx), n_tiles, T, _ptr(out), _ptr(val), _stream()), "argmax_finish")
    return (out, val) if return_value else out


def ivf_pick(hidden: torch.Tensor, lm_head: torch.Tensor, probes: torch.Tensor, offsets: torch.Tensor,
             order: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Best LM-head row of every row of ``hidden`` among the members of its probed clusters (``spec/ivf.py``):
    gathered GEMV over the plain or tile-packed head, then the argmax reduce of the LM head."""
    R, H = hidden.shape
    P = probes.shape[1]
    dev = hidden.device
    assert probes.dtype == torch.int32 and probes.is_contiguous() and hidden.stride(1) == 1
    pmax = torch.empty(P, R, dtype=torch.float32, device=dev)
    pidx = torch.empty(P, R, dtype=torch.int32, device=dev)
    if out is None:
        out = torch.empty(R, dtype=torch.int64, device=dev)
    assert out.dtype == torch.int64 and out.is_contiguous() and out.numel() == R
    rc = lib().b200_ivf_pick(_ptr(hidden), hidden.stride(0), _ptr(lm_head), lm_head.stride(0), is_packed(lm_head), H,
                             _ptr(probes), P, _ptr(offsets), _ptr(order), offsets.numel() - 1, order.numel(),
                             _ptr(pmax), _ptr(pidx), R, _ptr(err_word(dev)), _stream())
    _check(rc, "ivf_pick")
    _check(lib().b200_argmax_finish(_ptr(pmax), _ptr(pidx), P, R, _ptr(out), None, _stream()), "argmax_finish")
    return out


# --------------------------------------------------------------------------- norms
def add_rmsnorm(x: torch.Tensor, res: torch.Tensor | None, w: torch.Tensor, eps: float):
    T, H = x.shape
    y = torch.empty_like(x)
    new = torch.empty_like(x) if res is not None else x
    rc = lib().b200_add_rmsnorm(
        _ptr(x), _ptr(res), _ptr(w), _ptr(new) if res is not None else None, _ptr(y), T, H, eps, 1, _stream()
    )
    _check(rc, "add_rmsnorm")
    return new, y


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    return add_rmsnorm(x2, None, w, eps)[1].view(shape)


def mtp_in(tokens: torch.Tensor, embed_table: torch.Tensor, hidden: torch.Tensor, w_e: torch.Tensor, w_h: torch.Tensor,
           eps: float) -> torch.Tensor:
    """``[rmsnorm(embed[tokens]) | rmsnorm(hidden)]`` (zero-centred norms), the MTP block's ``fc`` input, one launch."""
    T, H = hidden.shape
    out = torch.empty(T, 2 * H, dtype=hidden.dtype, device=hidden.device)
    _check(lib().b200_mtp_in(_ptr(tokens), _ptr(embed_table), _ptr(hidden), _ptr(w_e), _ptr(w_h), _ptr(out), T, H,
                             embed_table.shape[0], eps, _stream()), "mtp_in")
    return out


def chain_accept(tokens: torch.Tensor, picks: torch.Tensor, n_valid: torch.Tensor, positions: torch.Tensor,
                 y: torch.Tensor, G: int, links: int, acc_out: torch.Tensor | None = None):
    """Greedy chain acceptance of a verify pass (``G`` rows per sequence) in one launch: accepted draft count per
    sequence, the MTP hidden row of the last accepted position, and the positions of ``links`` further chain links."""
    B = tokens.numel() // G
    H = y.shape[1]
    dev = y.device
    acc = acc_out if acc_out is not None else torch.empty(B, dtype=torch.int64, device=dev)
    h_sel = torch.empty(B, H, dtype=y.dtype, device=dev)
    link_pos = torch.empty(max(links, 1), B, dtype=torch.int64, device=dev)
    _check(lib().b200_chain_accept(_ptr(tokens), _ptr(picks), _ptr(n_valid), _ptr(positions), _ptr(y), B, G, H, links,
                                   _ptr(acc), _ptr(h_sel), _ptr(link_pos), _stream()), "chain_accept")
    return acc, h_sel, link_pos


def embed(tokens: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    T = tokens.shape[0]
    out = torch.empty(T, table.shape[1], dtype=table.dtype, device=table.device)
    _check(lib().b200_embed(_ptr(tokens), _ptr(table), _ptr(out), T, table.shape[1], table.shape[0], _stream()), "embed")
    return out


# --------------------------------------------------------------------------- MoE
_MOE_BT_FIXED = int(__import__("os").environ.get("ENGINE_MOE_BT", "0"))


def moe_bt(T: int, pairs_per_row: int, n_experts: int) -> int:
    """Token-tile width of the grouped GEMMs from the expected rows per routed expert (``ENGINE_MOE_BT`` fixes it)."""
    if _MOE_BT_FIXED:
        return _MOE_BT_FIXED
    per = T * max(1, pairs_per_row - 1) / max(1, n_experts)
    for bt in (16, 32, 64):
        if per <= bt:
            return bt
    # many rows per expert (prefill): 64-row tiles waste less on each expert's last tile than 128-row ones and run two
    # CTAs per SM (measured at 8192 rows, ~256 per expert: 970 us for the block against 1002 us with 128-row tiles)
    return 64


# widest token tile whose rows the gate/up GEMM fetches by index (0 turns the in-GEMM row gather off). 64 covers the
# prefill tiles too: no expert-sorted copy of x at any size (8 x 1024 tokens, 4 layers: 7.52 -> 7.29 ms per pass)
GATHER_MAX_BT = int(__import__("os").environ.get("ENGINE_MOE_GATHER_BT", "64"))
FUSED_MOE_NORM = True  # Model._moe_norm: combine + residual add + next RMSNorm as one kernel
ROUTE_PLAN_SPLIT = __import__("os").environ.get("ENGINE_ROUTE_PLAN_SPLIT", "0") == "1"  # routing and plan as two launches
ROUTE_PLAN_MAX_ROWS = 32  # up to one row per warp of a single CTA, routing and the expert plan run as one launch
# (measured at 128 rows: 30 us in one CTA against 5 + 3 us as a grid of warps followed by the plan CTA)


def moe_block(x: torch.Tensor, router: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, n_experts: int,
              top_k: int, shared_merged: bool, expert_map: torch.Tensor | None = None,
              partial_f32: bool = False, logits: torch.Tensor | None = None, residual: torch.Tensor | None = None,
              norm_w: torch.Tensor | None = None, eps: float = 1e-6):
    """Router GEMM, top-k, expert-sorted grouped gate/up + SiLU-mul, grouped down, weighted combine.

    With ``expert_map`` (global expert id -> local slot or -1) only the pairs of locally hosted experts
    are computed; ``partial_f32`` returns the fp32 partial sum that the caller adds across ranks. ``logits``
    (fp32 ``[T, rows of router]``) skips the router GEMM when the caller has already run it. With ``norm_w`` the
    combine kernel also adds ``residual`` and applies the next RMSNorm, and the call returns
    ``(new residual, normed)`` exactly as ``add_rmsnorm(moe_out, residual, norm_w, eps)`` would (reference:
    the fused down + combine + residual kernel, ``engine/fast/fused.py:635-692``)."""
    T, H = x.shape
    dev = x.device
    Et = w_gate_up.shape[0]
    inter = w_down.shape[2]
    Pn = top_k + (1 if shared_merged else 0)
    n_pairs = T * Pn
    L = lib()
    st = _stream()
    err = err_word(dev)
    if logits is None:
        logits = linear(x, router, out_dtype=torch.float32)
    wts = torch.empty(T, Pn, dtype=torch.float32, device=dev)
    idx = torch.empty(T, Pn, dtype=torch.int32, device=dev)
    ints = torch.empty(Et + 2 + 3 * n_pairs, dtype=torch.int32, device=dev)
    offsets, n_tiles = ints[: Et + 1], ints[Et + 1 : Et + 2]
    perm, inv = ints[Et + 2 : Et + 2 + n_pairs], ints[Et + 2 + n_pairs : Et + 2 + 2 * n_pairs]
    bt = moe_bt(T, Pn, n_experts)
    # the gate/up GEMM fetches each activation row by index, so no expert-sorted copy of x is made
    gather = bt <= GATHER_MAX_BT and x.stride(0) % 8 == 0 and x.stride(1) == 1
    src_rows = ints[Et + 2 + 2 * n_pairs :] if gather else None
    max_tiles = min(Et, n_pairs) + n_pairs // bt + 1
    tiles = torch.empty(max_tiles, 4, dtype=torch.int32, device=dev)
    if ROUTE_PLAN_SPLIT and T > ROUTE_PLAN_MAX_ROWS:
        _check(L.b200_moe_route(_ptr(logits), logits.stride(0), T, n_experts, top_k, int(shared_merged), _ptr(wts),
                                _ptr(idx), None, 0, _ptr(expert_map), st), "moe_route")
        _check(L.b200_moe_plan(_ptr(idx), n_pairs, Et, bt, _ptr(offsets), _ptr(tiles), _ptr(n_tiles), max_tiles,
                               _ptr(perm), _ptr(inv), _ptr(err), Pn, _ptr(src_rows), st), "moe_plan")
    else:
        # routing and plan in one launch: up to 32 rows in a single CTA, more as a grid whose last CTA builds the plan
        _check(L.b200_moe_route_plan(_ptr(logits), logits.stride(0), T, n_experts, top_k, int(shared_merged),
                                     _ptr(wts), _ptr(idx), _ptr(expert_map), Et, bt, _ptr(offsets), _ptr(tiles),
                                     _ptr(n_tiles), max_tiles, _ptr(perm), _ptr(inv), _ptr(err), _ptr(src_rows),
                                     _ptr(_ticket(dev)), st), "moe_route_plan")
    act = torch.empty(n_pairs, inter, dtype=x.dtype, device=dev)
    if gather:
        _check(L.b200_gemm_grouped(_ptr(x), _ptr(w_gate_up), _ptr(act), n_pairs, Et, inter, 2 * inter, H, inter,
                                   EPI_SILU_MUL, inter, bt, _ptr(tiles), _ptr(n_tiles), max_tiles, _ptr(err), 1,
                                   is_packed(w_gate_up), _ptr(src_rows), x.stride(0), st), "gemm_grouped(gate_up, gather)")
    else:
        xs = torch.empty(n_pairs, H, dtype=x.dtype, device=dev)
        _check(L.b200_moe_gather(_ptr(x), _ptr(perm), _ptr(offsets[Et:]), n_pairs, T, Pn, H, _ptr(xs), st), "moe_gather")
        _check(L.b200_gemm_grouped(_ptr(xs), _ptr(w_gate_up), _ptr(act), n_pairs, Et, inter, 2 * inter, H, inter,
                                   EPI_SILU_MUL, inter, bt, _ptr(tiles), _ptr(n_tiles), max_tiles, _ptr(err),
                                   split_k(inter, H, grouped=True), is_packed(w_gate_up), None, 0, st),
               "gemm_grouped(gate_up)")
    pair_out = torch.empty(n_pairs, H, dtype=x.dtype, device=dev)
    _check(L.b200_gemm_grouped(_ptr(act), _ptr(w_down), _ptr(pair_out), n_pairs, Et, H, H, inter, H, EPI_BF16, 0, bt,
                               _ptr(tiles), _ptr(n_tiles), max_tiles, _ptr(err), split_k(H, inter, grouped=True),
                               is_packed(w_down), None, 0, st),
           "gemm_grouped(down)")
    if norm_w is not None and not partial_f32:
        new_res = torch.empty(T, H, dtype=x.dtype, device=dev)
        y = torch.empty(T, H, dtype=x.dtype, device=dev)
        _check(L.b200_moe_combine_norm(_ptr(pair_out), _ptr(wts), _ptr(inv), T, Pn, H, _ptr(residual), _ptr(norm_w),
                                       _ptr(new_res), _ptr(y), eps, st), "moe_combine_norm")
        return new_res, y
    out = torch.empty(T, H, dtype=torch.float32 if partial_f32 else x.dtype, device=dev)
    _check(L.b200_moe_combine(_ptr(pair_out), _ptr(wts), _ptr(inv), T, Pn, H, None if partial_f32 else _ptr(out),
                              _ptr(out) if partial_f32 else None, st), "moe_combine")
    return out


# --------------------------------------------------------------------------- GDN
def gdn_decode(mixed, slots, conv_state, rec_state, conv_w, A_log, dt_bias, gnorm_w, n_k, n_v, dk, dv, eps,
               G: int = 1, ring=None) -> torch.Tensor:
    """Conv step + delta rule + gated norm for ``B*G`` rows (``G`` consecutive rows per slot)."""
    rows = mixed.shape[0]
    B = rows // G
    C = 2 * n_k * dk + n_v * dv
    conv_out = torch.empty(rows, C, dtype=mixed.dtype, device=mixed.device)
    out = torch.empty(rows, n_v * dv, dtype=mixed.dtype, device=mixed.device)
    slots32 = slots if slots.dtype == torch.int32 else slots.to(torch.int32)
    rc = lib().b200_gdn_decode(
        _ptr(mixed), mixed.stride(0), _ptr(slots32), _ptr(conv_state), _ptr(rec_state), _ptr(conv_w), _ptr(A_log),
        _ptr(dt_bias), _ptr(gnorm_w), _ptr(conv_out), _ptr(out), _ptr(ring[0]) if ring else None,
        _ptr(ring[1]) if ring else None, B, G, n_k, n_v, dk, dv, conv_w.shape[1], eps, _ptr(err_word(mixed.device)),
        _stream(),
    )
    _check(rc, "gdn_decode")
    return out


def ring_commit(conv_state, rec_state, ring, slots: torch.Tensor, keep_rows: torch.Tensor) -> None:
    """Slot state <- state after row ``keep_rows[b]`` of a verify pass, all GDN layers in one launch; sequences that
    keep every row are skipped (the step kernel already left that state in the slot)."""
    ring_conv, ring_rec = ring
    layers, G = ring_rec.shape[0], ring_rec.shape[2]
    assert ring_rec.is_contiguous() and ring_conv.is_contiguous() and slots.shape[0] <= ring_rec.shape[1]
    conv_bytes = conv_state[0, 0].numel() * conv_state.element_size()
    rec_bytes = rec_state[0, 0].numel() * rec_state.element_size()
    slots32 = slots if slots.dtype == torch.int32 else slots.to(torch.int32)
    keep64 = keep_rows if keep_rows.dtype == torch.int64 else keep_rows.to(torch.int64)
    rc = lib().b200_ring_commit(_ptr(conv_state), _ptr(rec_state), _ptr(ring_conv), _ptr(ring_rec), _ptr(slots32),
                                _ptr(keep64), layers, ring_rec.shape[1], slots.shape[0], G, conv_state.shape[1], conv_bytes, rec_bytes,
                                _stream())
    _check(rc, "ring_commit")


_meta_memo: dict = {}  # the span tables of the pass being run: every layer of a pass asks for the same ones


def _memo(key, make):
    """Single-entry memo per kind of table: the 40 layers of a prefill pass share one host build and one copy."""
    hit = _meta_memo.get(key[0])
    if hit is not None and hit[0] == key:
        return hit[1]
    val = make()
    _meta_memo[key[0]] = (key, val)
    return val


def _gdn_prefill_meta(seg_starts, seg_slots, T: int, dev):
    def make():
        nseg = len(seg_slots)
        chunks, seg_chunks, seq_of_row = [], [], []
        for i in range(nseg):
            a, b = seg_starts[i], seg_starts[i + 1]
            first = len(chunks)
            for r0 in range(a, b, 64):
                chunks.append((i, r0, min(64, b - r0), int(r0 == a)))
            seg_chunks.append((first, len(chunks) - first))
            seq_of_row.extend([i] * (b - a))
        meta = torch.tensor([c for ch in chunks for c in ch] + [c for sc in seg_chunks for c in sc] + seq_of_row
                            + list(seg_starts) + list(seg_slots), dtype=torch.int32).to(dev, non_blocking=True)
        o = 0
        chunks_t = meta[o : o + 4 * len(chunks)]; o += 4 * len(chunks)
        segc_t = meta[o : o + 2 * nseg]; o += 2 * nseg
        sor_t = meta[o : o + T]; o += T
        start_t = meta[o : o + nseg + 1]; o += nseg + 1
        slots_t = meta[o : o + nseg]
        return len(chunks), chunks_t, segc_t, sor_t, start_t, slots_t

    return _memo(("gdn", tuple(seg_starts), tuple(seg_slots), T, str(dev)), make)


def gdn_prefill(mixed, seg_starts, seg_slots, conv_state, rec_state, conv_w, A_log, dt_bias, gnorm_w, n_k, n_v, dk,
                dv, eps, meta=None) -> torch.Tensor:
    """Chunked prefill of the gated delta rule over packed spans (conv, WY transform, state scan, gated norm).

    ``meta``: the span tables as device tensors that the caller keeps up to date (``PrefillTables.gdn``); the host
    lists are then not read, which lets the call be captured in a CUDA graph."""
    if dk != dv or dk not in (32, 64, 128) or conv_w.shape[1] != 4 or mixed.stride(0) % 8 or (n_k * dk) % 4:
        return torch_ops.gdn_prefill_batched(
            mixed, seg_starts, seg_slots, conv_state, rec_state, conv_w, A_log, dt_bias, gnorm_w, n_k, n_v, dk, dv, eps
        )
    T = mixed.shape[0]
    dev = mixed.device
    if meta is not None:
        nseg, n_chunks, chunks_t, segc_t, sor_t, start_t, slots_t = meta
    else:
        nseg = len(seg_slots)
        n_chunks, chunks_t, segc_t, sor_t, start_t, slots_t = _gdn_prefill_meta(seg_starts, seg_slots, T, dev)
    C = 2 * n_k * dk + n_v * dv
    stride = lib().b200_gdn_prefill_work_stride(dk)
    work = torch.empty(n_chunks * n_v * stride, dtype=torch.float32, device=dev)
    conv_out = torch.empty(T, C, dtype=mixed.dtype, device=dev)
    o_tmp = torch.empty(T, n_v * dv, dtype=mixed.dtype, device=dev)
    out = torch.empty(T, n_v * dv, dtype=mixed.dtype, device=dev)
    rc = lib().b200_gdn_prefill(
        _ptr(mixed), mixed.stride(0), _ptr(sor_t), _ptr(start_t), _ptr(slots_t), _ptr(conv_state), _ptr(rec_state),
        _ptr(conv_w), _ptr(A_log), _ptr(dt_bias), _ptr(gnorm_w), _ptr(conv_out), _ptr(chunks_t), n_chunks,
        _ptr(segc_t), nseg, _ptr(work), _ptr(o_tmp), _ptr(out), T, n_k, n_v, dk, dv, eps, int(GDN_PREFILL_TC),
        _ptr(err_word(dev)), _stream(),
    )
    _check(rc, "gdn_prefill")
    return out


# --------------------------------------------------------------------------- attention
def attention(qkv, positions, seq_of_row, block_tables, kv_layer, q_norm, k_norm, n_q, n_kv, head_dim, rotary_dim,
              theta, eps, G: int, seg_starts=None, seg_pos0=None, meta=None) -> torch.Tensor:
    """q/k norm + RoPE + KV page write, then gated attention over the paged cache.

    ``G > 0``: every sequence has exactly ``G`` rows (decode ``G = 1``, verify ``G = k + 1``) and the
    flash-decoding kernel runs. ``G = 0``: ragged prefill spans; the page gather + softmax
    runs in PyTorch per sequence after the fused prep kernel.
    """
    rows = qkv.shape[0]
    dev = qkv.device
    q = torch.empty(rows, n_q, head_dim, dtype=qkv.dtype, device=dev)
    gate = torch.empty(rows, n_q * head_dim, dtype=qkv.dtype, device=dev)
    num_pages = kv_layer.shape[0]
    rc = lib().b200_attn_prep(
        _ptr(qkv), qkv.stride(0), _ptr(positions), _ptr(block_tables), block_tables.stride(0), _ptr(seq_of_row),
        _ptr(q_norm), _ptr(k_norm), _ptr(q), _ptr(gate), _ptr(kv_layer), rows, n_q, n_kv, head_dim, rotary_dim,
        theta, eps, num_pages, _ptr(err_word(dev)), _stream(),
    )
    _check(rc, "attn_prep")
    if G == 0:
        group = n_q // n_kv
        if head_dim in (64, 128, 256) and group in (1, 2, 4, 8):
            return flash_prefill(q, gate, kv_layer, block_tables, seg_starts, seg_pos0, meta=meta)
        return torch_ops.paged_attention(q, gate, kv_layer, block_tables, seg_starts, seg_pos0)
    B = rows // G
    if head_dim in (64, 128, 256) and (n_q // n_kv) in (1, 2, 4, 8):
        return flash_decode(q, gate, kv_layer, block_tables, positions, G)
    part_acc = torch.empty(rows, n_q, ATTN_Z, head_dim, dtype=torch.float32, device=dev)
    part_ml = torch.empty(rows, n_q, ATTN_Z, 2, dtype=torch.float32, device=dev)
    out = torch.empty(rows, n_q * head_dim, dtype=qkv.dtype, device=dev)
    rc = lib().b200_paged_attn(
        _ptr(q), _ptr(gate), _ptr(kv_layer), _ptr(block_tables), block_tables.stride(0), _ptr(positions),
        _ptr(part_acc), _ptr(part_ml), _ptr(out), B, G, n_q, n_kv, head_dim, ATTN_Z, num_pages, _stream(),
    )
    _check(rc, "paged_attn")
    return out


def flash_prefill(q: torch.Tensor, gate: torch.Tensor, kv_layer: torch.Tensor, block_tables: torch.Tensor,
                  seg_starts: list[int], seg_pos0: list[int], meta=None) -> torch.Tensor:
    """Causal gated attention of ragged prefill spans over the paged cache (tcgen05 flash kernel).

    ``q [T, n_q, D]`` normed and rotated; the spans' K/V are already in their pages. ``meta``: ``(rows per tile,
    n_tiles, tiles [n_tiles, 4], pos0 [nseg])`` kept on the device by the caller (``PrefillTables.flash``; entries
    with a span length of 0 are fillers that their CTAs skip); the host lists are then not read."""
    T, n_q, D = q.shape
    n_kv = kv_layer.shape[2]
    R = 128 // (n_q // n_kv)
    dev = q.device

    def make():
        tiles = []
        for i in range(len(seg_starts) - 1):
            n = seg_starts[i + 1] - seg_starts[i]
            tiles.extend((i, p0, seg_starts[i], n) for p0 in range(0, n, R))
        return (len(tiles), torch.tensor(tiles, dtype=torch.int32).reshape(-1, 4).to(dev, non_blocking=True),
                torch.tensor(seg_pos0, dtype=torch.int32).to(dev, non_blocking=True))

    if meta is not None:
        r_meta, n_tiles, tiles_t, pos0_t = meta
        if r_meta != R:
            raise ValueError(f"flash_prefill: the tile table was built for {r_meta} positions per tile, the kernel takes {R}")
    else:
        n_tiles, tiles_t, pos0_t = _memo(("flash", tuple(seg_starts), tuple(seg_pos0), R, str(dev)), make)
    out = torch.empty(T, n_q * D, dtype=q.dtype, device=dev)
    rc = lib().b200_flash_prefill(
        _ptr(q), _ptr(gate), _ptr(kv_layer), _ptr(out), _ptr(tiles_t), n_tiles, _ptr(pos0_t), _ptr(block_tables),
        block_tables.stride(0), kv_layer.shape[0], T, n_q, n_kv, D, 0, 1, None, None, 0, _ptr(err_word(dev)), _stream(),
    )
    _check(rc, "flash_prefill")
    return out


DECODE_ATTN_SMALL_TILES = __import__("os").environ.get("ENGINE_ATTN_DECODE_FORM", "1") == "1"  # 8-row Q / P atoms, 3 K/V stages
SPLIT_PAGES = int(__import__("os").environ.get("ENGINE_ATTN_SPLIT_PAGES", "8"))  # pages (64 tokens each) of context per decode-attention CTA: fixed for a server's lifetime, part of the numerics contract
_decode_tiles: dict = {}


def flash_decode(q: torch.Tensor, gate: torch.Tensor, kv_layer: torch.Tensor, block_tables: torch.Tensor,
                 positions: torch.Tensor, G: int) -> torch.Tensor:
    """Decode / verify attention (``G`` rows per sequence) on the tcgen05 flash kernel with split context.

    Each sequence is one query tile (its ``G`` positions x the GQA group fill the first rows of the 128-row
    MMA tile); the context is cut into runs of ``SPLIT_PAGES`` pages handled by separate CTAs whose partial
    results are merged in order. Only device tensors are touched, so the call can be captured in a CUDA graph."""
    rows, n_q, D = q.shape
    n_kv = kv_layer.shape[2]
    B = rows // G
    dev = q.device
    key = (B, G, dev.index)
    if key not in _decode_tiles:
        b = torch.arange(B, dtype=torch.int32)
        _decode_tiles[key] = torch.stack([b, torch.zeros_like(b), b * G, torch.full_like(b, G)], 1).contiguous().to(dev)
    tiles = _decode_tiles[key]
    n_splits = max(1, (block_tables.shape[1] + SPLIT_PAGES - 1) // SPLIT_PAGES)
    pos0 = positions[::G].to(torch.int32)
    part_acc = torch.empty(rows, n_q, n_splits, D, dtype=torch.float32, device=dev)
    part_ml = torch.empty(rows, n_q, n_splits, 2, dtype=torch.float32, device=dev)
    out = torch.empty(rows, n_q * D, dtype=q.dtype, device=dev)
    L = lib()
    rc = L.b200_flash_prefill(
        _ptr(q), _ptr(gate), _ptr(kv_layer), None, _ptr(tiles), B, _ptr(pos0), _ptr(block_tables),
        block_tables.stride(0), kv_layer.shape[0], rows, n_q, n_kv, D, SPLIT_PAGES, n_splits, _ptr(part_acc),
        _ptr(part_ml), 1 if (G == 1 and DECODE_ATTN_SMALL_TILES and n_q // n_kv <= 8) else 0, _ptr(err_word(dev)), _stream(),
    )
    _check(rc, "flash_decode")
    _check(L.b200_attn_combine(_ptr(part_acc), _ptr(part_ml), _ptr(gate), _ptr(out), rows, n_q, D, n_splits, _stream()),
           "attn_combine")
    return out


def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    return torch.argmax(logits, dim=-1)


__all__ = [n for n in dir() if not n.startswith("_")]
