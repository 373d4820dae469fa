"""Per-kernel timing against the measured roofline.

    python bench/kernel_bench.py [case ...] [--small]

Each case runs one kernel (or one fused op) of the decode / prefill path at the shapes of
Qwen3.6-35B-A3B, timed with CUDA events after warm-up, with an L2 flush (a 256 MB write) between
timed launches, and prints one JSON line: algorithmic bytes and FLOPs, microseconds, achieved
GB/s and TFLOP/s, and the fraction of the measured copy bandwidth / cuBLAS bf16 throughput from
``MEASURED_PEAKS.json`` (fallback 6650 GB/s and 1590 TFLOP/s when the file is absent).
``--small`` shrinks every case to a few hundred MB so that a profiler capture ends quickly.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from b200serve.ops import cuda_ops as C  # noqa: E402


def peaks() -> tuple[float, float, str]:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        p = json.loads(f.read_text())
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


PACK = False  # --packed: tile-pack the GEMM weights first (the layout the serving engine streams)


def pk(w, gate_up=False):
    return C.pack_weight(w, gate_up=gate_up) if PACK else w


_flush = None


def timed(fn, iters=10, warm=3):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        _flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters * 1e3  # microseconds


def report(name, us, nbytes, flops, **extra):
    hbm, tf, kind = peaks()
    gbs, tfl = nbytes / us / 1e3, flops / us / 1e6
    line = {"case": name, "us": round(us, 2), "bytes": nbytes, "flops": flops, "GBps": round(gbs, 1),
            "TFLOPs": round(tfl, 2), f"frac_of_{kind}_hbm": round(gbs / hbm, 3),
            f"frac_of_{kind}_bf16": round(tfl / tf, 3), "packed": PACK, **extra}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- cases
def case_moe_decode(small):
    """MoE block of one decode step: 128 rows, 256 experts top-8 + shared (weight streaming)."""
    T, E, H, I = 128, (64 if small else 256), 2048, 512
    x, router = bf(T, H), pk(bf(E + 1, H, scale=0.3))
    wgu, wd = pk(bf(E + 1, 2 * I, H, scale=0.02), True), pk(bf(E + 1, H, I, scale=0.02))
    us = timed(lambda: C.moe_block(x, router, wgu, wd, E, 8, True))
    w_bytes = (wgu.numel() + wd.numel() + router.numel()) * 2
    report("moe_decode_b128", us, w_bytes, 2 * T * 9 * 3 * H * I, experts=E)


def case_gemm_grouped(small):
    """The two grouped GEMMs alone on a fixed routing (gate/up + SiLU-mul, then down)."""
    T, E, H, I, P = 128, (64 if small else 256), 2048, 512, 9
    wgu, wd = pk(bf(E + 1, 2 * I, H, scale=0.02), True), pk(bf(E + 1, H, I, scale=0.02))
    n_pairs = T * P
    idx = torch.cat([torch.stack([torch.randperm(E, device="cuda")[:8] for _ in range(T)]),
                     torch.full((T, 1), E, device="cuda")], 1).to(torch.int32)
    ints = torch.zeros(E + 3 + 2 * n_pairs, dtype=torch.int32, device="cuda")
    offsets, n_tiles = ints[: E + 2], ints[E + 2 : E + 3]
    perm, inv = ints[E + 3 : E + 3 + n_pairs], ints[E + 3 + n_pairs :]
    bt = 16
    max_tiles = E + 1 + n_pairs // bt + 1
    tiles = torch.empty(max_tiles, 4, dtype=torch.int32, device="cuda")
    L, st = C.lib(), torch.cuda.current_stream().cuda_stream
    err = C.err_word(torch.device("cuda"))
    assert L.b200_moe_plan(idx.data_ptr(), n_pairs, E + 1, bt, offsets.data_ptr(), tiles.data_ptr(), n_tiles.data_ptr(),
                           max_tiles, perm.data_ptr(), inv.data_ptr(), err.data_ptr(), P, None, st) == 0
    xs, act, out = bf(n_pairs, H), torch.empty(n_pairs, I, dtype=torch.bfloat16, device="cuda"), torch.empty(
        n_pairs, H, dtype=torch.bfloat16, device="cuda")

    def up():
        L.b200_gemm_grouped(xs.data_ptr(), wgu.data_ptr(), act.data_ptr(), n_pairs, E + 1, I, 2 * I, H, I, 2, I, bt,
                            tiles.data_ptr(), n_tiles.data_ptr(), max_tiles, err.data_ptr(), 1, C.is_packed(wgu), None, 0, st)

    def down():
        L.b200_gemm_grouped(act.data_ptr(), wd.data_ptr(), out.data_ptr(), n_pairs, E + 1, H, H, I, H, 0, 0, bt,
                            tiles.data_ptr(), n_tiles.data_ptr(), max_tiles, err.data_ptr(), 1, C.is_packed(wd), None, 0, st)

    report("grouped_gate_up_silu", timed(up), wgu.numel() * 2, 2 * n_pairs * 2 * I * H, experts=E)
    report("grouped_down", timed(down), wd.numel() * 2, 2 * n_pairs * I * H, experts=E)


def case_gdn_decode(small):
    """Recurrent Gated-DeltaNet step of one layer: 128 sequences x 32 heads x 64 KB of fp32 state."""
    B = 32 if small else 128
    n_k, n_v, dk, dv = 16, 32, 128, 128
    Cd = 2 * n_k * dk + n_v * dv
    mixed = bf(B, Cd + n_v * dv + 2 * n_v)
    conv, rec = bf(B + 1, Cd, 3), torch.randn(B + 1, n_v, dk, dv, device="cuda") * 0.1
    args = (bf(Cd, 4, scale=0.3), torch.rand(n_v, device="cuda"), torch.randn(n_v, device="cuda"), bf(dv), n_k, n_v, dk, dv, 1e-6)
    slots = torch.arange(1, B + 1, dtype=torch.int32, device="cuda")
    us = timed(lambda: C.gdn_decode(mixed, slots, conv, rec, *args))
    report(f"gdn_decode_b{B}", us, 2 * B * n_v * dk * dv * 4, 6 * B * n_v * dk * dv)


def case_attn_decode(small):
    """Paged decode attention of one layer: 128 sequences, 1024-token context, 16 Q / 2 KV heads, D=256."""
    B, ctx = (32 if small else 128), 1024
    n_q, n_kv, D = 16, 2, 256
    pages_per = ctx // 64 + 1
    kv = bf(B * pages_per + 1, 2, n_kv, 64, D)
    tables = (torch.arange(B * pages_per, dtype=torch.int32, device="cuda").view(B, pages_per) + 1)
    qkv = bf(B, n_q * 2 * D + 2 * n_kv * D)
    pos = torch.full((B,), ctx, dtype=torch.int64, device="cuda")
    seq = torch.arange(B, dtype=torch.int32, device="cuda")
    qn, kn = bf(D, scale=0.1), bf(D, scale=0.1)
    us = timed(lambda: C.attention(qkv, pos, seq, tables, kv, qn, kn, n_q, n_kv, D, 64, 1e7, 1e-6, 1))
    report(f"attn_decode_b{B}_ctx{ctx}", us, B * (ctx + 1) * 2 * n_kv * D * 2, 4 * B * n_q * (ctx + 1) * D)


def case_lm_head(small):
    """LM head with fused argmax: 248320 x 2048 weights, 128 rows."""
    V = 65536 if small else 248320
    x, w = bf(128, 2048), pk(bf(V, 2048, scale=0.02))
    us = timed(lambda: C.lm_head_argmax(x, w))
    report("lm_head_argmax_b128", us, w.numel() * 2, 2 * 128 * V * 2048, vocab=V)


def case_gemm_decode(small):
    """Dense projections at decode size (128 rows): GDN in_proj 12352 x 2048 and out_proj 2048 x 4096."""
    for name, N, K in (("in_proj", 12352, 2048), ("out_proj", 2048, 4096), ("router", 257, 2048)):
        x, w = bf(128, K), pk(bf(N, K, scale=0.02))
        for bt in (0, 16, 32, 64, 128):  # 0: what the engine picks; smaller token tiles = more CTAs streaming the weights
            us = timed(lambda: C.linear(x, w, bt=bt))
            report(f"gemm_decode_{name}_b128", us, w.numel() * 2, 2 * 128 * N * K, bt=bt or "auto")


def case_gemm_decode_splitk(small):
    """Decode-size projections with the K loop split over a thread-block cluster (DSMEM reduction in rank order):
    token tile x split factor sweep, to see where spreading one weight tile over several SMs pays."""
    L, st = C.lib(), torch.cuda.current_stream().cuda_stream
    err = C.err_word(torch.device("cuda"))
    for name, N, K in (("in_proj", 12352, 2048), ("qkv_proj", 9216, 2048), ("out_proj", 2048, 4096)):
        x, w = bf(128, K), bf(N, K, scale=0.02)
        out = torch.empty(128, N, dtype=torch.bfloat16, device="cuda")
        for bt in (16, 32, 64, 128):
            for splits in (1, 2, 4, 8):
                def run():
                    rc = L.b200_gemm_dense(x.data_ptr(), w.data_ptr(), out.data_ptr(), 128, N, K, K, K, N, 0, 0, bt, None,
                                           None, err.data_ptr(), splits, 0, st)
                    assert rc == 0, rc
                report(f"gemm_decode_{name}_b128", timed(run), w.numel() * 2, 2 * 128 * N * K, bt=bt, splits=splits)


def case_gemm_prefill(small):
    """Dense projection at prefill size: 8192 rows x (12352 x 2048), compute bound."""
    T = 2048 if small else 8192
    x, w = bf(T, 2048), bf(12352, 2048, scale=0.02)
    us = timed(lambda: C.linear(x, w), iters=5)
    report(f"gemm_prefill_in_proj_T{T}", us, (w.numel() + x.numel() + T * 12352) * 2, 2 * T * 12352 * 2048)


def case_moe_prefill(small):
    """MoE block at prefill size: 8192 rows (grouped GEMMs with 128-row token tiles)."""
    T, E, H, I = (1024 if small else 8192), (64 if small else 256), 2048, 512
    x, router = bf(T, H), bf(E + 1, H, scale=0.3)
    wgu, wd = bf(E + 1, 2 * I, H, scale=0.02), bf(E + 1, H, I, scale=0.02)
    us = timed(lambda: C.moe_block(x, router, wgu, wd, E, 8, True), iters=5)
    report(f"moe_prefill_T{T}", us, (wgu.numel() + wd.numel()) * 2, 2 * T * 9 * 3 * H * I, experts=E)


def case_gdn_prefill(small):
    """Gated DeltaNet chunked prefill of one layer: 8 sequences x 1024 tokens, 32 value heads of 128 x 128
    (conv + WY transform + state pass + gated norm; tensor-core path unless ENGINE_GDN_TC=0)."""
    nseg, L = (2, 512) if small else (8, 1024)
    n_k, n_v, dk, dv = 16, 32, 128, 128
    Cd = 2 * n_k * dk + n_v * dv
    T = nseg * L
    mixed = bf(T, Cd + n_v * dv + 2 * n_v)
    conv, rec = bf(nseg + 1, Cd, 3), torch.randn(nseg + 1, n_v, dk, dv, device="cuda") * 0.1
    args = (bf(Cd, 4, scale=0.3), torch.rand(n_v, device="cuda"), torch.randn(n_v, device="cuda"), bf(dv), n_k, n_v, dk, dv, 1e-6)
    starts = [i * L for i in range(nseg + 1)]
    slots = list(range(1, nseg + 1))
    us = timed(lambda: C.gdn_prefill(mixed, starts, slots, conv, rec, *args), iters=5)
    # per (chunk, head): K K^T, Q K^T, T k, T v (64x64x128 each, 2 flops/mac), S w, S q, scores v, k^T v
    flops = (T // 64) * n_v * 2 * (4 * 64 * 64 * 128 + 2 * 64 * 128 * 128 + 64 * 64 * 128 + 128 * 64 * 128)
    report(f"gdn_prefill_{nseg}x{L}", us, mixed.numel() * 2 + T * n_v * dv * 2, flops, tensor_cores=C.GDN_PREFILL_TC)


def case_attn_prefill(small):
    """Causal gated flash attention of one prefill pass over the paged KV: one 8192-token sequence (or 8 x 1024 with
    --small), 16 Q / 2 KV heads, D = 256 (prep kernel + flash kernel)."""
    nseg, L = (8, 1024) if small else (1, 8192)
    n_q, n_kv, D = 16, 2, 256
    T = nseg * L
    pp = L // 64 + 1
    kv = bf(nseg * pp + 1, 2, n_kv, 64, D)
    tables = torch.arange(nseg * pp, dtype=torch.int32, device="cuda").view(nseg, pp) + 1
    qkv = bf(T, n_q * 2 * D + 2 * n_kv * D)
    pos = torch.arange(L, dtype=torch.int64, device="cuda").repeat(nseg)
    seq = torch.repeat_interleave(torch.arange(nseg, dtype=torch.int32, device="cuda"), L)
    qn, kn = bf(D, scale=0.1), bf(D, scale=0.1)
    starts = [i * L for i in range(nseg + 1)]
    us = timed(lambda: C.attention(qkv, pos, seq, tables, kv, qn, kn, n_q, n_kv, D, 64, 1e7, 1e-6, 0, starts, [0] * nseg), iters=5)
    flops = 4 * nseg * (L * (L + 1) // 2) * n_q * D
    report(f"attn_prefill_{nseg}x{L}", us, qkv.numel() * 2 + T * n_q * D * 2, flops)


def case_glue(small):
    """Row-wise glue of a decode step at 128 rows: residual add + RMSNorm, embedding gather, the MTP block's input
    kernel and the chain-acceptance kernel of a verify step (4 rows per sequence)."""
    T, H, V = 128, 2048, 248320 if not small else 32768
    x, r, w = bf(T, H), bf(T, H), bf(H, scale=0.1)
    report("add_rmsnorm_b128", timed(lambda: C.add_rmsnorm(x, r, w, 1e-6)), 4 * T * H * 2, 0)
    table = bf(V, H, scale=0.02)
    tok = torch.randint(0, V, (T,), device="cuda")
    report("embed_b128", timed(lambda: C.embed(tok, table)), 2 * T * H * 2, 0)
    report("mtp_in_b128", timed(lambda: C.mtp_in(tok, table, x, w, w, 1e-6)), 4 * T * H * 2, 0)
    G = 4
    picks, toks = torch.randint(0, 9, (T * G,), device="cuda"), torch.randint(0, 9, (T * G,), device="cuda")
    nv = torch.full((T,), G - 1, dtype=torch.int32, device="cuda")
    pos = torch.arange(T * G, device="cuda")
    y = bf(T * G, H)
    report("chain_accept_b128x4", timed(lambda: C.chain_accept(toks, picks, nv, pos, y, G, 2)), 2 * T * H * 2, 0)


def case_allreduce_loopback(small):
    """One-shot push all-reduce of a decode-size message (128 x 2048 bf16) on a one-rank group: the kernel's own
    cost without the NVLink hop (stores into this GPU's receive slot, flag release / wait, rank-order sum)."""
    from b200serve.parallel.symm import SymmComm

    comm = SymmComm(torch.device("cuda"), None, slot_elems=1 << 19, max_blocks=512)
    x, r = bf(128, 2048), bf(128, 2048)
    report("allreduce_push_loopback_128x2048", timed(lambda: comm.allreduce(x, r)), 3 * x.numel() * 2, 0)
    comm.close()


def case_ep_loopback(small):
    """The expert-parallel MoE block on a one-rank group at decode size: send, plan, gathering gate/up GEMM, scatter
    epilogue of the down GEMM, combine + residual + norm (every kernel of the multi-GPU path, peer stores local)."""
    from b200serve.parallel.ep import EpMoE

    T, E, H, I = 128, (64 if small else 256), 2048, 512
    router = pk(bf(E + 1, H, scale=0.3))
    wgu, wd = pk(bf(E + 1, 2 * I, H, scale=0.02), True), pk(bf(E + 1, H, I, scale=0.02))
    ep = EpMoE(torch.device("cuda"), None, E, H, 8, max_rows=T)
    x, r, w = bf(T, H), bf(T, H), bf(H, scale=0.1)
    us = timed(lambda: ep.forward(x, router, wgu, wd, residual=r, norm_w=w))
    report(f"ep_moe_loopback_b{T}", us, (wgu.numel() + wd.numel() + router.numel()) * 2, 2 * T * 9 * 3 * H * I, experts=E)
    ep.close()


def case_draft_ivf(small):
    """Shortlist draft pick (centroid GEMM, top-k, gathered GEMV, reduce) beside the full LM head with fused argmax,
    8 rows, 64 of 4096 clusters probed."""
    from b200serve.spec.ivf import IvfIndex

    V, H, R = (65536 if small else 248320), 2048, 8
    head = bf(V, H, scale=0.02)
    idx = IvfIndex.build(head, n_clusters=1024 if small else 4096, probes=64, iters=2)
    w = pk(head)
    x = bf(R, H)
    report(f"lm_head_argmax_b{R}", timed(lambda: C.lm_head_argmax(x, w)), V * H * 2, 2 * R * V * H)
    cand = int((idx.offsets[1:] - idx.offsets[:-1]).float().mean().item() * 64)
    report(f"draft_ivf_pick_b{R}", timed(lambda: idx.pick(C, x, w)), (idx.centroids.numel() + R * cand * H) * 2,
           2 * R * (idx.n_clusters + cand) * H, clusters=idx.n_clusters, probes=64, candidates_per_row=cand)


CASES = {k[5:]: v for k, v in globals().items() if k.startswith("case_")}

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("cases", nargs="*", default=list(CASES))
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--packed", action="store_true")
    a = ap.parse_args()
    PACK = a.packed
    for name in a.cases:
        CASES[name](a.small)
    C.check_errors(torch.device("cuda"))
