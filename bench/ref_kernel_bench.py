"""Same-box per-kernel baseline: the reference's own Triton kernels, unmodified, at the shapes of kernel_bench.py.

    python bench/ref_kernel_bench.py [case ...]

The reference engine cannot be served on this image (its load path needs a package that is not installed), but its
kernel wrappers take plain tensors. This script imports them from ``baseline/_ref/engine/fast`` exactly as they are
(`engine/fast/mfma.py:321-352`, `engine/fast/kernels.py:449-497, 697-713`, `engine/fast/flash_prefill.py:241-289`,
`engine/fast/moe_prefill.py:546-582`, `engine/fast/gdn_chunk.py:737-786`), builds inputs of the same shapes as
``bench/kernel_bench.py`` and times them the same way (CUDA events, warm-up, a 256 MB L2 flush between timed
launches). One JSON line per case: microseconds and achieved GB/s / TFLOP/s, or the exception that stopped the case
from launching on CUDA. Nothing of this repository's kernels is on the timed path.
"""

from __future__ import annotations

import argparse
import json
import sys
import traceback
import types
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"
sys.path.insert(0, str(REF))


def peaks() -> tuple[float, float, str]:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        p = json.loads(f.read_text())
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


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
    return total / iters * 1e3


def report(name, us, nbytes, flops, **extra):
    hbm, tf, kind = peaks()
    gbs, tfl = nbytes / us / 1e3, flops / us / 1e6
    print(json.dumps({"impl": "reference", "case": name, "us": round(us, 2), "bytes": nbytes, "flops": flops,
                      "GBps": round(gbs, 1), "TFLOPs": round(tfl, 2), f"frac_of_{kind}_hbm": round(gbs / hbm, 3),
                      f"frac_of_{kind}_bf16": round(tfl / tf, 3), **extra}), flush=True)


# --------------------------------------------------------------------------- cases
def case_gemm_decode():
    """engine.fast.mfma.gemv: the served decode GEMV, 16 rows per launch (128 rows = 8 launches, as the engine does)."""
    from engine.fast import mfma

    for name, N, K in (("in_proj", 12352, 2048), ("out_proj", 2048, 4096), ("lm_head", 248320, 2048)):
        w = bf(N, K, scale=0.02)
        for rows in (1, 16, 128):
            x = bf(rows, K)
            us = timed(lambda: mfma.gemv(x, w), iters=5 if N > 100000 else 10)
            report(f"gemv_{name}_rows{rows}", us, w.numel() * 2, 2 * rows * N * K)


def case_attn_decode():
    """engine.fast.kernels.paged_decode_attention: 128 sequences, 1024-token context, 16 Q / 2 KV heads, D = 256."""
    from engine.fast import kernels

    B, ctx, n_q, n_kv, D = 128, 1024, 16, 2, 256
    pages_per = ctx // 64 + 1
    k_pool, v_pool = bf(B * pages_per + 1, n_kv, 64, D), bf(B * pages_per + 1, n_kv, 64, D)
    table = torch.zeros(B + 1, pages_per, dtype=torch.int32, device="cuda")
    table[:B] = torch.arange(B * pages_per, dtype=torch.int32, device="cuda").view(B, pages_per) + 1
    q = bf(B, n_q, D)
    slots = torch.arange(B, dtype=torch.int64, device="cuda")
    lengths = torch.full((B,), ctx + 1, dtype=torch.int32, device="cuda")
    us = timed(lambda: kernels.paged_decode_attention(q, k_pool, v_pool, table, slots, lengths, D ** -0.5, use_triton=True))
    report(f"paged_decode_attention_b{B}_ctx{ctx}", us, B * (ctx + 1) * 2 * n_kv * D * 2, 4 * B * n_q * (ctx + 1) * D)


def case_gdn_decode():
    """engine.fast.kernels.gdn_fused_: the Triton recurrent step (the served HIP kernel has no CUDA build)."""
    from engine.fast import kernels

    B, n_k, n_v, dk, dv = 128, 16, 32, 128, 128
    key_dim = n_k * dk
    m = types.SimpleNamespace(
        num_v_heads=n_v, num_k_heads=n_k, head_k_dim=dk, head_v_dim=dv, key_dim=key_dim,
        A_log=torch.rand(n_v, device="cuda"), dt_bias=torch.randn(n_v, device="cuda"),
        norm=types.SimpleNamespace(weight=bf(dv), variance_epsilon=1e-6))
    state = torch.randn(B + 1, n_v, dk, dv, device="cuda") * 0.1
    slots = torch.arange(B, dtype=torch.int64, device="cuda")
    mixed = bf(B, 2 * key_dim + n_v * dv)
    a, b, z = bf(B, n_v), bf(B, n_v), bf(B, n_v * dv)
    us = timed(lambda: kernels.gdn_fused_(state, slots, mixed, a, b, z, m))
    report(f"gdn_fused_b{B}", us, 2 * B * n_v * dk * dv * 4, 6 * B * n_v * dk * dv)


def case_attn_prefill():
    """engine.fast.flash_prefill.flash_prefill_attention: one sequence, causal, paged KV (1024 and 8192 tokens)."""
    from engine.fast import flash_prefill

    n_q, n_kv, D = 16, 2, 256
    for L in (1024, 8192):
        pp = L // 64 + 1
        k_pool, v_pool = bf(pp + 1, n_kv, 64, D), bf(pp + 1, n_kv, 64, D)
        table = torch.arange(1, pp + 1, dtype=torch.int32, device="cuda")
        q, gate = bf(L, n_q, D), bf(L, n_q * D)
        us = timed(lambda: flash_prefill.flash_prefill_attention(q, k_pool, v_pool, table, 0, gate, D ** -0.5), iters=5)
        report(f"flash_prefill_1x{L}", us, (q.numel() + gate.numel() + L * n_q * D) * 2, 4 * (L * (L + 1) // 2) * n_q * D)


def case_moe_prefill():
    """engine.fast.moe_prefill.moe_prefill: routed experts of a prefill pass (256 experts, top-8), 8192 rows."""
    from engine.fast import moe_prefill

    E, H, I, k = 256, 2048, 512, 8
    wgu, wd = bf(E, 2 * I, H, scale=0.02), bf(E, H, I, scale=0.02)
    for T in (128, 8192):
        x = bf(T, H)
        idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)])
        wts = torch.rand(T, k, device="cuda").to(torch.bfloat16)
        us = timed(lambda: moe_prefill.moe_prefill(x, idx, wts, wgu, wd), iters=5)
        report(f"moe_prefill_T{T}", us, (wgu.numel() + wd.numel()) * 2, 2 * T * k * 3 * H * I)


def case_gdn_prefill():
    """engine.fast.gdn_chunk.chunk: conv + WY transform + state pass of one 1024-token sequence (32 value heads)."""
    from engine.fast import gdn_chunk

    L, n_k, n_v, dk, dv = 1024, 16, 32, 128, 128
    Cd = 2 * n_k * dk + n_v * dv
    qkv = bf(L, Cd)
    conv_state, conv_w = bf(Cd, 4), bf(Cd, 1, 4, scale=0.3)
    a, b = bf(L, n_v), bf(L, n_v)
    a_log, dt_bias = torch.rand(n_v, device="cuda"), torch.randn(n_v, device="cuda")
    state = torch.randn(n_v, dk, dv, device="cuda") * 0.1
    us = timed(lambda: gdn_chunk.chunk(qkv, conv_state, conv_w, a, b, a_log, dt_bias, state, n_k), iters=5)
    flops = (L // 64) * n_v * 2 * (4 * 64 * 64 * 128 + 2 * 64 * 128 * 128 + 64 * 64 * 128 + 128 * 64 * 128)
    report(f"gdn_chunk_1x{L}", us, qkv.numel() * 2 + L * n_v * dv * 2, flops)


CASES = {k[5:]: v for k, v in globals().items() if k.startswith("case_")}

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("cases", nargs="*", default=list(CASES))
    a = ap.parse_args()
    if not (REF / "engine" / "fast").exists():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/engine/fast is absent"}))
        sys.exit(0)
    for name in a.cases:
        try:
            CASES[name]()
        except Exception as e:  # noqa: BLE001 - the failing line is the result for that kernel
            tb = traceback.extract_tb(e.__traceback__)[-1]
            print(json.dumps({"impl": "reference", "case": name, "failed": repr(e)[:300],
                              "at": f"{Path(tb.filename).name}:{tb.lineno}"}), flush=True)
        torch.cuda.synchronize()
