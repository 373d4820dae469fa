"""Fused compute + collective kernels against the library path, device-timed, max over ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench/collective_bench.py [case ...]

Cases (one JSON line each, printed by rank 0):

* ``seq_parallel``: tensor-parallel prefill block at T = 8192 rows: out_proj K-shard GEMM -> reduce-scatter -> residual +
  RMSNorm -> all-gather -> in_proj column-shard GEMM. ``fused`` = the GEMM epilogue stores fp32 tiles into the owner's
  slots over NVLink, the norm kernel pushes rows to every rank, the next GEMM starts per arrived shard
  (``parallel/sp.py``); ``nccl_rs_ag_cublas`` = torch.matmul + NCCL reduce_scatter / all_gather;
  ``gemm_nccl_allreduce`` = this repository's GEMM with an NCCL all-reduce. Roofline of the fused form: the slower of
  its FLOPs at the measured bf16 peak and its NVLink bytes at 770 GB/s per direction.
* ``ep_moe``: one expert-parallel MoE block (dispatch, grouped GEMMs, combine) for 128 rows per rank at the real
  layer shape (256 experts, hidden 2048, expert width 512): ``parallel/ep.py`` against the same block on one GPU.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from b200serve.ops import cuda_ops, torch_ops  # noqa: E402

NVLINK_GBS = 770.0  # measured peer copy per direction on this class of machine


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        p = json.loads(f.read_text())
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def timed(fn, dev, iters=10, warm=3) -> float:
    """Microseconds per call, CUDA events on this rank's stream, max over ranks."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / iters * 1e3], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def case_seq_parallel(rank, world, dev):
    from b200serve.parallel.sp import SeqParallel

    H, eps = 2048, 1e-6
    sp = SeqParallel(dev, dist.group.WORLD, max_rows=8192, hidden=H)
    T, Ks, N2 = 8192, 4096 // world, 12352 // world // 8 * 8
    rpr = T // world
    x = (torch.randn(T, Ks, device=dev) * 0.5).to(torch.bfloat16)
    w_o = (torch.randn(H, Ks, device=dev) * 0.05).to(torch.bfloat16)
    w_n = torch.zeros(H, device=dev, dtype=torch.bfloat16)
    w_i = (torch.randn(N2, H, device=dev) * 0.05).to(torch.bfloat16)
    res = torch.randn(rpr, H, device=dev).to(torch.bfloat16)

    def fused():
        rows = sp.gemm_reduce_scatter(x, w_o)
        return sp.gemm_gathered(sp.reduce_norm_allgather(rows, res, w_n, eps)[1], w_i)

    rs_out = torch.empty(rpr, H, device=dev, dtype=torch.bfloat16)
    ag_out = torch.empty(T, H, device=dev, dtype=torch.bfloat16)

    def library():
        part = x @ w_o.t()
        dist.reduce_scatter_tensor(rs_out, part)
        mine = torch_ops.rmsnorm(rs_out + res, w_n, eps)
        dist.all_gather_into_tensor(ag_out, mine)
        return ag_out @ w_i.t()

    def allreduce_path():
        h = cuda_ops.linear(x, w_o, out_dtype=torch.float32)
        dist.all_reduce(h)
        return cuda_ops.linear(cuda_ops.rmsnorm(h.to(torch.bfloat16), w_n, eps), w_i)

    us = {name: timed(fn, dev) for name, fn in (("fused", fused), ("nccl_rs_ag_cublas", library), ("gemm_nccl_allreduce", allreduce_path))}
    # where the fused pipeline spends its time on rank 0 (events between the three kernels)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(10)]
    torch.cuda.synchronize()
    dist.barrier()
    for it in range(10):
        ev[it][0].record()
        rows = sp.gemm_reduce_scatter(x, w_o)
        ev[it][1].record()
        full = sp.reduce_norm_allgather(rows, res, w_n, eps)[1]
        ev[it][2].record()
        sp.gemm_gathered(full, w_i)
        ev[it][3].record()
    torch.cuda.synchronize()
    stages = [round(sum(ev[it][i].elapsed_time(ev[it][i + 1]) for it in range(10)) * 100, 1) for i in range(3)]
    cuda_ops.check_errors(dev)
    _hbm, tf, kind = peaks()
    flops = 2 * T * H * Ks + 2 * T * N2 * H
    link_bytes = (world - 1) / world * T * H * (4 + 2)  # fp32 partial tiles out, bf16 normed rows out
    roof_us = max(flops / tf / 1e6, link_bytes / NVLINK_GBS / 1e3)
    if rank == 0:
        print(json.dumps({"case": "seq_parallel", "world": world, "T": T, "us": {k: round(v, 1) for k, v in us.items()},
                          "stages_rank0_us": {"gemm_reduce_scatter": stages[0], "reduce_norm_allgather": stages[1],
                                              "gathered_gemm": stages[2]},
                          "flops_per_gpu": flops, "nvlink_bytes_out_per_gpu": int(link_bytes),
                          f"roofline_us_{kind}": round(roof_us, 1), "achieved_over_roofline": round(roof_us / us["fused"], 3),
                          "fused_vs_library": round(us["nccl_rs_ag_cublas"] / us["fused"], 3)}), flush=True)
    dist.barrier()
    sp.close()


def case_ep_moe(rank, world, dev):
    from b200serve.parallel.ep import EpMoE

    E, H, I, k, T = 256, 2048, 512, 8, 128
    g = torch.Generator(device=dev).manual_seed(11)
    router = (torch.randn(E + 1, H, device=dev, generator=g) * 0.3).to(torch.bfloat16)
    per = E // world
    lgu = (torch.randn(per + 1, 2 * I, H, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    ld = (torch.randn(per + 1, H, I, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    lgu, ld = cuda_ops.pack_weight(lgu, gate_up=True), cuda_ops.pack_weight(ld)
    ep = EpMoE(dev, dist.group.WORLD, E, H, k, max_rows=T)
    x = torch.randn(T, H, device=dev).to(torch.bfloat16)
    res = torch.randn(T, H, device=dev).to(torch.bfloat16)
    nw = torch.zeros(H, device=dev, dtype=torch.bfloat16)
    us = timed(lambda: ep.forward(x, router, lgu, ld, residual=res, norm_w=nw), dev, iters=20)
    cuda_ops.check_errors(dev)
    hbm, _tf, kind = peaks()
    w_bytes = (lgu.numel() + ld.numel() + router.numel()) * 2
    link_bytes = (world - 1) / world * T * k * H * 2 * 2  # rows out and expert outputs back, bf16
    roof_us = max(w_bytes / hbm / 1e3, link_bytes / NVLINK_GBS / 1e3)
    if rank == 0:
        print(json.dumps({"case": "ep_moe", "world": world, "rows_per_rank": T, "experts_per_rank": per + 1,
                          "us": round(us, 1), "weight_bytes_per_gpu": w_bytes, "nvlink_bytes_out_per_gpu": int(link_bytes),
                          f"roofline_us_{kind}": round(roof_us, 1), "achieved_over_roofline": round(roof_us / us, 3)}),
              flush=True)
    dist.barrier()
    ep.close()


CASES = {"seq_parallel": case_seq_parallel, "ep_moe": case_ep_moe}

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("cases", nargs="*", default=list(CASES))
    a = ap.parse_args()
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    try:
        for name in a.cases:
            CASES[name](rank, world, dev)
    finally:
        dist.destroy_process_group()
