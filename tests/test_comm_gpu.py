"""NVLink collective kernels on one GPU: loopback group, and a wait that runs out cleanly."""

import ctypes
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def test_loopback_allreduce_adds_residual():
    from b200serve.ops import cuda_ops
    from b200serve.parallel.symm import SymmComm

    dev = torch.device("cuda")
    comm = SymmComm(dev, None, slot_elems=1 << 18, max_blocks=64)
    for rep in range(3):  # epochs advance and parities alternate
        x = torch.randn(33, 2048, device=dev).to(torch.bfloat16)
        r = torch.randn(33, 2048, device=dev).to(torch.bfloat16)
        assert torch.equal(comm.allreduce(x, r), x + r)
        xf = torch.randn(5, 512, device=dev)
        assert torch.equal(comm.allreduce(xf, out_dtype=torch.float32), xf)
    cuda_ops.check_errors(dev)
    comm.close()


@pytest.mark.parametrize("T,H", [(33, 2048), (5, 128), (128, 2048), (3, 4096)])
def test_loopback_allreduce_with_residual_and_norm_matches_the_separate_kernels(T, H):
    """All-reduce + residual + next RMSNorm in one launch against all-reduce, then the add + norm kernel."""
    from b200serve.ops import cuda_ops
    from b200serve.parallel.symm import SymmComm

    dev = torch.device("cuda")
    comm = SymmComm(dev, None, slot_elems=1 << 20, max_blocks=256)
    assert comm.norm_fits(T, H)
    for rep in range(3):
        part = torch.randn(T, H, device=dev)  # fp32 partial, as the expert-parallel MoE block produces
        res = torch.randn(T, H, device=dev).to(torch.bfloat16)
        w = (torch.randn(H, device=dev) * 0.1).to(torch.bfloat16)
        want_res, want_y = cuda_ops.add_rmsnorm(comm.allreduce(part), res, w, 1e-6)
        got_res, got_y = comm.allreduce_norm(part, res, w, 1e-6)
        assert torch.equal(got_res, want_res)
        # the sum of squares is added in another order: at most one bf16 step apart
        assert torch.allclose(got_y.float(), want_y.float(), rtol=1e-2, atol=1e-3)
        want_res, want_y = cuda_ops.add_rmsnorm(comm.allreduce(part), None, w, 1e-6)
        got_res, got_y = comm.allreduce_norm(part, None, w, 1e-6)
        assert torch.equal(got_res, want_res) and torch.allclose(got_y.float(), want_y.float(), rtol=1e-2, atol=1e-3)
    cuda_ops.check_errors(dev)
    comm.close()


def test_absent_peer_times_out_with_a_status_and_leaves_the_context_usable():
    """A two-rank context whose second rank never runs: the bounded wait gives up after about a
    second, the kernel records ERR_WAIT_PEER and returns, and later launches still work."""
    from b200serve.ops import cuda_ops
    from b200serve.parallel import symm

    dev = torch.device("cuda")
    comm = symm.SymmComm(dev, None, slot_elems=1 << 16, max_blocks=16)
    # pretend to be rank 0 of 2; "rank 1" is this GPU's own memory, and nothing ever sets its flags
    big = symm.SymmComm(dev, None, slot_elems=1 << 16, max_blocks=16)
    ctx = comm.ctx
    ctx.world = 2
    ctx.recv[1] = big._own["recv"]
    ctx.flags[1] = big._own["flags"]
    # the receive area of a 2-rank group is twice as large: use the second allocation for both
    ctx.recv[0] = big._own["recv"]
    x = torch.ones(4, 1024, device=dev, dtype=torch.bfloat16)
    out = torch.full_like(x, 7.0)
    rc = symm._lib().b200_allreduce_push(ctypes.byref(ctx), x.data_ptr(), 0, None, out.data_ptr(), None, x.numel(),
                                         torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(cuda_ops.err_word(dev).item()) == 4
    with pytest.raises(cuda_ops.KernelError):
        cuda_ops.check_errors(dev)
    assert (out == 7.0).all()  # untouched
    ctx.world = 1
    y = torch.randn(8, 256, device=dev).to(torch.bfloat16)
    a = torch.empty_like(y)
    assert cuda_ops.linear(y, torch.eye(256, device=dev, dtype=torch.bfloat16)).equal(y)
    cuda_ops.check_errors(dev)
    comm.close(); big.close()
    del a


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_rank_allreduce_over_nvlink():
    env = {"NCCL_NVLS_ENABLE": "0"}
    import os

    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29611", str(ROOT / "tests/dist_worker.py"),
                        "allreduce"], capture_output=True, text=True, timeout=600, env={**os.environ, **env})
    assert r.returncode == 0 and "OK allreduce" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_expert_parallel_moe_loopback_matches_the_local_block():
    """One-rank group: dispatch, scatter epilogue and combine run against this GPU's own buffers."""
    from b200serve.ops import cuda_ops
    from b200serve.parallel.ep import EpMoE

    dev = torch.device("cuda")
    E, H, I, k = 16, 256, 128, 2
    g = torch.Generator(device=dev).manual_seed(3)
    router = (torch.randn(E + 1, H, device=dev, generator=g) * 0.3).to(torch.bfloat16)
    wgu = (torch.randn(E + 1, 2 * I, H, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(E + 1, H, I, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    ep = EpMoE(dev, None, E, H, k, max_rows=600)
    lgu, ld = ep.local_experts(wgu, wd)
    nw = (torch.randn(H, device=dev, generator=g) * 0.1).to(torch.bfloat16)
    for T in (1, 50, 200, 600, 3):  # 600 rows: token tiles too wide for the gathering GEMM, rows are compacted first
        x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
        res = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
        got = ep.forward(x, router, lgu, ld)
        ref = cuda_ops.moe_block(x, router, wgu, wd, E, k, True)
        cuda_ops.check_errors(dev)
        assert torch.equal(got, ref), (T, (got.float() - ref.float()).abs().max().item())
        got_res, got_y = ep.forward(x, router, lgu, ld, residual=res, norm_w=nw, eps=1e-6)
        ref_res, ref_y = cuda_ops.add_rmsnorm(ref, res, nw, 1e-6)
        cuda_ops.check_errors(dev)
        assert torch.equal(got_res, ref_res) and torch.equal(got_y, ref_y), T
    ep.close()


def test_expert_parallel_moe_reports_a_full_receive_region():
    """A capacity factor below what a call needs must set the error word, never drop rows silently."""
    from b200serve.ops import cuda_ops
    from b200serve.parallel.ep import EpMoE

    dev = torch.device("cuda")
    E, H, I, k = 16, 256, 128, 2
    g = torch.Generator(device=dev).manual_seed(4)
    router = (torch.randn(E + 1, H, device=dev, generator=g) * 0.3).to(torch.bfloat16)
    wgu = (torch.randn(E + 1, 2 * I, H, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(E + 1, H, I, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    ep = EpMoE(dev, None, E, H, k, max_rows=512, capacity_factor=0.1)
    assert ep.cap_src < 512 * 3
    lgu, ld = ep.local_experts(wgu, wd)
    x = torch.randn(512, H, device=dev, generator=g).to(torch.bfloat16)
    ep.forward(x, router, lgu, ld)
    with pytest.raises(cuda_ops.KernelError):
        cuda_ops.check_errors(dev)
    # the context stays usable for calls that fit
    x = torch.randn(8, H, device=dev, generator=g).to(torch.bfloat16)
    got = ep.forward(x, router, lgu, ld)
    cuda_ops.check_errors(dev)
    assert torch.equal(got, cuda_ops.moe_block(x, router, wgu, wd, E, k, True))
    ep.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_rank_expert_parallel_moe():
    import os

    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29631", str(ROOT / "tests/dist_worker.py"),
                        "ep_moe"], capture_output=True, text=True, timeout=600,
                       env={**os.environ, "NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0 and "OK ep_moe" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_sequence_parallel_kernels_loopback():
    """One-rank group: GEMM -> reduce-scatter, norm + all-gather push and the gathered GEMM against fp32."""
    from b200serve.ops import cuda_ops, torch_ops
    from b200serve.parallel.sp import SeqParallel

    dev = torch.device("cuda")
    H = 512
    sp = SeqParallel(dev, None, max_rows=512, hidden=H)
    g = torch.Generator(device=dev).manual_seed(5)
    for T in (16, 48, 512):
        x = (torch.randn(T, 256, device=dev, generator=g) * 0.5).to(torch.bfloat16)
        w_o = (torch.randn(H, 256, device=dev, generator=g) * 0.05).to(torch.bfloat16)
        res = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
        w_n = (torch.randn(H, device=dev, generator=g) * 0.1).to(torch.bfloat16)
        w_i = (torch.randn(384, H, device=dev, generator=g) * 0.05).to(torch.bfloat16)
        for _ in range(3):
            rows = sp.gemm_reduce_scatter(x, w_o)
            mine, full = sp.reduce_norm_allgather(rows, res, w_n, 1e-6)
            assert torch.equal(sp.norm_allgather(mine, w_n, 1e-6), full)
            y = sp.gemm_gathered(full, w_i)
            torch.cuda.synchronize()
            cuda_ops.check_errors(dev)
            want = ((x.float() @ w_o.float().t()).to(torch.bfloat16).float() + res.float()).to(torch.bfloat16)
            assert (mine.float() - want.float()).abs().max().item() <= 0.02 * want.float().abs().max().item()
            assert (full.float() - torch_ops.rmsnorm(mine, w_n, 1e-6).float()).abs().max().item() < 0.05
            want_y = full.float() @ w_i.float().t()
            assert (y.float() - want_y).abs().max().item() <= 0.02 * want_y.abs().max().item() + 1e-3
    sp.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_rank_sequence_parallel_gemms():
    import os

    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29641", str(ROOT / "tests/dist_worker.py"),
                        "seq_parallel"], capture_output=True, text=True, timeout=600,
                       env={**os.environ, "NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0 and "OK seq_parallel" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_rank_data_parallel_attention_with_expert_parallel_moe():
    import os

    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29651", str(ROOT / "tests/dist_worker.py"),
                        "dp_ep_model"], capture_output=True, text=True, timeout=600,
                       env={**os.environ, "NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0 and "OK dp_ep_model" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def _gemm_allreduce(comm, x, w, residual=None, bt=0):
    """The tensor-parallel output projection (GEMM whose epilogue is the all-reduce) on a symmetric context."""
    from b200serve.ops import cuda_ops
    from b200serve.parallel import symm

    L = symm._lib()
    P, I = ctypes.c_void_p, ctypes.c_int
    L.b200_gemm_allreduce.argtypes = [ctypes.c_void_p, P, P, P, P, I, I, I, I, I, I, P]
    L.b200_gemm_allreduce.restype = I
    T, K = x.shape
    N = w.shape[0]
    out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
    rc = L.b200_gemm_allreduce(ctypes.byref(comm.ctx), x.data_ptr(), w.data_ptr(),
                               None if residual is None else residual.data_ptr(), out.data_ptr(), T, N, K, x.stride(0),
                               w.stride(0), bt, torch.cuda.current_stream().cuda_stream)
    if rc:
        raise cuda_ops.KernelError(f"gemm_allreduce failed with code {rc}")
    return out


@pytest.mark.parametrize("T,N,K", [(1, 256, 128), (33, 2048, 512), (128, 2048, 4096)])
def test_gemm_with_allreduce_epilogue_loopback_against_fp32(T, N, K):
    """One-rank group: the tile goes TMEM -> receive slot -> rank-order sum (+ residual) -> bf16. Checked against the
    fp32 product, and bit for bit against the plain GEMM followed by the same rounding steps."""
    from b200serve.ops import cuda_ops
    from b200serve.parallel.symm import SymmComm

    dev = torch.device("cuda")
    comm = SymmComm(dev, None, slot_elems=1 << 19, max_blocks=512)
    g = torch.Generator(device=dev).manual_seed(T + N)
    w = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    for rep in range(3):  # epochs advance, receive parities alternate
        x = torch.randn(T, K, device=dev, generator=g).to(torch.bfloat16)
        r = torch.randn(T, N, device=dev, generator=g).to(torch.bfloat16)
        ref = x.float() @ w.float().t()
        got = _gemm_allreduce(comm, x, w)
        err = (got.float() - ref).abs().max().item()
        assert err <= 2e-2 * max(1.0, ref.abs().max().item()), (rep, err)
        assert torch.equal(got, cuda_ops.linear(x, w))
        got_r = _gemm_allreduce(comm, x, w, r)
        want_r = (cuda_ops.linear(x, w).float() + r.float()).to(torch.bfloat16)
        assert torch.equal(got_r, want_r)
    cuda_ops.check_errors(dev)
    comm.close()


def test_two_thousand_back_to_back_collectives_never_read_a_stale_slot():
    """Stale-read stress: every call's inputs depend on the call number, every result is checked (on the device, one
    read-back at the end). Covers the push all-reduce, the GEMM + all-reduce epilogue and the expert-parallel block,
    whose flags and receive slots are reused with alternating parity / advancing epochs
    (reference: epoch-dependent fill + check over thousands of calls, tools/tp_bench.py:231-250)."""
    from b200serve.ops import cuda_ops
    from b200serve.parallel.ep import EpMoE
    from b200serve.parallel.symm import SymmComm

    dev = torch.device("cuda")
    comm = SymmComm(dev, None, slot_elems=1 << 16, max_blocks=64)
    g = torch.Generator(device=dev).manual_seed(9)
    base = torch.randn(8, 512, device=dev, generator=g)
    w = (torch.randn(256, 512, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    E, H, I, k = 8, 256, 128, 2
    router = (torch.randn(E + 1, H, device=dev, generator=g) * 0.3).to(torch.bfloat16)
    wgu = (torch.randn(E + 1, 2 * I, H, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(E + 1, H, I, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    ep = EpMoE(dev, None, E, H, k, max_rows=16)
    lgu, ld = ep.local_experts(wgu, wd)
    xe = torch.randn(16, H, device=dev, generator=g)
    bad = torch.zeros(3, dtype=torch.int64, device=dev)
    for i in range(2000):
        x = (base + 0.01 * (i % 97)).to(torch.bfloat16)
        res = (base * 0.5 - 0.02 * (i % 31)).to(torch.bfloat16)
        bad[0] += (comm.allreduce(x, res) != x + res).any()
        want = (cuda_ops.linear(x, w).float() + 0.0).to(torch.bfloat16)
        bad[1] += (_gemm_allreduce(comm, x, w) != want).any()
        if i % 4 == 0:  # the MoE block is a dozen launches: every fourth call keeps the test short
            rows = (xe + 0.01 * (i % 53)).to(torch.bfloat16)[: 1 + i % 16]
            bad[2] += (ep.forward(rows, router, lgu, ld) != cuda_ops.moe_block(rows, router, wgu, wd, E, k, True)).any()
    assert bad.tolist() == [0, 0, 0]
    cuda_ops.check_errors(dev)
    ep.close()
    comm.close()
