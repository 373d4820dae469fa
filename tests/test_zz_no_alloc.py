"""The allocation-free greedy-head entry point, called through its exported C symbol.

Some embedders of the kernel library run inside a fixed device-memory plan and cannot call
``cudaMalloc`` (nor a framework allocator that might): ``b200_lm_head_argmax_noalloc`` keeps its
per-tile partial results in an array inside the library instead of a caller-provided workspace.
This file is collected last on purpose, so a failure here cannot hide another test's result.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ROWS, MAX_TILES, TOO_LARGE = 256, 2048, -20


def _entry():
    from b200serve.ops.build import lib_path

    lib = ctypes.CDLL(str(lib_path()))
    fn = lib.b200_lm_head_argmax_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 5 + [ctypes.c_void_p, ctypes.c_void_p]
    return fn


def _call(fn, x, w, err):
    T, K = x.shape
    idx = torch.full((T,), -1, dtype=torch.int64, device=x.device)
    val = torch.full((T,), float("nan"), dtype=torch.float32, device=x.device)
    rc = fn(x.data_ptr(), w.data_ptr(), idx.data_ptr(), val.data_ptr(), T, w.shape[0], K, x.stride(0), w.stride(0),
            err.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return rc, idx, val


def test_noalloc_matches_workspace_entry_point_twice_in_a_row():
    from b200serve.ops import cuda_ops

    fn = _entry()
    dev = torch.device("cuda")
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    g = torch.Generator(device=dev).manual_seed(5)
    # two different problems back to back: the second must not see anything of the first
    for T, V, K in ((37, 20000, 256), (200, 5000, 512)):
        x = torch.randn(T, K, device=dev, generator=g).to(torch.bfloat16)
        w = torch.randn(V, K, device=dev, generator=g).to(torch.bfloat16)
        rc, idx, val = _call(fn, x, w, err)
        assert rc == 0
        ref_idx, ref_val = cuda_ops.lm_head_argmax(x, w, return_value=True)
        torch.cuda.synchronize()
        assert torch.equal(idx, ref_idx)
        assert torch.allclose(val, ref_val, atol=1e-3, rtol=1e-3)
        logits = x.float() @ w.float().t()
        assert torch.allclose(val, logits.max(-1).values, atol=2e-2, rtol=1e-2)
    assert int(err.item()) == 0


def test_noalloc_rejects_sizes_beyond_its_scratch():
    fn = _entry()
    dev = torch.device("cuda")
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    x = torch.zeros(MAX_ROWS + 1, 64, dtype=torch.bfloat16, device=dev)
    w = torch.zeros(256, 64, dtype=torch.bfloat16, device=dev)
    rc, idx, _ = _call(fn, x, w, err)
    assert rc == TOO_LARGE
    assert (idx == -1).all()  # nothing was launched
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device=dev)
    rc = fn(x.data_ptr(), w.data_ptr(), idx.data_ptr(), None, 4, (MAX_TILES + 1) * 128, 64, 64, 64, err.data_ptr(),
            torch.cuda.current_stream().cuda_stream)
    assert rc == TOO_LARGE
