"""Tensor + expert parallelism without a cluster: CPU ranks over gloo (and 2 GPUs when present)."""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def _launch(mode: str, nproc: int, port: int, env: dict | None = None, timeout: int = 600):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), str(ROOT / "tests/dist_worker.py"), mode]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env={**os.environ, **(env or {})})


def test_shard_shapes():
    from b200serve.config import ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.parallel.tp import local_config, shard_weights

    cfg = ModelConfig.tiny(num_attention_heads=4, num_key_value_heads=2)
    w = random_weights(cfg, seed=0, dtype=torch.float32)
    for world in (2,):
        lc = local_config(cfg, world)
        assert lc.linear_num_value_heads == cfg.linear_num_value_heads // world
        for rank in range(world):
            s = shard_weights(w, rank, world)
            gdn, attn = s.layers[0], s.layers[3]
            assert gdn.in_proj.shape[0] == lc.gdn_in_rows and gdn.out_proj.shape == (cfg.hidden_size, lc.gdn_value_dim)
            assert gdn.conv_w.shape[0] == lc.gdn_conv_dim and gdn.A_log.shape[0] == lc.linear_num_value_heads
            assert attn.in_proj.shape[0] == lc.attn_q_rows + 2 * lc.attn_kv_rows
            hosted = [(i % world) == rank for i in range(4)]
            for lw, h in zip(s.layers, hosted):
                assert lw.w_gate_up.shape[0] == cfg.num_experts // world + int(h)
                assert (lw.expert_map >= 0).sum().item() == lw.w_gate_up.shape[0]
            assert s.lm_head.shape[0] == cfg.vocab_size // world and s.vocab_start == rank * cfg.vocab_size // world
    with pytest.raises(ValueError):
        local_config(cfg, 3)


def test_two_cpu_ranks_match_the_unsharded_engine():
    r = _launch("tp_model", 2, 29621, env={"CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 0 and "OK tp_model" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_four_cpu_ranks_share_kv_heads_and_match_the_unsharded_engine():
    """More ranks than KV heads: ranks of a group hold copies of the same KV head."""
    r = _launch("tp_model", 4, 29624, env={"CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 0 and "OK tp_model" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_ranks_fused_collectives_match_the_unsharded_engine():
    r = _launch("tp_model", 2, 29622, env={"NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0 and "OK tp_model" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_lockstep_replica_on_two_cpu_ranks():
    r = _launch("lockstep", 2, 29623, env={"CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 0 and "OK lockstep" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_ranks_with_different_memory_budgets_agree_on_the_smallest_kv_pool():
    r = _launch("kv_agree", 2, 29625, env={"CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 0 and "OK kv_agree" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_a_failure_on_one_rank_tears_the_whole_lockstep_replica_down():
    r = _launch("lockstep_failure", 2, 29626, env={"CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 0 and "OK lockstep_failure" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_served_tensor_parallel_replica_speculates_like_a_single_process(tmp_path):
    """MTP speculation inside a leader + follower replica: same tokens as a single-process server without it."""
    from http_util import ServerProc, ids_of

    from b200serve.models.tiny import write_tiny_checkpoint

    write_tiny_checkpoint(tmp_path, lm_head_std=0.5)
    tp = ServerProc(tmp_path, extra=["--gpus-per-replica", "2"], env={"CUDA_VISIBLE_DEVICES": "", "ENGINE_MTP": "1", "ENGINE_SPEC_K": "2"})
    one = ServerProc(tmp_path, env={"CUDA_VISIBLE_DEVICES": "", "ENGINE_MTP": "0"})
    try:
        for n in (40, 130):
            prompt = [7 + (i * 13) % 500 for i in range(n)]
            a, _ = tp.completion(prompt, 16)
            b, _ = one.completion(prompt, 16)
            assert ids_of(a) == ids_of(b)
        h = tp.health()
        assert h.get("mtp_verify_steps", 0) > 0
    finally:
        tp.stop()
        one.stop()


@pytest.mark.parametrize("world,port", [(2, 29641), (3, 29642)])
def test_layer_split_replica_on_cpu_ranks_matches_the_unsplit_engine(world, port):
    r = _launch("pp_model", world, port, env={"CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 0 and "OK pp_model" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_layer_split_replica_on_two_gpus_matches_the_unsplit_engine():
    r = _launch("pp_model", 2, 29643, env={"NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0 and "OK pp_model" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_served_layer_split_replica_on_cpu_ranks(tmp_path):
    """`--gpus-per-replica 2 --replica-split layers` without GPUs: each process loads only its run of layers."""
    from http_util import ServerProc, ids_of

    from b200serve.models.tiny import write_tiny_checkpoint

    write_tiny_checkpoint(tmp_path, lm_head_std=0.5)
    pp = ServerProc(tmp_path, extra=["--gpus-per-replica", "2", "--replica-split", "layers"],
                    env={"CUDA_VISIBLE_DEVICES": "", "ENGINE_MTP": "0"})
    one = ServerProc(tmp_path, env={"CUDA_VISIBLE_DEVICES": "", "ENGINE_MTP": "0"})
    try:
        prompt = [5 + (i * 11) % 300 for i in range(100)]
        a, _ = pp.completion(prompt, 12)
        b, _ = one.completion(prompt, 12)
        assert ids_of(a) == ids_of(b)
        again, u2 = pp.completion(prompt, 12)
        assert u2["prompt_tokens_details"]["cached_tokens"] > 0 and ids_of(again) == ids_of(a)
    finally:
        pp.stop()
        one.stop()


def test_served_tensor_parallel_replica_on_cpu_ranks(tmp_path):
    """`--gpus-per-replica 2` on a machine without GPUs: leader + follower processes over gloo, over HTTP."""
    from http_util import ServerProc, ids_of

    from b200serve.models.tiny import write_tiny_checkpoint

    write_tiny_checkpoint(tmp_path, lm_head_std=0.5)
    tp = ServerProc(tmp_path, extra=["--gpus-per-replica", "2"], env={"CUDA_VISIBLE_DEVICES": "", "ENGINE_MTP": "0"})
    one = ServerProc(tmp_path, env={"CUDA_VISIBLE_DEVICES": "", "ENGINE_MTP": "0"})
    try:
        prompt = [5 + (i * 11) % 300 for i in range(100)]
        a, ua = tp.completion(prompt, 12)
        b, _ = one.completion(prompt, 12)
        assert ids_of(a) == ids_of(b)
        again, u2 = tp.completion(prompt, 12)
        assert u2["prompt_tokens_details"]["cached_tokens"] > 0 and ids_of(again) == ids_of(a)
    finally:
        tp.stop()
        one.stop()
