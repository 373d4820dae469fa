"""The engine on the CUDA kernel path: batching must not change a request's greedy tokens."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(max_seqs=8, graphs=True):
    from b200serve.config import EngineConfig, ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.sched.engine import Engine

    cfg = ModelConfig.tiny()
    w = random_weights(cfg, seed=0, device="cuda", dtype=torch.bfloat16, std=0.05, lm_head_std=0.5)
    ecfg = EngineConfig(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=max_seqs, mtp=False, kv_pages=256,
                        cuda_graphs=graphs, decode_buckets=(1, 4, 8))
    return Engine(w, ecfg)


def _prompts(n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(3, 1024, (int(torch.randint(16, 200, (1,), generator=g)),), generator=g).tolist() for _ in range(n)]


def test_gpu_batched_equals_solo_with_graphs():
    from b200serve.ops import cuda_ops
    from b200serve.sched.request import Sampling

    prompts = _prompts(8)
    s = Sampling(max_tokens=24, ignore_eos=True)
    eng = _mk()
    batched = [g.output for g in eng.generate(prompts, s)]
    assert eng._graphs is not None and eng._graphs.buckets and not eng._graphs.errors
    assert all(len(o) == 24 for o in batched)
    solo_eng = _mk()
    for p, out in zip(prompts[:3], batched[:3]):
        solo_eng.cache.clear()
        assert solo_eng.generate([p], s)[0].output == out
    eager = _mk(graphs=False)
    assert [g.output for g in eager.generate(prompts[:3], s)] == batched[:3]
    cuda_ops.check_errors(torch.device("cuda"))


def test_gpu_session_tail_reuse_matches_cold():
    from b200serve.sched.request import Sampling

    eng = _mk()
    p = _prompts(1, seed=3)[0]
    s = Sampling(max_tokens=9, ignore_eos=True)
    a = eng.generate([p], s)[0]
    nxt = p + a.output + [5, 6, 7]
    c = eng.generate([nxt], s)[0]
    assert c.cached_tokens >= len(p)
    assert len(c.output) == 9


def test_gpu_mtp_speculation_keeps_outputs():
    """Chained MTP verify steps on the CUDA kernels (G rows per sequence, GDN state ring) never change tokens."""
    from b200serve.config import EngineConfig, ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.ops import cuda_ops
    from b200serve.sched.engine import Engine
    from b200serve.sched.request import Sampling

    cfg = ModelConfig.tiny(head_dim=64, num_attention_heads=4, num_key_value_heads=1)
    w = random_weights(cfg, seed=0, device="cuda", dtype=torch.bfloat16, std=0.05, lm_head_std=0.5)
    prompts = _prompts(4, seed=21)
    s = Sampling(max_tokens=20, ignore_eos=True)

    def run(mtp, k=0):
        ecfg = EngineConfig(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=8, mtp=mtp, spec_k=k, kv_pages=256,
                            decode_buckets=(4, 8))
        eng = Engine(w, ecfg)
        return eng, [g.output for g in eng.generate(prompts, s)]

    _, plain = run(False)
    eng, spec = run(True, 2)
    truth = {tuple(p): o for p, o in zip(prompts, plain)}
    assert spec == plain
    assert eng.stats["mtp_verify_steps"] > 0
    eng2 = Engine(w, EngineConfig(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=8, mtp=True, spec_k=3, kv_pages=256))
    eng2.spec.draft_override = lambda g, k: truth[tuple(g.prompt)][len(g.output):len(g.output) + k]
    forced = [g.output for g in eng2.generate(prompts, s)]
    assert forced == plain and eng2.stats["mtp_accepted"] == eng2.stats["mtp_proposed"] > 0
    cuda_ops.check_errors(torch.device("cuda"))
    # drafts from the vocabulary shortlist (captured in the verify graphs, tile-packed head): same outputs
    w2 = random_weights(cfg, seed=0, device="cuda", dtype=torch.bfloat16, std=0.05, lm_head_std=0.5)
    eng3 = Engine(w2, EngineConfig(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=8, mtp=True, spec_k=2, kv_pages=256,
                                   decode_buckets=(4, 8), draft_ivf=16, draft_ivf_probes=4, pack_weights=True))
    assert eng3.model.draft_index is not None
    short = [g.output for g in eng3.generate(prompts, s)]
    assert short == plain and eng3.stats["mtp_verify_steps"] > 0
    cuda_ops.check_errors(torch.device("cuda"))


def test_gpu_engine_with_tile_packed_weights_keeps_tokens():
    """Packing the GEMM weights (``EngineConfig.pack_weights``) is a layout change only: same greedy tokens."""
    from b200serve.config import EngineConfig, ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.ops import cuda_ops
    from b200serve.sched.engine import Engine
    from b200serve.sched.request import Sampling

    prompts = _prompts(5, seed=3)
    s = Sampling(max_tokens=12, ignore_eos=True)
    plain = [g.output for g in _mk().generate(prompts, s)]
    cfg = ModelConfig.tiny(moe_intermediate_size=128, shared_expert_intermediate_size=128)
    outs = []
    for pack in (False, True):
        w = random_weights(cfg, seed=0, device="cuda", dtype=torch.bfloat16, std=0.05, lm_head_std=0.5)
        ecfg = EngineConfig(max_model_len=1024, prefill_chunk_tokens=64, max_seqs=8, mtp=False, kv_pages=256,
                            decode_buckets=(1, 4, 8), pack_weights=pack)
        eng = Engine(w, ecfg)
        if pack:
            assert cuda_ops.is_packed(eng.model.w.layers[0].w_gate_up) and cuda_ops.is_packed(eng.model.w.lm_head)
        outs.append([g.output for g in eng.generate(prompts, s)])
        cuda_ops.check_errors(eng.device)
    assert outs[0] == outs[1]
    assert len(plain) == len(prompts)


def test_gpu_captured_prefill_passes_keep_tokens():
    """One request's short spans as padded, captured passes (filler rows on the scratch slot and page, fixed-length
    span tables on the device): same tokens as the passes run kernel by kernel, first turn and next turn, with the
    MTP block inside the graph."""
    from b200serve.config import EngineConfig, ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.ops import cuda_ops
    from b200serve.sched.engine import Engine
    from b200serve.sched.request import Sampling

    cfg = ModelConfig.tiny(head_dim=64, num_attention_heads=4, num_key_value_heads=1)
    w = random_weights(cfg, seed=0, device="cuda", dtype=torch.bfloat16, std=0.05, lm_head_std=0.5)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(3, 1024, (n,), generator=g).tolist() for n in (1, 37, 64, 65, 200, 256, 300, 700)]
    s = Sampling(max_tokens=8, ignore_eos=True)

    def mk(graphs):
        return Engine(w, EngineConfig(max_model_len=2048, prefill_chunk_tokens=256, max_seqs=4, mtp=True, spec_k=2, kv_pages=160,
                                      prefill_graphs=graphs, decode_buckets=(1, 4)))

    plain, padded = mk(False), mk(True)
    assert padded._pgraphs is not None
    for p in prompts:
        a = plain.generate([p], s)[0]
        b = padded.generate([p], s)[0]
        assert a.output == b.output, len(p)
        turn = p + a.output + [9, 8, 7, 6, 5]
        assert plain.generate([turn], s)[0].output == padded.generate([turn], s)[0].output, len(p)
    assert not padded._pgraphs.errors, padded._pgraphs.errors
    assert sorted(padded._pgraphs.buckets) == [128, 256, 512]
    assert all(b.graph is not None and b.launches > 0 for b in padded._pgraphs.buckets.values())
    assert padded.stats["prefill_graph_passes"] > len(prompts)
    cuda_ops.check_errors(torch.device("cuda"))
