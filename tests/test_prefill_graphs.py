"""Captured prefill passes: the padded span layout, and the engine taking them (kernel by kernel on the CPU)."""

import pytest
import torch

from b200serve.sched.graphs import GDN_CHUNK_ROWS, prefill_layout, span_chunks, span_tiles


@pytest.mark.parametrize("rows", [128, 256, 512, 1024])
def test_every_span_length_gives_the_same_launch_shape(rows):
    for n in range(1, rows - GDN_CHUNK_ROWS + 1):
        starts = prefill_layout(n, rows)
        assert starts[0] == 0 and starts[1] == n and starts[3] == rows
        assert all(b > a for a, b in zip(starts, starts[1:]))  # no empty span
        chunks, per_span = span_chunks(starts)
        assert len(chunks) == rows // GDN_CHUNK_ROWS + 1
        assert sum(c[2] for c in chunks) == rows and all(1 <= c[2] <= GDN_CHUNK_ROWS for c in chunks)
        assert [c[1] for c in chunks] == sorted(c[1] for c in chunks)
        assert sum(k for _, k in per_span) == len(chunks) and [f for f, _ in per_span] == [0, per_span[0][1], per_span[0][1] + per_span[1][1]]
        for r_tile in (16, 32, 128):
            n_tiles = rows // r_tile + 3
            tiles = span_tiles(starts, r_tile, n_tiles)
            assert len(tiles) == n_tiles
            real = [t for t in tiles if t[3] > 0]
            assert sum(min(r_tile, t[3] - t[1]) for t in real) == rows
            assert all(t == (0, 0, 0, 0) for t in tiles[len(real):])
    with pytest.raises(ValueError):
        prefill_layout(rows - GDN_CHUNK_ROWS + 1, rows)
    with pytest.raises(ValueError):
        prefill_layout(0, rows)


def _engine(w, mtp, graphs, chunk=256):
    from b200serve.config import EngineConfig
    from b200serve.sched.engine import Engine

    ecfg = EngineConfig(max_model_len=2048, prefill_chunk_tokens=chunk, max_seqs=4, mtp=mtp, spec_k=2 if mtp else 0, kv_pages=160,
                        device="cpu", graphs_on_cpu=True, prefill_graphs=graphs, decode_buckets=(1, 4))
    return Engine(w, ecfg)


@pytest.mark.parametrize("mtp", [False, True])
def test_padded_passes_keep_tokens_and_states(mtp):
    """One request at a time (its spans run as padded passes), then its next turn on the cached context (which reads
    the recurrent state and the KV pages that the padded passes left), against the same engine without them."""
    from b200serve.config import ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.sched.request import Sampling

    cfg = ModelConfig.tiny()
    w = random_weights(cfg, seed=0, dtype=torch.float32, std=0.05, lm_head_std=0.5)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(3, 1024, (n,), generator=g).tolist() for n in (1, 37, 64, 65, 200, 256, 300, 700)]
    s = Sampling(max_tokens=6, ignore_eos=True)
    plain, padded = _engine(w, mtp, False), _engine(w, mtp, True)
    assert padded._pgraphs is not None and plain._pgraphs is None
    for p in prompts:
        a = plain.generate([p], s)[0]
        b = padded.generate([p], s)[0]
        assert a.output == b.output, len(p)
        turn = p + a.output + [9, 8, 7, 6, 5]
        a2 = plain.generate([turn], s)[0]
        b2 = padded.generate([turn], s)[0]
        assert b2.cached_tokens == a2.cached_tokens > 0 or len(p) < 64
        assert a2.output == b2.output
    assert padded.stats["prefill_graph_passes"] > len(prompts) and not padded._pgraphs.errors
    assert sorted(padded._pgraphs.buckets) == [128, 256, 512]
    if mtp:
        assert padded.stats["mtp_verify_steps"] > 0


def test_packed_and_long_spans_run_the_general_path():
    from b200serve.config import ModelConfig
    from b200serve.models.checkpoint import random_weights
    from b200serve.sched.request import Sampling

    cfg = ModelConfig.tiny()
    w = random_weights(cfg, seed=0, dtype=torch.float32, std=0.05, lm_head_std=0.5)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(3, 1024, (n,), generator=g).tolist() for n in (50, 90, 130)]
    s = Sampling(max_tokens=4, ignore_eos=True)
    plain, padded = _engine(w, False, False), _engine(w, False, True)
    assert [x.output for x in plain.generate(prompts, s)] == [x.output for x in padded.generate(prompts, s)]
    assert padded.stats["prefill_graph_passes"] == 0  # three requests packed into one pass
    big = _engine(w, False, True, chunk=2048)
    long_prompt = torch.randint(3, 1024, (1500,), generator=g).tolist()
    out = big.generate([long_prompt], s)[0]
    assert big.stats["prefill_graph_passes"] == 0 and len(out.output) == 4  # 1,500 tokens exceed the largest graph


def test_warmup_builds_every_padded_size_and_the_bench_tool_runs_without_a_gpu():
    import json
    import subprocess
    import sys
    from pathlib import Path

    from b200serve.config import ModelConfig
    from b200serve.models.checkpoint import random_weights

    w = random_weights(ModelConfig.tiny(), seed=0, dtype=torch.float32, std=0.05, lm_head_std=0.5)
    eng = _engine(w, False, True, chunk=2048)
    eng.warmup()
    assert sorted(eng._pgraphs.buckets) == [128, 256, 512, 1024] and not eng._pgraphs.errors
    assert eng.stats["prefill_graph_passes"] == 0  # counters start from zero after the warm-up
    root = Path(__file__).resolve().parents[1]
    r = subprocess.run([sys.executable, str(root / "bench/prefill_graph_bench.py"), "--tiny", "--start", "200", "--news", "20,90", "--reps", "1"],
                       capture_output=True, text=True, timeout=600, env={**__import__("os").environ, "CUDA_VISIBLE_DEVICES": ""})
    assert r.returncode == 0, r.stderr[-2000:]
    rows = [json.loads(ln) for ln in r.stdout.strip().splitlines() if ln.startswith("{")]
    assert [x["new_tokens"] for x in rows] == [20, 90] and [x["graph_rows"] for x in rows] == [128, 256]
    assert all(x["last_row_max_abs_diff"] < 1e-4 for x in rows)
