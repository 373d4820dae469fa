"""The fp32 torch model against Hugging Face's ``qwen3_5_moe`` implementation."""

import pytest
import torch

from b200serve.config import ModelConfig
from b200serve.models.checkpoint import hf_state_dict, random_weights
from b200serve.models.qwen36 import Model, PackedBatch

transformers = pytest.importorskip("transformers")


def _hf_model(w):
    from transformers import Qwen3_5MoeForCausalLM
    from transformers.models.qwen3_5_moe.configuration_qwen3_5_moe import Qwen3_5MoeTextConfig

    text = w.config.to_hf_dict()["text_config"]
    text.pop("eos_token_ids", None)
    cfg = Qwen3_5MoeTextConfig(**text)
    cfg._attn_implementation = "eager"
    hf = Qwen3_5MoeForCausalLM(cfg).float().eval()
    state = {}
    for k, v in hf_state_dict(w).items():
        if k.startswith("mtp."):
            continue
        state[k.replace("model.language_model.", "model.")] = v.float()
    missing, unexpected = hf.load_state_dict(state, strict=False)
    assert not unexpected, unexpected
    assert all("rotary" in m for m in missing), missing
    return hf


def test_prefill_and_decode_match_hf():
    torch.manual_seed(0)
    cfg = ModelConfig.tiny(mtp_num_hidden_layers=0)
    w = random_weights(cfg, seed=0, dtype=torch.float32, std=0.05)
    hf = _hf_model(w)
    model = Model(w, num_pages=8, state_slots=3)
    n = 75
    toks = torch.randint(0, cfg.vocab_size, (n + 3,))
    with torch.no_grad():
        ref = hf(input_ids=toks[None]).logits[0]
    table = torch.tensor([[1, 2, 3]], dtype=torch.int32)
    # chunked prefill: 40 + 35 rows, then 3 decode steps
    out = []
    for a, b in ((0, 40), (40, n)):
        h = model.forward(PackedBatch.prefill([toks[a:b].tolist()], [1], [a], table, "cpu"))
        out.append(model.logits(h))
    for t in range(n, n + 3):
        h = model.forward(PackedBatch.uniform(toks[t : t + 1], [t], [1], table, 1, "cpu"))
        out.append(model.logits(h))
    got = torch.cat(out)
    err = (got - ref).abs().max().item()
    assert err < 2e-4 * max(1.0, ref.abs().max().item()), err
    assert (got.argmax(-1) == ref.argmax(-1)).all()


def test_batched_gdn_prefill_and_verify_ring_match_serial():
    from b200serve.ops import torch_ops as O

    torch.manual_seed(1)
    cfg = ModelConfig.tiny()
    n_k, n_v, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    C = cfg.gdn_conv_dim
    lens = [5, 130, 64]
    starts = [0, 5, 135, 199]
    mixed = torch.randn(199, cfg.gdn_in_rows)
    conv_w = torch.randn(C, 4) * 0.3
    A_log, dt_bias, gw = torch.rand(n_v), torch.randn(n_v), 1 + 0.1 * torch.randn(dv)
    conv0, rec0 = torch.randn(4, C, 3), torch.randn(4, n_v, dk, dv) * 0.1
    args = (conv_w, A_log, dt_bias, gw, n_k, n_v, dk, dv, 1e-6)
    c1, r1 = conv0.clone(), rec0.clone()
    ref = O.gdn_prefill(mixed, starts, [1, 3, 2], c1, r1, *args)
    c2, r2 = conv0.clone(), rec0.clone()
    got = O.gdn_prefill_batched(mixed, starts, [1, 3, 2], c2, r2, *args)
    assert torch.allclose(ref, got, atol=2e-5, rtol=1e-4)
    assert torch.allclose(c1, c2) and torch.allclose(r1, r2, atol=2e-5, rtol=1e-4)
    # decode continues from the prefill state exactly as a longer prefill would
    more = torch.randn(3 * 4, cfg.gdn_in_rows)  # 3 sequences x 4 rows
    slots = torch.tensor([1, 3, 2])
    c3, r3 = c1.clone(), r1.clone()
    ring = (torch.empty(3, 4, C, 3), torch.empty(3, 4, n_v, dk, dv))
    ver = O.gdn_decode(more, slots, c3, r3, *args, G=4, ring=ring)
    c4, r4 = c1.clone(), r1.clone()
    for j in range(4):
        step = O.gdn_decode(more[j::4].contiguous(), slots, c4, r4, *args)
        assert torch.allclose(step, ver[j::4], atol=1e-6)
        assert torch.allclose(ring[1][:, j], r4[slots], atol=1e-6)
    for i, s in enumerate([1, 3, 2]):
        full = torch.cat([mixed[starts[i]:starts[i + 1]], more[i * 4:(i + 1) * 4]])
        c5, r5 = conv0.clone(), rec0.clone()
        out = O.gdn_prefill(full, [0, full.shape[0]], [s], c5, r5, *args)
        assert torch.allclose(out[-4:], ver[i * 4:(i + 1) * 4], atol=5e-5, rtol=1e-3)
