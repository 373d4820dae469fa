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
        h = model.forward(PackedBatch(toks[a:b], [0, b - a], [1], [a], table), "prefill")
        out.append(model.logits(h))
    for t in range(n, n + 3):
        h = model.forward(PackedBatch(toks[t : t + 1], [0, 1], [1], [t], table), "decode")
        out.append(model.logits(h))
    got = torch.cat(out)
    err = (got - ref).abs().max().item()
    assert err < 2e-4 * max(1.0, ref.abs().max().item()), err
    assert (got.argmax(-1) == ref.argmax(-1)).all()
