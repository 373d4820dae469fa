"""Writer of a tiny random checkpoint of the real architecture, in HF layout, with a tokenizer.

Used by the CPU contract tests and as the smallest end-to-end serving example: 3 Gated-DeltaNet
layers + 1 gated-attention layer, hidden 128, 8 experts top-2 + 1 shared, vocab 1024, one MTP
block, weights ~N(0, 0.02) (the reference's fixture has the same role:
``.vibesys/shared/cpu_check/tiny_checkpoint.py:93-150``). The tokenizer is a byte-level BPE
trained in-process with the chat special tokens and a chat template that has the real template's
switches: ``enable_thinking``, tools, tool calls with mapping arguments, reasoning history.
"""

from __future__ import annotations

from pathlib import Path

import torch

from ..config import ModelConfig
from .checkpoint import random_weights, save_checkpoint

SPECIAL_TOKENS = ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>"]

CHAT_TEMPLATE = (
    "{% if tools %}<|im_start|>system\nYou may call these tools:\n"
    "{% for t in tools %}\n{{ t | tojson }}{% endfor %}<|im_end|>\n{% endif %}"
    "{% for m in messages %}"
    "{% if m.role == 'assistant' %}<|im_start|>assistant\n"
    "{% if m.reasoning_content is string %}<think>\n{{ m.reasoning_content }}\n</think>\n\n{% endif %}"
    "{{ m.content or '' }}"
    "{% for c in m.tool_calls or [] %}{% set f = c.function if c.function is defined else c %}"
    "\n<tool_call>\n<function={{ f.name }}>"
    "{% for k, v in f.arguments | items %}\n<parameter={{ k }}>\n{{ v if v is string else v | tojson }}\n</parameter>{% endfor %}"
    "\n</function>\n</tool_call>{% endfor %}<|im_end|>\n"
    "{% elif m.content is string %}<|im_start|>{{ m.role }}\n{{ m.content }}<|im_end|>\n"
    "{% else %}<|im_start|>{{ m.role }}\n{% for part in m.content %}{{ part.text }}{% endfor %}<|im_end|>\n"
    "{% endif %}{% endfor %}"
    "{% if add_generation_prompt %}<|im_start|>assistant\n"
    "{% if enable_thinking is defined and enable_thinking is false %}<think>\n\n</think>\n\n"
    "{% else %}<think>\n{% endif %}{% endif %}"
)

_CORPUS = [
    "The quick brown fox jumps over the lazy dog while the engine streams one token at a time.\n",
    "def schedule(requests):\n    for r in sorted(requests, key=len):\n        yield r  # continuous batching\n",
    "Question: what is the capital of France? Answer: Paris. Question: 2 + 2 = 4.\n",
    '{"role": "user", "content": "hello world"}\n',
]


def build_tokenizer(vocab_size: int):
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    from transformers import PreTrainedTokenizerFast

    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(
        vocab_size=vocab_size, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), special_tokens=SPECIAL_TOKENS,
        show_progress=False,
    )
    tok.train_from_iterator(_CORPUS * 16, trainer)
    return PreTrainedTokenizerFast(
        tokenizer_object=tok, eos_token="<|im_end|>", pad_token="<|endoftext|>",
        additional_special_tokens=["<|im_start|>"], chat_template=CHAT_TEMPLATE,
    )


def write_tiny_checkpoint(path: str | Path, cfg: ModelConfig | None = None, seed: int = 0, std: float = 0.02,
                          lm_head_std: float | None = None, per_expert: bool = False) -> ModelConfig:
    """Write config, generation config, tokenizer and random BF16 weights (``mtp.*`` included)."""
    path = Path(path)
    cfg = cfg or ModelConfig.tiny()
    tokenizer = build_tokenizer(min(cfg.vocab_size, 512))
    cfg.eos_token_ids = [tokenizer.convert_tokens_to_ids("<|im_end|>"), tokenizer.convert_tokens_to_ids("<|endoftext|>")]
    weights = random_weights(cfg, seed=seed, dtype=torch.bfloat16, std=std, lm_head_std=lm_head_std)
    save_checkpoint(weights, path, per_expert=per_expert)
    tokenizer.save_pretrained(str(path))
    return cfg
