"""Typed configuration: model architecture and engine knobs.

``ModelConfig`` mirrors the text part of the Hugging Face ``qwen3_5_moe``
config (the reference reads the same fields through Transformers,
``engine/fast/model.py:296-360``). ``EngineConfig`` collects every serving knob
in one dataclass built from CLI flags and ``ENGINE_*`` environment variables
(the reference spreads ~97 ``ENGINE_*`` reads over its modules,
``engine/server.py:627-690``).
"""

from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field, fields
from pathlib import Path
from typing import Any

PAGE_SIZE = 64  # tokens per KV page (reference: engine/fast/model.py:45)
GDN_CHUNK = 64  # rows per Gated-DeltaNet prefill chunk


@dataclass
class ModelConfig:
    vocab_size: int = 248320
    hidden_size: int = 2048
    num_hidden_layers: int = 40
    layer_types: list[str] = field(default_factory=list)
    full_attention_interval: int = 4
    num_attention_heads: int = 16
    num_key_value_heads: int = 2
    head_dim: int = 256
    partial_rotary_factor: float = 0.25
    rope_theta: float = 10000000.0
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4
    num_experts: int = 256
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 512
    shared_expert_intermediate_size: int = 512
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 262144
    mtp_num_hidden_layers: int = 1
    eos_token_ids: list[int] = field(default_factory=list)

    def __post_init__(self) -> None:
        if not self.layer_types:
            k = self.full_attention_interval
            self.layer_types = [
                "full_attention" if (i + 1) % k == 0 else "linear_attention"
                for i in range(self.num_hidden_layers)
            ]
        if len(self.layer_types) != self.num_hidden_layers:
            raise ValueError("layer_types must have one entry per layer")

    # ---- derived sizes -------------------------------------------------
    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def gdn_key_dim(self) -> int:
        return self.linear_num_key_heads * self.linear_key_head_dim

    @property
    def gdn_value_dim(self) -> int:
        return self.linear_num_value_heads * self.linear_value_head_dim

    @property
    def gdn_conv_dim(self) -> int:
        return 2 * self.gdn_key_dim + self.gdn_value_dim

    @property
    def gdn_in_rows(self) -> int:
        """Rows of the merged ``qkv|z|b|a`` input projection."""
        return self.gdn_conv_dim + self.gdn_value_dim + 2 * self.linear_num_value_heads

    @property
    def attn_q_rows(self) -> int:
        return self.num_attention_heads * self.head_dim * 2  # query and gate, interleaved per head

    @property
    def attn_kv_rows(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def attention_layers(self) -> list[int]:
        return [i for i, t in enumerate(self.layer_types) if t == "full_attention"]

    @property
    def gdn_layers(self) -> list[int]:
        return [i for i, t in enumerate(self.layer_types) if t == "linear_attention"]

    @property
    def num_kv_layers(self) -> int:
        """Attention layers that own KV pages: the stack's plus the MTP block's."""
        return len(self.attention_layers) + self.mtp_num_hidden_layers

    def kv_bytes_per_token(self, itemsize: int = 2) -> int:
        return self.num_kv_layers * 2 * self.num_key_value_heads * self.head_dim * itemsize

    def gdn_state_bytes(self) -> int:
        """Bytes of recurrent (fp32) plus conv (bf16) state of one sequence over all GDN layers."""
        rec = self.linear_num_value_heads * self.linear_key_head_dim * self.linear_value_head_dim * 4
        conv = self.gdn_conv_dim * (self.linear_conv_kernel_dim - 1) * 2
        return len(self.gdn_layers) * (rec + conv)

    def param_count(self) -> int:
        h = self.hidden_size
        moe = (
            self.num_experts * 3 * h * self.moe_intermediate_size
            + 3 * h * self.shared_expert_intermediate_size
            + self.num_experts * h
            + h
        )
        gdn = self.gdn_in_rows * h + self.gdn_value_dim * h + self.gdn_conv_dim * self.linear_conv_kernel_dim
        attn = (self.attn_q_rows + 2 * self.attn_kv_rows) * h + self.num_attention_heads * self.head_dim * h
        total = 2 * self.vocab_size * h
        for t in self.layer_types:
            total += moe + (gdn if t == "linear_attention" else attn) + 2 * h
        return total

    # ---- construction --------------------------------------------------
    @classmethod
    def qwen36_35b_a3b(cls) -> "ModelConfig":
        return cls()

    @classmethod
    def tiny(cls, **overrides: Any) -> "ModelConfig":
        """Small model of the same hybrid architecture: 3 GDN layers + 1 gated-attention layer."""
        base = dict(
            vocab_size=1024,
            hidden_size=128,
            num_hidden_layers=4,
            full_attention_interval=4,
            num_attention_heads=4,
            num_key_value_heads=1,
            head_dim=32,
            partial_rotary_factor=0.25,
            linear_num_key_heads=2,
            linear_num_value_heads=4,
            linear_key_head_dim=32,
            linear_value_head_dim=32,
            linear_conv_kernel_dim=4,
            num_experts=8,
            num_experts_per_tok=2,
            moe_intermediate_size=64,
            shared_expert_intermediate_size=64,
            max_position_embeddings=4096,
            mtp_num_hidden_layers=1,
        )
        base.update(overrides)
        return cls(**base)

    @classmethod
    def from_hf_dict(cls, cfg: dict[str, Any]) -> "ModelConfig":
        text = cfg.get("text_config", cfg)
        rope = text.get("rope_parameters") or text.get("rope_scaling") or {}
        rope_type = rope.get("rope_type", rope.get("type", "default"))
        if rope_type != "default":
            raise ValueError(f"unsupported rope type {rope_type!r}")  # reference: model.py:312-314
        names = {f.name for f in fields(cls)}
        kwargs = {k: v for k, v in text.items() if k in names}
        kwargs["partial_rotary_factor"] = rope.get(
            "partial_rotary_factor", text.get("partial_rotary_factor", 1.0)
        )
        kwargs["rope_theta"] = float(rope.get("rope_theta", text.get("rope_theta", 10000.0)))
        kwargs.setdefault("mtp_num_hidden_layers", int(text.get("mtp_num_hidden_layers", 0) or 0))
        eos = text.get("eos_token_id", cfg.get("eos_token_id"))
        kwargs["eos_token_ids"] = [] if eos is None else ([eos] if isinstance(eos, int) else list(eos))
        kwargs.pop("layer_types", None)
        out = cls(layer_types=list(text.get("layer_types") or []), **kwargs)
        return out

    @classmethod
    def from_pretrained(cls, path: str | os.PathLike) -> "ModelConfig":
        path = Path(path)
        cfg = cls.from_hf_dict(json.loads((path / "config.json").read_text()))
        gen = path / "generation_config.json"
        if gen.exists():  # may list several end ids (reference: generator.py:670-676)
            eos = json.loads(gen.read_text()).get("eos_token_id")
            if eos is not None:
                cfg.eos_token_ids = [eos] if isinstance(eos, int) else list(eos)
        return cfg

    def to_hf_dict(self) -> dict[str, Any]:
        text = asdict(self)
        eos = text.pop("eos_token_ids")
        text["eos_token_id"] = eos[0] if eos else None
        text["model_type"] = "qwen3_5_moe_text"
        text["hidden_act"] = "silu"
        text["attention_bias"] = False
        text["tie_word_embeddings"] = False
        text["rope_parameters"] = {
            "rope_type": "default",
            "rope_theta": text.pop("rope_theta"),
            "partial_rotary_factor": self.partial_rotary_factor,
        }
        return {
            "architectures": ["Qwen3_5MoeForConditionalGeneration"],
            "model_type": "qwen3_5_moe",
            "dtype": "bfloat16",
            "text_config": text,
            "tie_word_embeddings": False,
        }


def _env(name: str, default: Any, cast: Any = None) -> Any:
    raw = os.environ.get(name)
    if raw is None or raw == "":
        return default
    cast = cast or type(default)
    if cast is bool:
        return raw.lower() not in ("0", "false", "off", "no")
    return cast(raw)


@dataclass
class EngineConfig:
    """Serving knobs. CLI flags keep the reference's names; env twins are ``ENGINE_*``."""

    model: str = ""
    revision: str | None = None
    served_model_name: str | None = None
    host: str = "127.0.0.1"
    port: int = 8000
    max_model_len: int = 262144
    prefill_chunk_tokens: int = 2048
    prefix_cache_tokens: int = 4194304
    prefix_cache_entries: int = 128
    prefix_cache_gib: float = 16.0
    replicas: int | None = None
    gpus_per_replica: int | None = None
    replica_devices: str | None = None
    # engine sizing
    device: str = "auto"  # "auto" | "cpu" | "cuda"
    dtype: str = "auto"  # "auto": fp32 on CPU, bf16 on CUDA
    max_seqs: int = 128  # concurrent running sequences (state slots in use by requests)
    state_slots: int = 0  # 0: max_seqs + room for prefix-cache snapshots
    kv_pages: int = 0  # 0: size from free device memory
    kv_fraction: float = 0.85
    reserve_gb: float = 6.0
    prefill_pack_tokens: int = 8192
    # an uncached prompt part of at most this many tokens is prefilled as one span without a snapshot (0: always
    # chunk-aligned spans with a snapshot at the last chunk boundary, so that other requests can share the prefix)
    one_pass_max: int = 0
    decode_buckets: tuple[int, ...] = (1, 2, 4, 8, 16, 32, 64, 128, 256)
    cuda_graphs: bool = True
    graphs_on_cpu: bool = False  # tests: run the decode-graph scheduling (buckets, run-ahead) without a CUDA device
    run_ahead: bool = True  # launch decode step n + 1 from device-built inputs before the host has read step n
    # captured prefill passes for one request's short span (a session's next turn, a short prompt): padded row counts
    # of the graphs; a span of up to rows - 64 tokens fits the graph of `rows`
    prefill_graphs: bool = False
    prefill_graph_rows: tuple[int, ...] = (128, 256, 512, 1024)
    # tile-pack the GEMM weights on the GPU (in place: the engine then owns the weights; not under tensor parallelism)
    pack_weights: bool = False
    # parallelism inside one replica
    tp: int = 1
    ep: int = 1
    fused_collectives: bool = True
    # speculation
    mtp: bool = True
    spec_k: int = 0  # 0: policy picks; >0: fixed draft depth
    spec_kmax: int = 3  # deepest draft chain the policy may choose (up to 7, as the reference's k in {1,3,4,5,7})
    # draft tokens from a vocabulary shortlist (spec/ivf.py) instead of the full LM head: 0 = off, else the number of
    # clusters of the index built at load; draft_ivf_probes clusters are scored exactly per draft
    draft_ivf: int = 0
    draft_ivf_probes: int = 64
    # observability
    loop_timers: bool = False
    req_stamps: bool = False

    @classmethod
    def from_env(cls, **overrides: Any) -> "EngineConfig":
        cfg = cls()
        env_map = {
            "max_seqs": "ENGINE_SLOTS",
            "kv_fraction": "ENGINE_KV_FRACTION",
            "reserve_gb": "ENGINE_RESERVE_GB",
            "prefill_pack_tokens": "ENGINE_PREFILL_PACK_TOKENS",
            "one_pass_max": "ENGINE_PREFILL_ONE_PASS_MAX",
            "cuda_graphs": "ENGINE_CUDA_GRAPHS",
            "run_ahead": "ENGINE_RUNAHEAD",
            "prefill_graphs": "ENGINE_PREFILL_GRAPHS",
            "pack_weights": "ENGINE_PACK_WEIGHTS",
            "tp": "ENGINE_TP",
            "ep": "ENGINE_EP",
            "fused_collectives": "ENGINE_FUSED_COLLECTIVES",
            "mtp": "ENGINE_MTP",
            "spec_k": "ENGINE_SPEC_K",
            "spec_kmax": "ENGINE_SPEC_KMAX",
            "draft_ivf": "ENGINE_DRAFT_IVF",
            "draft_ivf_probes": "ENGINE_DRAFT_IVF_PROBES",
            "loop_timers": "ENGINE_LOOP_TIMERS",
            "req_stamps": "ENGINE_REQ_STAMPS",
            "device": "ENGINE_DEVICE",
            "kv_pages": "ENGINE_KV_PAGES",
            "state_slots": "ENGINE_STATE_SLOTS",
        }
        for attr, env in env_map.items():
            setattr(cfg, attr, _env(env, getattr(cfg, attr)))
        buckets = os.environ.get("ENGINE_DECODE_BUCKETS")
        if buckets:
            cfg.decode_buckets = tuple(sorted({int(b) for b in buckets.split(",")}))
        rows = os.environ.get("ENGINE_PREFILL_GRAPH_ROWS")
        if rows:
            cfg.prefill_graph_rows = tuple(sorted({int(r) for r in rows.split(",")}))
        for k, v in overrides.items():
            if v is not None:
                setattr(cfg, k, v)
        return cfg
