"""Weights: Hugging Face safetensors loader, tiny-checkpoint writer, random init.

The engine reads the BF16 HF checkpoint layout of ``Qwen/Qwen3.6-35B-A3B``
directly (no Transformers modelling code on the load path), including the
``mtp.*`` tensors that Transformers drops (reference: ``engine/mtp.py:154-188``),
and repacks it for the kernels:

* GDN ``in_proj_qkv | z | b | a`` become one ``[rows, H]`` matrix, attention
  ``q | k | v`` likewise, so each mixer input is one GEMM
  (reference packs the same way for its GEMV, ``engine/fast/fused.py:75-91``).
* Experts are stacked ``[E, 2I, H]`` / ``[E, H, I]``; when the shared expert has
  the routed experts' width it is appended as expert ``E`` and the shared gate as
  router row ``E``, which turns the shared path into one more (always selected)
  pair of the grouped GEMM.
"""

from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable

import torch

from ..config import ModelConfig

INDEX = "model.safetensors.index.json"


@dataclass
class LayerWeights:
    kind: str  # "linear_attention" | "full_attention"
    input_norm: torch.Tensor
    post_norm: torch.Tensor
    # mixer
    in_proj: torch.Tensor  # GDN: qkv|z|b|a rows; attention: q(+gate)|k|v rows
    out_proj: torch.Tensor
    conv_w: torch.Tensor | None = None  # [C, K]
    A_log: torch.Tensor | None = None
    dt_bias: torch.Tensor | None = None
    gnorm_w: torch.Tensor | None = None
    q_norm: torch.Tensor | None = None
    k_norm: torch.Tensor | None = None
    # MoE
    router: torch.Tensor | None = None  # [E (+1 shared gate), H]
    w_gate_up: torch.Tensor | None = None  # [E (+1), 2I, H]
    w_down: torch.Tensor | None = None  # [E (+1), H, I]
    shared_merged: bool = True
    shared_gate_up: torch.Tensor | None = None  # only when not merged
    shared_down: torch.Tensor | None = None
    shared_gate: torch.Tensor | None = None
    expert_map: torch.Tensor | None = None  # expert parallelism: global expert id -> local slot or -1

    def tensors(self):
        for k, v in self.__dict__.items():
            if isinstance(v, torch.Tensor):
                yield k, v


@dataclass
class MTPWeights:
    fc: torch.Tensor  # [H, 2H]
    pre_fc_norm_embedding: torch.Tensor
    pre_fc_norm_hidden: torch.Tensor
    norm: torch.Tensor
    layer: LayerWeights


@dataclass
class Weights:
    config: ModelConfig
    embed: torch.Tensor
    lm_head: torch.Tensor
    final_norm: torch.Tensor
    layers: list[LayerWeights] = field(default_factory=list)
    mtp: MTPWeights | None = None
    vocab_start: int = 0  # first vocabulary row held by this rank's lm_head shard
    full_vocab: int = 0  # vocabulary size of the whole model when lm_head is a shard

    @property
    def device(self) -> torch.device:
        return self.embed.device

    @property
    def dtype(self) -> torch.dtype:
        return self.embed.dtype

    def _map(self, fn: Callable[[str, torch.Tensor], torch.Tensor]) -> "Weights":
        def layer(lw: LayerWeights) -> LayerWeights:
            kw = dict(lw.__dict__)
            for k, v in lw.tensors():
                kw[k] = fn(k, v)
            return LayerWeights(**kw)

        mtp = None
        if self.mtp is not None:
            m = self.mtp
            mtp = MTPWeights(
                fn("fc", m.fc),
                fn("norm", m.pre_fc_norm_embedding),
                fn("norm", m.pre_fc_norm_hidden),
                fn("norm", m.norm),
                layer(m.layer),
            )
        return Weights(
            self.config,
            fn("embed", self.embed),
            fn("lm_head", self.lm_head),
            fn("norm", self.final_norm),
            [layer(lw) for lw in self.layers],
            mtp,
            self.vocab_start,
            self.full_vocab,
        )

    def to(self, device: torch.device | str | None = None, dtype: torch.dtype | None = None) -> "Weights":
        """Move/cast. ``A_log`` and ``dt_bias`` stay fp32 whatever ``dtype`` is."""

        def fn(name: str, t: torch.Tensor) -> torch.Tensor:
            if not t.is_floating_point():
                return t.to(device=device)
            dt = torch.float32 if name in ("A_log", "dt_bias") else dtype
            return t.to(device=device, dtype=dt)

        return self._map(fn)

    def nbytes(self) -> int:
        total = 0

        def fn(_n: str, t: torch.Tensor) -> torch.Tensor:
            nonlocal total
            total += t.numel() * t.element_size()
            return t

        self._map(fn)
        return total


# --------------------------------------------------------------------------- name handling
_CORE = re.compile(r"^(?:model\.)?(?:language_model\.)*(?:model\.)?(embed_tokens|layers|norm)\.(.*)$")


def canonical_name(name: str) -> str | None:
    """Map a checkpoint tensor name to ``embed_tokens.* | layers.N.* | norm.* | lm_head.* | mtp.*``.

    HF exports nest the text model under varying ``model.language_model.`` prefixes;
    vision tensors map to ``None``.
    """
    if name.startswith("mtp."):
        return name
    if name.startswith("lm_head.") or name.endswith("lm_head.weight"):
        return "lm_head.weight"
    if "visual" in name:
        return None
    m = _CORE.match(name)
    if m:
        return f"{m.group(1)}.{m.group(2)}"
    return None


class _TensorSource:
    """Random access to a (possibly sharded) safetensors checkpoint by canonical name."""

    def __init__(self, path: Path) -> None:
        from safetensors import safe_open

        self.path = path
        self._open = safe_open
        self.where: dict[str, tuple[str, str]] = {}
        index = path / INDEX
        if index.exists():
            weight_map = json.loads(index.read_text())["weight_map"]
        else:
            weight_map = {}
            for shard in sorted(path.glob("*.safetensors")):
                with safe_open(str(shard), framework="pt") as f:
                    for k in f.keys():
                        weight_map[k] = shard.name
        for raw, shard in weight_map.items():
            canon = canonical_name(raw)
            if canon is not None:
                self.where[canon] = (shard, raw)
        self._readers: dict[str, Any] = {}

    def has(self, name: str) -> bool:
        return name in self.where

    def get(self, name: str) -> torch.Tensor:
        shard, raw = self.where[name]
        if shard not in self._readers:
            self._readers[shard] = self._open(str(self.path / shard), framework="pt")
        return self._readers[shard].get_tensor(raw)


def _load_layer(src: _TensorSource, prefix: str, kind: str, cfg: ModelConfig) -> LayerWeights:
    g = lambda n: src.get(prefix + n)  # noqa: E731
    if kind == "linear_attention":
        la = "linear_attn."
        in_proj = torch.cat(
            [g(la + "in_proj_qkv.weight"), g(la + "in_proj_z.weight"), g(la + "in_proj_b.weight"), g(la + "in_proj_a.weight")],
            dim=0,
        )
        mixer = dict(
            in_proj=in_proj,
            out_proj=g(la + "out_proj.weight"),
            conv_w=g(la + "conv1d.weight").squeeze(1).contiguous(),
            A_log=g(la + "A_log").float(),
            dt_bias=g(la + "dt_bias").float(),
            gnorm_w=g(la + "norm.weight"),
        )
    else:
        sa = "self_attn."
        in_proj = torch.cat([g(sa + "q_proj.weight"), g(sa + "k_proj.weight"), g(sa + "v_proj.weight")], dim=0)
        mixer = dict(
            in_proj=in_proj,
            out_proj=g(sa + "o_proj.weight"),
            q_norm=g(sa + "q_norm.weight"),
            k_norm=g(sa + "k_norm.weight"),
        )
    mlp = prefix + "mlp."
    E = cfg.num_experts
    if src.has(mlp + "experts.gate_up_proj"):
        gate_up = src.get(mlp + "experts.gate_up_proj")
        down = src.get(mlp + "experts.down_proj")
    else:  # one tensor per expert and projection
        gate_up = torch.stack(
            [
                torch.cat([src.get(f"{mlp}experts.{e}.gate_proj.weight"), src.get(f"{mlp}experts.{e}.up_proj.weight")], 0)
                for e in range(E)
            ]
        )
        down = torch.stack([src.get(f"{mlp}experts.{e}.down_proj.weight") for e in range(E)])
    router = src.get(mlp + "gate.weight")
    sh_gu = torch.cat([src.get(mlp + "shared_expert.gate_proj.weight"), src.get(mlp + "shared_expert.up_proj.weight")], 0)
    sh_down = src.get(mlp + "shared_expert.down_proj.weight")
    sh_gate = src.get(mlp + "shared_expert_gate.weight")
    moe = _pack_moe(router, gate_up, down, sh_gu, sh_down, sh_gate)
    return LayerWeights(
        kind=kind,
        input_norm=g("input_layernorm.weight"),
        post_norm=g("post_attention_layernorm.weight"),
        **mixer,
        **moe,
    )


def _pack_moe(router, gate_up, down, sh_gu, sh_down, sh_gate) -> dict[str, Any]:
    if sh_gu.shape[0] == gate_up.shape[1]:
        return dict(
            router=torch.cat([router, sh_gate], 0),
            w_gate_up=torch.cat([gate_up, sh_gu[None]], 0),
            w_down=torch.cat([down, sh_down[None]], 0),
            shared_merged=True,
        )
    return dict(
        router=router, w_gate_up=gate_up, w_down=down, shared_merged=False,
        shared_gate_up=sh_gu, shared_down=sh_down, shared_gate=sh_gate,
    )


def load_checkpoint(path: str | Path, device: str | torch.device = "cpu", dtype: torch.dtype | None = None,
                    shard: tuple[int, int] | None = None, experts: tuple[int, int] | None = None,
                    layers: tuple[int, int] | None = None) -> Weights:
    """Read a HF-layout checkpoint directory into engine ``Weights`` on ``device``.

    ``shard = (rank, world)`` keeps only that rank's tensor/expert-parallel part: every layer is
    cut on the host right after it is read, so a rank never holds more than one full layer.
    ``experts = (rank, world)`` keeps all dense weights and only that rank's routed experts plus the shared one
    (data-parallel attention with expert-parallel MoE, ``parallel/ep.py``); the MTP block is not loaded then.
    ``layers = (rank, world)`` reads only that rank's run of layers of a layer-split replica (``parallel/pp.py``): the
    result is what ``parallel.pp.split_layers`` makes of the full weights, without ever holding them."""
    path = Path(path)
    cfg = ModelConfig.from_pretrained(path)
    src = _TensorSource(path)
    out_cfg = cfg
    cut = lambda lw, i: lw  # noqa: E731
    v0, v1 = 0, cfg.vocab_size
    if shard is not None and shard[1] > 1:
        from ..parallel.tp import local_config, shard_layer

        rank, world = shard
        out_cfg = local_config(cfg, world)
        cut = lambda lw, i: shard_layer(lw, cfg, rank, world, i)  # noqa: E731
        per = (cfg.vocab_size + world - 1) // world
        v0, v1 = rank * per, min(cfg.vocab_size, (rank + 1) * per)
    if experts is not None and experts[1] > 1:
        from ..parallel.ep import shard_layer_experts

        cut = lambda lw, i: shard_layer_experts(lw, cfg.num_experts, experts[0], experts[1])  # noqa: E731
    if layers is not None and layers[1] > 1:
        import copy

        from ..parallel.pp import layer_range

        first, end = layer_range(len(cfg.layer_types), layers[0], layers[1])
        local = copy.deepcopy(cfg)
        local.layer_types = list(cfg.layer_types[first:end])
        local.num_hidden_layers = end - first
        local.mtp_num_hidden_layers = 0
        run = [_layer_to(_load_layer(src, f"layers.{i}.", cfg.layer_types[i], cfg), device, dtype) for i in range(first, end)]
        boundary = src.get(f"layers.{end}.input_layernorm.weight") if end < len(cfg.layer_types) else src.get("norm.weight")
        return Weights(local, src.get("embed_tokens.weight").to(device=device, dtype=dtype),
                       src.get("lm_head.weight").to(device=device, dtype=dtype).contiguous(),
                       boundary.to(device=device, dtype=dtype), run, None, vocab_start=0, full_vocab=cfg.vocab_size)
    layers = []
    for i, kind in enumerate(cfg.layer_types):
        layers.append(_layer_to(cut(_load_layer(src, f"layers.{i}.", kind, cfg), i), device, dtype))
    mtp = None
    if cfg.mtp_num_hidden_layers and src.has("mtp.fc.weight") and not (experts is not None and experts[1] > 1):
        lw = cut(_load_layer(src, "mtp.layers.0.", "full_attention", cfg), len(cfg.layer_types))
        mtp = MTPWeights(
            fc=src.get("mtp.fc.weight").to(device=device, dtype=dtype),
            pre_fc_norm_embedding=src.get("mtp.pre_fc_norm_embedding.weight").to(device=device, dtype=dtype),
            pre_fc_norm_hidden=src.get("mtp.pre_fc_norm_hidden.weight").to(device=device, dtype=dtype),
            norm=src.get("mtp.norm.weight").to(device=device, dtype=dtype),
            layer=_layer_to(lw, device, dtype),
        )
    else:
        cfg.mtp_num_hidden_layers = 0
        out_cfg.mtp_num_hidden_layers = 0
    return Weights(
        out_cfg,
        src.get("embed_tokens.weight").to(device=device, dtype=dtype),
        src.get("lm_head.weight")[v0:v1].to(device=device, dtype=dtype).contiguous(),
        src.get("norm.weight").to(device=device, dtype=dtype),
        layers,
        mtp,
        vocab_start=v0,
        full_vocab=cfg.vocab_size,
    )


def _layer_to(lw: LayerWeights, device, dtype) -> LayerWeights:
    kw = dict(lw.__dict__)
    for k, v in lw.tensors():
        dt = torch.float32 if k in ("A_log", "dt_bias") else dtype
        kw[k] = v.to(device=device, dtype=dt) if v.is_floating_point() else v.to(device=device)
    return LayerWeights(**kw)


# --------------------------------------------------------------------------- random init
def _randn(shape, std, gen, device, dtype):
    if device is not None and torch.device(device).type == "cuda":
        t = torch.empty(shape, device=device, dtype=dtype)
        t.normal_(0.0, std, generator=gen)
        return t
    return (torch.randn(shape, generator=gen, dtype=torch.float32) * std).to(dtype)


def random_layer(cfg: ModelConfig, kind: str, gen, device, dtype, std: float = 0.02) -> LayerWeights:
    H = cfg.hidden_size
    r = lambda *s: _randn(s, std, gen, device, dtype)  # noqa: E731
    n = lambda d: _randn((d,), std, gen, device, dtype)  # noqa: E731
    if kind == "linear_attention":
        nv = cfg.linear_num_value_heads
        if device is not None and torch.device(device).type == "cuda":
            A = torch.empty(nv, device=device).uniform_(1.0, 16.0, generator=gen)
            dt = torch.empty(nv, device=device).uniform_(-1.0, 1.0, generator=gen)
        else:
            A = torch.empty(nv).uniform_(1.0, 16.0, generator=gen)
            dt = torch.empty(nv).uniform_(-1.0, 1.0, generator=gen)
        mixer = dict(
            in_proj=r(cfg.gdn_in_rows, H),
            out_proj=r(H, cfg.gdn_value_dim),
            conv_w=_randn((cfg.gdn_conv_dim, cfg.linear_conv_kernel_dim), 0.3, gen, device, dtype),
            A_log=torch.log(A).float(),
            dt_bias=dt.float(),
            gnorm_w=1.0 + n(cfg.linear_value_head_dim),
        )
    else:
        mixer = dict(
            in_proj=r(cfg.attn_q_rows + 2 * cfg.attn_kv_rows, H),
            out_proj=r(H, cfg.num_attention_heads * cfg.head_dim),
            q_norm=n(cfg.head_dim),
            k_norm=n(cfg.head_dim),
        )
    E, I, Is = cfg.num_experts, cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size
    merged = I == Is
    Et = E + 1 if merged else E
    moe = dict(router=r(Et, H), w_gate_up=r(Et, 2 * I, H), w_down=r(Et, H, I), shared_merged=merged)
    if not merged:
        moe.update(shared_gate_up=r(2 * Is, H), shared_down=r(H, Is), shared_gate=r(1, H))
    return LayerWeights(kind=kind, input_norm=n(H), post_norm=n(H), **mixer, **moe)


def random_weights(
    cfg: ModelConfig,
    seed: int = 0,
    device: str | torch.device = "cpu",
    dtype: torch.dtype = torch.bfloat16,
    std: float = 0.02,
    lm_head_std: float | None = None,
) -> Weights:
    """Random-init weights of the given architecture, created on ``device`` (no disk)."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev if dev.type == "cuda" else "cpu")
    gen.manual_seed(seed)
    H = cfg.hidden_size
    embed = _randn((cfg.vocab_size, H), std, gen, dev, dtype)
    layers = [random_layer(cfg, kind, gen, dev, dtype, std) for kind in cfg.layer_types]
    lm_head = _randn((cfg.vocab_size, H), lm_head_std or std, gen, dev, dtype)
    final_norm = _randn((H,), std, gen, dev, dtype)
    mtp = None
    if cfg.mtp_num_hidden_layers:
        mtp = MTPWeights(
            fc=_randn((H, 2 * H), std, gen, dev, dtype),
            pre_fc_norm_embedding=_randn((H,), std, gen, dev, dtype),
            pre_fc_norm_hidden=_randn((H,), std, gen, dev, dtype),
            norm=_randn((H,), std, gen, dev, dtype),
            layer=random_layer(cfg, "full_attention", gen, dev, dtype, std),
        )
    return Weights(cfg, embed, lm_head, final_norm, layers, mtp)


# --------------------------------------------------------------------------- writer
def hf_state_dict(w: Weights, per_expert: bool = False) -> dict[str, torch.Tensor]:
    """Engine weights back to HF tensor names (``model.language_model.*``, ``lm_head``, ``mtp.*``)."""
    cfg = w.config
    out: dict[str, torch.Tensor] = {}

    def layer(prefix: str, lw: LayerWeights) -> None:
        out[prefix + "input_layernorm.weight"] = lw.input_norm
        out[prefix + "post_attention_layernorm.weight"] = lw.post_norm
        if lw.kind == "linear_attention":
            la = prefix + "linear_attn."
            c, v, nv = cfg.gdn_conv_dim, cfg.gdn_value_dim, cfg.linear_num_value_heads
            out[la + "in_proj_qkv.weight"] = lw.in_proj[:c]
            out[la + "in_proj_z.weight"] = lw.in_proj[c : c + v]
            out[la + "in_proj_b.weight"] = lw.in_proj[c + v : c + v + nv]
            out[la + "in_proj_a.weight"] = lw.in_proj[c + v + nv :]
            out[la + "out_proj.weight"] = lw.out_proj
            out[la + "conv1d.weight"] = lw.conv_w[:, None, :]
            out[la + "A_log"] = lw.A_log
            out[la + "dt_bias"] = lw.dt_bias
            out[la + "norm.weight"] = lw.gnorm_w
        else:
            sa = prefix + "self_attn."
            q, kv = cfg.attn_q_rows, cfg.attn_kv_rows
            out[sa + "q_proj.weight"] = lw.in_proj[:q]
            out[sa + "k_proj.weight"] = lw.in_proj[q : q + kv]
            out[sa + "v_proj.weight"] = lw.in_proj[q + kv :]
            out[sa + "o_proj.weight"] = lw.out_proj
            out[sa + "q_norm.weight"] = lw.q_norm
            out[sa + "k_norm.weight"] = lw.k_norm
        mlp = prefix + "mlp."
        E, I = cfg.num_experts, cfg.moe_intermediate_size
        out[mlp + "gate.weight"] = lw.router[:E]
        if per_expert:
            for e in range(E):
                out[f"{mlp}experts.{e}.gate_proj.weight"] = lw.w_gate_up[e, :I]
                out[f"{mlp}experts.{e}.up_proj.weight"] = lw.w_gate_up[e, I:]
                out[f"{mlp}experts.{e}.down_proj.weight"] = lw.w_down[e]
        else:
            out[mlp + "experts.gate_up_proj"] = lw.w_gate_up[:E]
            out[mlp + "experts.down_proj"] = lw.w_down[:E]
        if lw.shared_merged:
            sgu, sd, sg = lw.w_gate_up[E], lw.w_down[E], lw.router[E:]
        else:
            sgu, sd, sg = lw.shared_gate_up, lw.shared_down, lw.shared_gate
        Is = sgu.shape[0] // 2
        out[mlp + "shared_expert.gate_proj.weight"] = sgu[:Is]
        out[mlp + "shared_expert.up_proj.weight"] = sgu[Is:]
        out[mlp + "shared_expert.down_proj.weight"] = sd
        out[mlp + "shared_expert_gate.weight"] = sg

    base = "model.language_model."
    out[base + "embed_tokens.weight"] = w.embed
    out[base + "norm.weight"] = w.final_norm
    out["lm_head.weight"] = w.lm_head
    for i, lw in enumerate(w.layers):
        layer(f"{base}layers.{i}.", lw)
    if w.mtp is not None:
        out["mtp.fc.weight"] = w.mtp.fc
        out["mtp.pre_fc_norm_embedding.weight"] = w.mtp.pre_fc_norm_embedding
        out["mtp.pre_fc_norm_hidden.weight"] = w.mtp.pre_fc_norm_hidden
        out["mtp.norm.weight"] = w.mtp.norm
        layer("mtp.layers.0.", w.mtp.layer)
    return {k: v.detach().cpu().contiguous() for k, v in out.items()}


def save_checkpoint(w: Weights, path: str | Path, per_expert: bool = False) -> None:
    """Write ``config.json``, ``generation_config.json`` and safetensors shards with an index."""
    from safetensors.torch import save_file

    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    state = hf_state_dict(w, per_expert=per_expert)
    main = {k: v for k, v in state.items() if not k.startswith("mtp.")}
    mtp = {k: v for k, v in state.items() if k.startswith("mtp.")}
    save_file(main, str(path / "model-00001-of-00002.safetensors"), metadata={"format": "pt"})
    weight_map = dict.fromkeys(main, "model-00001-of-00002.safetensors")
    if mtp:
        save_file(mtp, str(path / "model-00002-of-00002.safetensors"), metadata={"format": "pt"})
        weight_map.update(dict.fromkeys(mtp, "model-00002-of-00002.safetensors"))
    (path / INDEX).write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    (path / "config.json").write_text(json.dumps(w.config.to_hf_dict(), indent=1))
    eos = w.config.eos_token_ids
    (path / "generation_config.json").write_text(json.dumps({"eos_token_id": eos if eos else None}))
