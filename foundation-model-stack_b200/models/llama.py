"""The Llama dense decoder: configuration, variants, layer plan and checkpoint adapter
(fms/models/llama.py).

This file is all that is specific to the architecture.  It maps ``config.json`` to ``LLaMAConfig``
(fms/models/hf/config_utils/param_builders.py:37-58, :512-546), ``LLaMAConfig`` to a ``DecoderSpec``
(pre-norm RMSNorm, rotary grouped-query attention, SwiGLU feed-forward in every layer,
fms/models/llama.py:65-116), and HF tensor names to the engine's (fms/models/llama.py:648-673), with
the row permutation of the q and k projections (:685-748) and the fusion of q/k/v and of gate/up
(fms/utils/serialization.py:182-270).
"""
from __future__ import annotations

import dataclasses
import re
from typing import Any, Dict, List, Optional

import torch

from ..config.model_config import ModelConfig
from ..config.specs import (BlockSpec, DecoderSpec, FeedForwardSpec, LayerCall, MixerSpec, NormSpec, PositionSpec)
from ..weights.adapters import register_adapter, register_adapter_step
from ..weights.sources import TensorLayout
from . import register_architecture, register_model
from .base import Model


@dataclasses.dataclass
class LLaMAConfig(ModelConfig):
    """Fields and defaults of fms/models/llama.py:42-62.  ``hidden_dim`` (the feed-forward's hidden size)
    is ours: when None it is ``multiple_of * ceil(int(hidden_grow_factor * emb_dim) / multiple_of)`` as the
    reference computes it (fms/modules/feedforward.py:227-233); a config.json gives it directly."""

    src_vocab_size: int = 32_000
    emb_dim: int = 4096
    norm_eps: float = 1e-5
    nheads: int = 32
    kvheads: int = 0
    nlayers: int = 32
    pad_id: int = -1
    hidden_grow_factor: float = 8 / 3
    multiple_of: int = 256
    activation_fn: str = "swish"
    p_dropout: float = 0.0
    max_expected_seq_len: int = 4096
    attn_bias: bool = False
    mlp_bias: bool = False
    tie_heads: bool = False
    rope_theta: float = 10_000.0
    rope_scaling: dict = dataclasses.field(default_factory=dict)
    hidden_dim: Optional[int] = None

    def __post_init__(self) -> None:
        if self.nheads <= 0 or self.emb_dim % self.nheads:
            raise ValueError(f"emb_dim {self.emb_dim} must be a multiple of nheads {self.nheads}")
        kv = self.kvheads or self.nheads
        if self.nheads % kv:
            raise ValueError(f"nheads {self.nheads} must be a multiple of kvheads {kv}")
        if self.p_dropout != 0.0:
            raise ValueError("p_dropout must be 0: this library generates only")

    @property
    def head_dim(self) -> int:
        return self.emb_dim // self.nheads  # fms/models/llama.py:67-68

    @property
    def n_kvheads(self) -> int:
        return self.kvheads or self.nheads  # fms/models/llama.py:89-93

    @property
    def ffn_hidden(self) -> int:
        if self.hidden_dim is not None:
            return int(self.hidden_dim)
        hidden = int(self.hidden_grow_factor * self.emb_dim)
        if self.multiple_of:
            hidden = self.multiple_of * ((hidden + self.multiple_of - 1) // self.multiple_of)
        return hidden


def _config_from_json(values: Dict[str, Any]) -> LLaMAConfig:
    names = values.get("architectures")
    if names and names[0] != "LlamaForCausalLM":
        raise ValueError(f"config.json is of architecture {names[0]!r}, not LlamaForCausalLM")
    required = ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                "rms_norm_eps"]
    absent = [k for k in required if k not in values]
    if absent:
        raise ValueError(f"config.json lacks {absent}")
    hidden, heads = values["hidden_size"], values["num_attention_heads"]
    if values.get("head_dim") not in (None, hidden // heads):
        raise ValueError(f"head_dim {values['head_dim']} differs from hidden_size / num_attention_heads = "
                         f"{hidden // heads}; the reference's Llama has no separate head size")
    act = values.get("hidden_act", "silu")
    if act not in ("silu", "swish"):
        raise ValueError(f"hidden_act {act!r}: the reference's Llama uses SiLU only")
    rope_theta, rope_scaling = values.get("rope_theta"), values.get("rope_scaling")
    if values.get("rope_parameters") is not None:  # param_builders.py:18-34
        rope_theta = values["rope_parameters"]["rope_theta"]
        rope_scaling = values["rope_parameters"].get("rope_scaling")
    return LLaMAConfig(
        src_vocab_size=values["vocab_size"],
        emb_dim=hidden,
        norm_eps=values["rms_norm_eps"],
        nheads=heads,
        kvheads=values.get("num_key_value_heads", heads) or 0,
        nlayers=values["num_hidden_layers"],
        hidden_grow_factor=values["intermediate_size"] / hidden,
        multiple_of=1,
        hidden_dim=values["intermediate_size"],
        max_expected_seq_len=values.get("max_position_embeddings", 4096),
        attn_bias=bool(values.get("attention_bias", False)),
        mlp_bias=bool(values.get("mlp_bias", False)),
        tie_heads=bool(values.get("tie_word_embeddings", False)),
        rope_theta=10_000.0 if rope_theta is None else float(rope_theta),
        rope_scaling=dict(rope_scaling or {}),
    )


class LLaMA(Model):
    architecture = "llama"
    default_source = "hf"

    def __init__(self, config: Optional[LLaMAConfig] = None, **kwargs) -> None:
        config = config if config is not None else LLaMAConfig()
        super().__init__(config.updated(**kwargs))  # fms/models/llama.py:368-372

    @classmethod
    def config_from_json(cls, values: dict) -> LLaMAConfig:
        return _config_from_json(values)

    def config_json(self) -> dict:
        c = self.config
        out = {
            "architectures": ["LlamaForCausalLM"], "model_type": "llama",
            "vocab_size": c.src_vocab_size, "hidden_size": c.emb_dim, "intermediate_size": c.ffn_hidden,
            "num_hidden_layers": c.nlayers, "num_attention_heads": c.nheads, "num_key_value_heads": c.n_kvheads,
            "rms_norm_eps": c.norm_eps, "rope_theta": c.rope_theta, "max_position_embeddings": c.max_expected_seq_len,
            "tie_word_embeddings": c.tie_heads, "hidden_act": "silu", "attention_bias": c.attn_bias,
            "mlp_bias": c.mlp_bias,
        }
        if c.rope_scaling:
            out["rope_scaling"] = dict(c.rope_scaling)
        return out

    def decoder_spec(self) -> DecoderSpec:
        c = self.config
        position = PositionSpec("rope", head_dim=c.head_dim, theta=float(c.rope_theta),
                                max_positions=c.max_expected_seq_len, scaling=tuple(sorted(c.rope_scaling.items())))
        norm = NormSpec("rmsnorm", c.emb_dim, float(c.norm_eps))
        block = BlockSpec(
            mixer=MixerSpec("attention", dim=c.emb_dim, nheads=c.nheads, kvheads=c.n_kvheads, head_dim=c.head_dim,
                            bias=c.attn_bias, window=0, scale=None, position=position),
            feed_forward=FeedForwardSpec("glu", dim=c.emb_dim, hidden=c.ffn_hidden, activation=c.activation_fn,
                                         bias=c.mlp_bias),
            mixer_norm=norm, feed_forward_norm=norm, arrangement="pre_norm",
            names=("ln", "attn", "ff_ln", "ff_sub_layer"),
        )
        return DecoderSpec(
            vocab_size=c.src_vocab_size, dim=c.emb_dim, layers=tuple(block for _ in range(c.nlayers)),
            schedule=tuple(LayerCall(i) for i in range(c.nlayers)), final_norm=norm, tie_head=c.tie_heads,
            max_positions=c.max_expected_seq_len,
            names=("base_model.embedding", "base_model.layers", "base_model.dec_norm", "head"),
        )

    def checkpoint_layout(self) -> List[TensorLayout]:
        """The tensors of an HF Llama checkpoint of this configuration."""
        c = self.config
        d, hd, h, kv, f = c.emb_dim, c.head_dim, c.nheads, c.n_kvheads, c.ffn_hidden
        out = [TensorLayout("model.embed_tokens.weight", (c.src_vocab_size, d), "embedding")]
        for i in range(c.nlayers):
            p = f"model.layers.{i}."
            out += [
                TensorLayout(p + "input_layernorm.weight", (d,), "gain"),
                TensorLayout(p + "self_attn.q_proj.weight", (h * hd, d), "matrix"),
                TensorLayout(p + "self_attn.k_proj.weight", (kv * hd, d), "matrix"),
                TensorLayout(p + "self_attn.v_proj.weight", (kv * hd, d), "matrix"),
                TensorLayout(p + "self_attn.o_proj.weight", (d, h * hd), "matrix"),
                TensorLayout(p + "post_attention_layernorm.weight", (d,), "gain"),
                TensorLayout(p + "mlp.gate_proj.weight", (f, d), "matrix"),
                TensorLayout(p + "mlp.up_proj.weight", (f, d), "matrix"),
                TensorLayout(p + "mlp.down_proj.weight", (d, f), "matrix"),
            ]
            if c.attn_bias:
                out += [TensorLayout(p + f"self_attn.{n}_proj.bias", (r,), "zeros")
                        for n, r in (("q", h * hd), ("k", kv * hd), ("v", kv * hd), ("o", d))]
            if c.mlp_bias:
                out += [TensorLayout(p + f"mlp.{n}_proj.bias", (r,), "zeros")
                        for n, r in (("gate", f), ("up", f), ("down", d))]
        out.append(TensorLayout("model.norm.weight", (d,), "gain"))
        if not c.tie_heads:
            out.append(TensorLayout("lm_head.weight", (c.src_vocab_size, d), "head"))
        return out


# ---- variants (fms/models/llama.py:456-561) ----------------------------------------------------------

_micro = LLaMAConfig(emb_dim=192, nheads=4, nlayers=5, max_expected_seq_len=1024, src_vocab_size=256)
_7b = LLaMAConfig()
_13b = LLaMAConfig(emb_dim=5120, nheads=40, nlayers=40)
_70b = LLaMAConfig(emb_dim=8192, nheads=64, kvheads=8, nlayers=80, hidden_grow_factor=28672 / 8192,
                   multiple_of=4096)
_8b_llama3 = LLaMAConfig(src_vocab_size=128256, emb_dim=4096, norm_eps=1e-5, nheads=32, kvheads=8, nlayers=32,
                         hidden_grow_factor=3.5, multiple_of=1024, max_expected_seq_len=8192, rope_theta=500_000.0)


# two tiny shapes for trying things out (a few layers, sizes that are no powers of two, grouped and single kv heads)
_tiny_a = LLaMAConfig(src_vocab_size=256, emb_dim=64, nheads=4, kvheads=2, nlayers=2, hidden_dim=176,
                      max_expected_seq_len=64)
_tiny_b = LLaMAConfig(src_vocab_size=384, emb_dim=96, nheads=3, kvheads=1, nlayers=3, hidden_dim=256, norm_eps=1e-6,
                      rope_theta=500_000.0, max_expected_seq_len=128, tie_heads=True)


def _factory(config: LLaMAConfig):
    def make(**kwargs) -> LLaMA:
        return LLaMA(config, **kwargs)

    return make


register_architecture("llama", LLaMA, config_json_names=("LlamaForCausalLM",))
for _name, _cfg in (("micro", _micro), ("7b", _7b), ("2-7b", _7b), ("13b", _13b), ("2-13b", _13b), ("70b", _70b),
                    ("2-70b", _70b), ("3-8b", _8b_llama3), ("tiny-a", _tiny_a), ("tiny-b", _tiny_b)):
    register_model("llama", _name, _factory(_cfg))


# ---- checkpoint adapter: HF names and layouts -> the engine's ----------------------------------------

_HF_TO_ENGINE = [  # fms/models/llama.py:649-663
    (r"^lm_head\.weight", "head.weight"),
    (r"^model\.embed_tokens\.weight", "base_model.embedding.weight"),
    (r"^model\.norm", "base_model.dec_norm"),
    (r"^model\.layers", "base_model.layers"),
    (r"self_attn\.k_proj", "attn.in_proj.key"),
    (r"self_attn\.v_proj", "attn.in_proj.value"),
    (r"self_attn\.q_proj", "attn.in_proj.query"),
    (r"self_attn\.o_proj", "attn.dense"),
    (r"mlp\.gate_proj", "ff_sub_layer.wg"),
    (r"mlp\.up_proj", "ff_sub_layer.w1"),
    (r"mlp\.down_proj", "ff_sub_layer.w2"),
    (r"input_layernorm", "ln"),
    (r"post_attention_layernorm", "ff_ln"),
]


def _hf_to_engine_names(tensors: Dict[str, torch.Tensor], config: LLaMAConfig = None, **_) -> Dict[str, torch.Tensor]:
    out = {}
    for name, t in tensors.items():
        if name.endswith("rotary_emb.inv_freq"):
            continue  # a table some exporters store; the frequencies are computed from the configuration
        if config is not None and config.tie_heads and name == "lm_head.weight":
            continue  # a tied head has no storage of its own (fms/models/llama.py:414-423)
        new = name
        for pattern, repl in _HF_TO_ENGINE:
            new = re.sub(pattern, repl, new)
        out[new] = t
    return out


_ROPE_ROWS = re.compile(r"attn\.in_proj\.(query|key)\.(weight|bias)$")


def _hf_rope_rows_to_interleaved(tensors: Dict[str, torch.Tensor], config: LLaMAConfig = None, **_):
    """HF keeps each head's rotary pairs as (first half, second half); the engine rotates adjacent
    pairs, so rows 0..hd/2-1 and hd/2..hd-1 of each head are interleaved
    (fms/models/llama.py:730-736)."""
    hd = config.head_dim
    out = {}
    for name, t in tensors.items():
        if _ROPE_ROWS.search(name) and t.shape[0] > 1:
            rows = t.shape[0]
            n = rows // hd
            if t.dim() == 2:
                t = t.view(n, 2, hd // 2, t.shape[1]).transpose(1, 2).reshape(rows, t.shape[1])
            else:
                t = t.view(n, 2, hd // 2).transpose(1, 2).reshape(rows)
        out[name] = t
    return out


def _fuse(tensors: Dict[str, torch.Tensor], parts: List[str], fused: str, **_) -> Dict[str, torch.Tensor]:
    """Concatenates rows of e.g. ``X.query.weight, X.key.weight, X.value.weight`` into ``X.qkv_fused.weight``
    where all parts are present; incomplete sets are left, so that the loader reports them."""
    out = dict(tensors)
    first = re.compile(re.escape(parts[0]) + r"\.(weight|bias)$")
    for name in list(tensors):
        m = first.search(name)
        if not m:
            continue
        names = [name[: m.start()] + p + "." + m.group(1) for p in parts]
        if all(n in out for n in names):
            pieces = [out.pop(n) for n in names]
            widest = max((p.dtype for p in pieces), key=lambda dt: torch.finfo(dt).bits if dt.is_floating_point else 0)
            out[name[: m.start()] + fused + "." + m.group(1)] = torch.cat([p.to(widest) for p in pieces], dim=0)
    return out


def _weight_fusion(tensors: Dict[str, torch.Tensor], **kw) -> Dict[str, torch.Tensor]:
    """[q; k; v] -> qkv_fused and [gate; up] -> wg1_fused, gate first
    (fms/utils/serialization.py:182-270; fms/modules/feedforward.py:291)."""
    out = _fuse(tensors, ["in_proj.query", "in_proj.key", "in_proj.value"], "in_proj.qkv_fused")
    return _fuse(out, ["ff_sub_layer.wg", "ff_sub_layer.w1"], "ff_sub_layer.wg1_fused")


_META_TO_ENGINE = [  # fms/models/llama.py:618-645: the names of Meta's own checkpoints
    (r"^tok_embeddings", "base_model.embedding"),
    (r"^norm", "base_model.dec_norm"),
    (r"^output", "head"),
    (r"^layers", "base_model.layers"),
    (r"\.attention\.", ".attn."),
    (r"attn\.wq", "attn.in_proj.query"),
    (r"attn\.wk", "attn.in_proj.key"),
    (r"attn\.wv", "attn.in_proj.value"),
    (r"attn\.wo", "attn.dense"),
    (r"attention_norm", "ln"),
    (r"feed_forward\.w1", "ff_sub_layer.wg"),
    (r"feed_forward\.w2", "ff_sub_layer.w2"),
    (r"feed_forward\.w3", "ff_sub_layer.w1"),
    (r"ffn_norm", "ff_ln"),
]


def _meta_to_engine_names(tensors: Dict[str, torch.Tensor], config: LLaMAConfig = None, **_) -> Dict[str, torch.Tensor]:
    """Meta's names; their q and k rows already lie as adjacent rotary pairs, so no rows are moved."""
    out = {}
    for name, t in tensors.items():
        if name == "rope.freqs":
            continue  # a table; the frequencies are computed from the configuration
        if config is not None and config.tie_heads and name == "output.weight":
            continue
        new = name
        for pattern, repl in _META_TO_ENGINE:
            new = re.sub(pattern, repl, new)
        out[new] = t
    return out


register_adapter_step("llama", "meta_to_fms_names", _meta_to_engine_names)
register_adapter_step("llama", "hf_to_fms_names", _hf_to_engine_names)
register_adapter_step("llama", "hf_to_fms_rope", _hf_rope_rows_to_interleaved)
register_adapter_step("llama", "weight_fusion", _weight_fusion)
register_adapter("llama", "hf", ["hf_to_fms_names", "hf_to_fms_rope", "weight_fusion"])
register_adapter("llama", "meta", ["meta_to_fms_names", "weight_fusion"])
register_adapter("llama", "fms", ["weight_fusion"])
