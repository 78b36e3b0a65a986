"""Typed descriptions of a decoder's layers: what an architecture's configuration is turned into, and
what the generic decoder is built from.

An architecture (``models/llama.py``) maps its configuration to one ``DecoderSpec``.  Every size and
constant of a part stands in its spec; no part looks at the architecture's configuration.  ``kind`` names
the implementation in the registries of ``fms_b200.parts``, so a spec with an unknown kind fails when
the model is built, not while it runs.  Layers may differ from one another (another mixer, another
feed-forward), and ``schedule`` is the order in which layers run: it may name a layer twice, and a call
may read another layer's cache instead of writing its own.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional, Tuple


@dataclasses.dataclass(frozen=True)
class NormSpec:
    kind: str  # "rmsnorm"
    dim: int
    eps: float
    options: Tuple[Tuple[str, Any], ...] = ()


@dataclasses.dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys inside a mixer."""

    kind: str  # "rope" | "none"
    head_dim: int = 0
    theta: float = 10000.0
    max_positions: int = 0
    scaling: Tuple[Tuple[str, Any], ...] = ()  # e.g. (("rope_type", "llama3"), ("factor", 8.0), ...)

    def scaling_dict(self) -> Dict[str, Any]:
        return dict(self.scaling)


@dataclasses.dataclass(frozen=True)
class MixerSpec:
    """The token mixer of a layer.  For ``kind == "attention"``: grouped-query softmax attention over the
    cache.  ``window`` 0 keeps all keys; W > 0 keeps, for the query at position p, keys p-W+1..p.
    ``scale`` None means 1/sqrt(head_dim).  Other kinds carry their sizes in ``options``."""

    kind: str
    dim: int
    nheads: int = 0
    kvheads: int = 0
    head_dim: int = 0
    bias: bool = False
    window: int = 0
    scale: Optional[float] = None
    position: PositionSpec = PositionSpec("none")
    options: Tuple[Tuple[str, Any], ...] = ()


@dataclasses.dataclass(frozen=True)
class FeedForwardSpec:
    """``kind == "glu"``: down(act(gate(x)) * up(x)) with fused [gate; up] rows."""

    kind: str
    dim: int
    hidden: int
    activation: str = "silu"
    bias: bool = False
    options: Tuple[Tuple[str, Any], ...] = ()


@dataclasses.dataclass(frozen=True)
class BlockSpec:
    """One layer: its norms, mixer and feed-forward and their arrangement, which names the block class in the
    registry (``fms_b200.parts.register_block``).  ``arrangement == "pre_norm"``:
    x += mixer(norm1(x)); x += feed_forward(norm2(x)).  The names are those under which the layer's
    parts appear in weight names (``ln``, ``attn``, ``ff_ln``, ``ff_sub_layer`` for Llama)."""

    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    mixer_norm: NormSpec
    feed_forward_norm: NormSpec
    arrangement: str = "pre_norm"
    names: Tuple[str, str, str, str] = ("ln", "attn", "ff_ln", "ff_sub_layer")
    options: Tuple[Tuple[str, Any], ...] = ()  # what another arrangement needs (a residual multiplier, ...)


@dataclasses.dataclass(frozen=True)
class LayerCall:
    """One entry of the schedule: run ``layer``; ``cache_of`` names the layer whose cache entry it uses
    (its own by default).  A call with ``writes_cache == False`` only reads that entry."""

    layer: int
    cache_of: Optional[int] = None
    writes_cache: bool = True

    @property
    def cache_layer(self) -> int:
        return self.layer if self.cache_of is None else self.cache_of


@dataclasses.dataclass(frozen=True)
class DecoderSpec:
    vocab_size: int
    dim: int
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[LayerCall, ...]
    final_norm: NormSpec
    tie_head: bool
    max_positions: int
    # prefixes of weight names: embedding, layer list, final norm, head
    names: Tuple[str, str, str, str] = ("base_model.embedding", "base_model.layers", "base_model.dec_norm", "head")
    embedding_scale: float = 1.0  # the embedded rows are multiplied by it as they enter the residual stream
    logit_scale: float = 1.0  # the logits are multiplied by it

    def __post_init__(self):
        n = len(self.layers)
        for call in self.schedule:
            if not (0 <= call.layer < n and 0 <= call.cache_layer < n):
                raise ValueError(f"schedule entry {call} names a layer outside 0..{n - 1}")
