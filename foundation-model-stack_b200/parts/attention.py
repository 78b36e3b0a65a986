"""Grouped-query softmax attention over the cache: the reference's ``MultiHeadAttention`` with fused
QKV (fms/modules/attention.py:707-943, :622-704).

    qkv = x Wqkv^T (+ b), rows [q heads; k heads; v heads]          attention.py:653-657, :704
    q, k rotated by the position encoding, before caching           attention.py:878-881
    k, v written at each token's position into its slot's blocks    (reference: torch.cat, :186-212)
    o = softmax(q k^T * scale, causal by position, window) v        attention.py:215-294
    y = o Wdense^T (+ b)                                            attention.py:937

Query head h uses key/value head h // (nheads / kvheads).  A token at position p sees the cached
positions p-window+1..p (all of 0..p without a window), whatever else is in the batch and however the
sequence was cut into steps.

Interface of a mixer (what a block calls):

    cache_request() -> KVRequest | StateRequest | None
    forward(x, batch, cache_view, writes_cache) -> y       x, y: [tokens, dim] in the compute dtype
"""
from __future__ import annotations

import math

from ..cache.requests import KVRequest
from ..config.specs import MixerSpec
from ..kernels import ops
from .base import Part
from .linear import Linear
from .registry import build_position, register_mixer


class MultiHeadAttention(Part):
    def __init__(self, spec: MixerSpec) -> None:
        super().__init__()
        if spec.nheads <= 0 or spec.kvheads <= 0 or spec.nheads % spec.kvheads:
            raise ValueError(f"nheads {spec.nheads} must be a positive multiple of kvheads {spec.kvheads}")
        if spec.head_dim <= 0 or spec.head_dim % 16 or spec.head_dim > 256:
            raise ValueError(f"head size {spec.head_dim} is not supported: a multiple of 16 up to 256 is")
        self.spec = spec
        self.nheads, self.kvheads, self.head_dim = spec.nheads, spec.kvheads, spec.head_dim
        self.scale = 1.0 / math.sqrt(spec.head_dim) if spec.scale is None else float(spec.scale)
        self.window = int(spec.window)
        qkv_rows = (spec.nheads + 2 * spec.kvheads) * spec.head_dim
        in_proj = self.add("in_proj", Part())
        self.qkv = in_proj.add("qkv_fused", Linear(spec.dim, qkv_rows, spec.bias))
        self.dense = self.add("dense", Linear(spec.nheads * spec.head_dim, spec.dim, spec.bias))
        # not a child: the encoding has no checkpoint tensors of its own and may be shared
        self.position = build_position(spec.position)
        if self.position.score_bias() is not None:
            raise ValueError(f"position encoding {spec.position.kind!r} adds to the attention scores; the attention "
                             "kernels of this mixer take no such term")

    def finalize(self, device, dtype) -> None:
        super().finalize(device, dtype)
        self.position.finalize(device, dtype)

    def cache_request(self):
        return KVRequest(self.kvheads, self.head_dim, self.window)

    def forward(self, x, batch, cache_view, writes_cache: bool = True):
        # the position part applies the projection, encodes q and k and writes k and v into the cache
        q = self.position.project(x, self.qkv, batch, cache_view, self.nheads, self.kvheads, self.head_dim, writes_cache)
        o = ops.attention(q, batch, cache_view, self.nheads, self.kvheads, self.head_dim, self.scale, self.window)
        return self.dense.forward(o)

    def kernel_libraries(self, dtype):
        return (super().kernel_libraries(dtype) + self.position.kernel_libraries(dtype)
                + ["elementwise", f"attention_hd{self.head_dim}"])


register_mixer("attention", MultiHeadAttention)
