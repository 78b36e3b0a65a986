"""One layer: norms, mixer and feed-forward in their arrangement.

The residual stream is float32.  A sublayer's output is not added to it by the sublayer: it is handed to the
next norm, which adds it to the stream in the same pass that norms it.  So a block's ``forward`` takes the
pending output of the layer before and returns its own last sublayer's output, still pending.

Interface of a block (what the decoder calls); ``BlockSpec.arrangement`` names the class in the registry:

    cache_request() -> what its mixer asks of the cache (KVRequest | StateRequest | None)
    forward(residual, pending, batch, cache_view, writes_cache, dtype) -> pending
        residual [tokens, dim] float32, updated in place; pending [tokens, dim] in the compute dtype or None

``PreNormBlock`` ("pre_norm", fms/models/llama.py:118-167): x += mixer(norm(x)); x += feed_forward(norm(x)).
"""
from __future__ import annotations

from ..config.specs import BlockSpec
from .base import Part
from .registry import build_feed_forward, build_mixer, build_norm, register_block


class PreNormBlock(Part):
    def __init__(self, spec: BlockSpec) -> None:
        super().__init__()
        n_mixer_norm, n_mixer, n_ff_norm, n_ff = spec.names
        self.mixer_norm = self.add(n_mixer_norm, build_norm(spec.mixer_norm))
        self.mixer = self.add(n_mixer, build_mixer(spec.mixer))
        self.feed_forward_norm = self.add(n_ff_norm, build_norm(spec.feed_forward_norm))
        self.feed_forward = self.add(n_ff, build_feed_forward(spec.feed_forward))

    def cache_request(self):
        return self.mixer.cache_request()

    def forward(self, residual, pending, batch, cache_view, writes_cache, dtype):
        h = self.mixer_norm.apply(residual, pending, dtype)
        a = self.mixer.forward(h, batch, cache_view, writes_cache)
        h = self.feed_forward_norm.apply(residual, a, dtype)
        return self.feed_forward.forward(h)


Block = PreNormBlock  # the name under which earlier callers know it
register_block("pre_norm", PreNormBlock)
