"""Position encodings: what happens to queries and keys on their way into the cache.

A mixer that attends over cached keys hands its position part the step's rows and its fused projection and gets
the queries back; in between the part applies the projection, encodes q and k for each row's position and writes
k and v into the cache.  So the mixer does not know what kind of encoding it has, and an encoding can keep the
fusion that suits it (the rotary part's decode path is ONE kernel: product, rotation and cache write).

Interface of a position encoding (what a mixer calls; the reference's ``PositionEncoder``,
fms/modules/positions.py:9-36, has ``adjusted_qk`` and ``adjusted_mask``):

    project(x, linear, batch, cache_view, nheads, kvheads, head_dim, writes_cache) -> q
        x [tokens, dim]; ``linear``: the mixer's fused projection (rows [q heads; k heads; v heads]).  Returns q
        [tokens, nheads * head_dim], encoded; k (encoded) and v lie in the cache afterwards, each row at its
        sequence's slot and place ``batch.positions``.  A row's position, for the encoding, is
        ``batch.position_ids`` where the batch has them, else ``batch.positions``.
    score_bias() -> None, or what an encoding adds to the attention scores.  The built-in attention kernels take no
        bias and the built-in mixer refuses an encoding that returns one; such an encoding comes with a mixer
        (and kernels) of its own.

``PositionEncoding`` is the base and encodes nothing.  ``RotaryEmbedding`` rotates adjacent pairs (2i, 2i+1) of
every head by the angle position * inv_f[i], inv_f[i] = 1 / theta^(2i / head_dim), all in float32
(fms/modules/positions.py:124-132 for the frequencies, :438-456 for the rotation); "llama3" rescales the
frequencies as fms/modules/positions.py:171-196 does.  The reference keeps a table of cos/sin per position; here
the kernel that writes keys into the cache computes them from the frequency vector, so no table exists and no
length limit comes from it.
"""
from __future__ import annotations

import math

import torch

from ..config.specs import PositionSpec
from ..kernels import ops
from .base import Part
from .registry import register_position


def rotary_inverse_frequencies(head_dim: int, theta: float, scaling: dict) -> torch.Tensor:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2)[: head_dim // 2].float() / head_dim))
    kind = scaling.get("rope_type", scaling.get("type", "regular")) if scaling else "regular"
    if kind in ("regular", "default", None):
        return inv
    if kind == "llama3":
        factor = float(scaling["factor"])
        low = float(scaling["low_freq_factor"])
        high = float(scaling["high_freq_factor"])
        old = float(scaling["original_max_position_embeddings"])
        wavelen = 2 * math.pi / inv
        slowed = torch.where(wavelen > old / low, inv / factor, inv)
        smooth = (old / wavelen - low) / (high - low)
        blended = (1 - smooth) * slowed / factor + smooth * slowed
        medium = ~(wavelen < old / high) * ~(wavelen > old / low)
        return torch.where(medium, blended, slowed)
    raise ValueError(f"rope scaling {kind!r} is not supported (supported: regular, llama3)")


class PositionEncoding(Part):
    """Encodes nothing: q and k go into attention as the projection gives them."""

    def __init__(self, spec: PositionSpec = None) -> None:
        super().__init__()
        self.spec = spec

    def project(self, x, linear, batch, cache_view, nheads: int, kvheads: int, head_dim: int, writes_cache: bool = True):
        return ops.qkv_rope_store(x, linear.tensor("weight"), linear.tensor("bias"), None, batch, cache_view, nheads,
                                  kvheads, head_dim, writes_cache)

    def score_bias(self):
        return None

    def kernel_libraries(self, dtype):
        return ["elementwise"]


_frequencies_on_device = {}  # (PositionSpec, device) -> float32 [head_dim / 2]; a few hundred bytes each


class RotaryEmbedding(PositionEncoding):
    def __init__(self, spec: PositionSpec) -> None:
        super().__init__(spec)
        if spec.head_dim % 2:
            raise ValueError("rotary embedding needs an even head size")
        self._inv_freq_host = rotary_inverse_frequencies(spec.head_dim, spec.theta, spec.scaling_dict())
        self._inv_freq = None

    def finalize(self, device, dtype) -> None:
        # one device tensor for all layers with the same frequencies: constants that nothing writes, and what a step's
        # layers share (the table of sines and cosines of many tokens) is kept by the tensor it was made from
        key = (self.spec, str(torch.device(device)))
        if key not in _frequencies_on_device:
            _frequencies_on_device[key] = self._inv_freq_host.to(device=device, dtype=torch.float32).contiguous()
        self._inv_freq = _frequencies_on_device[key]

    def rotary_frequencies(self):
        return self._inv_freq

    def project(self, x, linear, batch, cache_view, nheads: int, kvheads: int, head_dim: int, writes_cache: bool = True):
        """For a few bfloat16 rows one kernel (the weight-streaming product with rotation and cache write in its
        epilogue), else the product and the rotation-and-store kernel."""
        return ops.qkv_rope_store(x, linear.tensor("weight"), linear.tensor("bias"), self.rotary_frequencies(), batch,
                                  cache_view, nheads, kvheads, head_dim, writes_cache)


register_position("rope", RotaryEmbedding)
register_position("none", PositionEncoding)
