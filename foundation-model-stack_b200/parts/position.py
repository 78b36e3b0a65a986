"""Position encodings applied to queries and keys inside a mixer.

``RotaryEmbedding`` rotates adjacent pairs (2i, 2i+1) of every head by the angle position * inv_f[i],
inv_f[i] = 1 / theta^(2i / head_dim), all in float32 (fms/modules/positions.py:124-132 for the
frequencies, :438-456 for the rotation); "llama3" rescales the frequencies as
fms/modules/positions.py:171-196 does.  The reference keeps a table of cos/sin per position; here the
kernel that writes keys into the cache computes them from the frequency vector, so no table exists and
no length limit comes from it.

Interface of a position encoding (what a mixer calls):

    rotary_frequencies() -> float32 tensor [head_dim / 2] or None

None means that queries and keys are left as they are.  An encoding that is not a rotation of pairs
would add a method of its own and a mixer that knows it.
"""
from __future__ import annotations

import math

import torch

from ..config.specs import PositionSpec
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


class RotaryEmbedding(Part):
    def __init__(self, spec: PositionSpec) -> None:
        super().__init__()
        if spec.head_dim % 2:
            raise ValueError("rotary embedding needs an even head size")
        self.spec = spec
        self._inv_freq_host = rotary_inverse_frequencies(spec.head_dim, spec.theta, spec.scaling_dict())
        self._inv_freq = None

    def finalize(self, device, dtype) -> None:
        self._inv_freq = self._inv_freq_host.to(device=device, dtype=torch.float32).contiguous()

    def rotary_frequencies(self):
        return self._inv_freq


class NoPosition(Part):
    def __init__(self, spec: PositionSpec) -> None:
        super().__init__()

    def rotary_frequencies(self):
        return None


register_position("rope", RotaryEmbedding)
register_position("none", NoPosition)
