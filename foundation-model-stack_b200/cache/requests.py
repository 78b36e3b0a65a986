"""What a mixer asks of the cache.  Layers whose requests are equal share one group of storage."""
from __future__ import annotations

import dataclasses
from typing import Tuple

import torch


@dataclasses.dataclass(frozen=True)
class KVRequest:
    """Keys and values of every cached position (``window == 0``) or of the last ``window`` positions."""

    kvheads: int
    head_dim: int
    window: int = 0


@dataclasses.dataclass(frozen=True)
class StateRequest:
    """A tensor of fixed size per sequence, zero when the sequence starts.  ``dtype`` None means the
    model's compute dtype."""

    shape: Tuple[int, ...]
    dtype: object = None  # torch.dtype or None
    name: str = "state"
