"""Where checkpoint tensors come from: files, or a seeded random generator.

A source answers, by checkpoint tensor name, ``spec(name) -> (dtype, shape)`` and ``get(name) -> tensor``.
The loader needs no more, so a model with random weights goes through the same adapter and the same
checks as one read from disk.
"""
from __future__ import annotations

import hashlib
import math
from typing import Dict, List, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsFile, find_checkpoint_files


class FileSource:
    def __init__(self, model_path: str) -> None:
        self.files = [SafetensorsFile(p) for p in find_checkpoint_files(model_path)]
        self._where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for k in f.keys():
                self._where.setdefault(k, f)

    def keys(self) -> List[str]:
        return list(self._where)

    def spec(self, name: str):
        return self._where[name].spec(name)

    def get(self, name: str) -> torch.Tensor:
        return self._where[name].get(name)


class TensorLayout:
    """One checkpoint tensor of an architecture: its name, shape and how random weights fill it."""

    __slots__ = ("name", "shape", "init")

    def __init__(self, name: str, shape: Sequence[int], init: str) -> None:
        self.name = name
        self.shape = tuple(shape)
        # "matrix", "embedding", "head": N(0, std)   "gain": 1 + U(-0.1, 0.1)   "zeros"; the reference's own
        # initialisation (RandomSource(init="fms")) tells the three kinds of matrices apart
        self.init = init


class RandomSource:
    """Seeded random weights: matrices and embeddings ~ N(0, 0.02), norm gains 1 + U(-0.1, 0.1).  Each
    tensor has a generator of its own, seeded by (seed, name), so values do not depend on the order in
    which tensors are asked for.  The same seed gives the same values on the same kind of device."""

    def __init__(self, layout: Sequence[TensorLayout], seed: int, dtype: torch.dtype = torch.bfloat16,
                 device="cpu", std: float = 0.02, gain_dtype: torch.dtype = None, init: str = "baseline") -> None:
        """``init="fms"``: as the reference initialises a fresh model — linear layers trunc_normal(0, 0.02) cut at
        +-2 (fms/modules/attention.py:689-692, fms/modules/feedforward.py:269-283), the embedding
        trunc_normal(std = width^-0.5) (fms/models/llama.py:231-235), the head N(0, (width * vocabulary)^-0.25)
        (fms/models/llama.py:387-393), gains 1 (fms/modules/layernorm.py:50-54)."""
        if init not in ("baseline", "fms"):
            raise ValueError(f'init {init!r}: "baseline" or "fms"')
        self.init = init
        self.layout = {t.name: t for t in layout}
        self.seed = int(seed)
        self.dtype = dtype
        self.gain_dtype = gain_dtype or dtype
        self.device = torch.device(device)
        self.std = std

    def keys(self) -> List[str]:
        return list(self.layout)

    def spec(self, name: str):
        t = self.layout[name]
        return (self.gain_dtype if t.init == "gain" else self.dtype), t.shape

    def get(self, name: str) -> torch.Tensor:
        t = self.layout[name]
        digest = hashlib.sha256(f"{self.seed}:{name}".encode()).digest()
        g = torch.Generator(device=self.device)
        g.manual_seed(int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF)
        if t.init in ("matrix", "embedding", "head"):
            x = torch.empty(t.shape, dtype=torch.float32, device=self.device)
            if self.init == "fms" and t.init == "head":
                x.normal_(0.0, 1.0 / math.sqrt(math.sqrt(t.shape[0] * t.shape[1])), generator=g)
            elif self.init == "fms":
                std = t.shape[1] ** -0.5 if t.init == "embedding" else 0.02
                torch.nn.init.trunc_normal_(x, mean=0.0, std=std, a=-2.0, b=2.0, generator=g)
            else:
                x.normal_(0.0, self.std, generator=g)
            return x.to(self.dtype)
        if t.init == "gain":
            if self.init == "fms":
                return torch.ones(t.shape, dtype=self.gain_dtype, device=self.device)
            x = torch.empty(t.shape, dtype=torch.float32, device=self.device).uniform_(-0.1, 0.1, generator=g)
            return (1.0 + x).to(self.gain_dtype)
        if t.init == "zeros":
            return torch.zeros(t.shape, dtype=self.dtype, device=self.device)
        raise ValueError(f"unknown init {t.init!r}")
