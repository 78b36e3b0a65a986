"""Choosing the next token: greedy, or temperature sampling with an optional top-k cut — what the
reference's ``generate`` samples with (fms/utils/generation.py:316-328).

Greedy takes the largest logit, the lowest index among equals.  Sampling divides the logits by the
temperature, drops everything below the k-th largest value when ``top_k`` > 0, takes the softmax in
float32 and draws once.  The draw of request r at step s uses the uniform number hash(seed, r, s), so a
request's tokens do not depend on its batch (the reference draws from torch's global generator).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops


class Sampler:
    def __init__(self, do_sample: bool = True, temperature: float = 1.0, top_k: int = 10, seed: int = 0) -> None:
        if do_sample and not temperature > 0:
            raise ValueError(f"temperature must be positive, not {temperature}")
        if top_k < 0:
            raise ValueError(f"top_k must not be negative, not {top_k}")
        self.do_sample = bool(do_sample)
        self.temperature = float(temperature)
        self.top_k = int(top_k)
        self.seed = int(seed)

    def __call__(self, logits: torch.Tensor, requests: torch.Tensor, step: int,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits [rows, vocab] float32; requests [rows] int32 (each row's request number); returns int32
        token ids [rows] on the device."""
        if not self.do_sample:
            return ops.argmax(logits, out)
        return ops.sample(logits, self.temperature, self.top_k, self.seed, requests, step, out)
