"""What an architecture is to the rest of the library.

An architecture subclasses ``Model`` and says four things: how its ``config.json`` becomes its typed
configuration, what layers that configuration means (a ``DecoderSpec``), which tensors its checkpoints
hold (for random weights and for checks), and — through the adapter registry of ``fms_b200.weights`` —
how checkpoint names map to the engine's.  Everything else (loading, cache, stepping, generation) is
shared.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config.specs import DecoderSpec
from ..weights.loader import load_weights
from ..weights.sources import TensorLayout


class Model:
    architecture = ""
    default_source = "hf"

    def __init__(self, config) -> None:
        self.config = config
        self.decoder = None
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None
        self._engine = None

    # ---- what an architecture provides -------------------------------------------------------
    @classmethod
    def config_from_json(cls, values: dict):
        raise NotImplementedError

    def config_json(self) -> dict:
        raise NotImplementedError

    def decoder_spec(self) -> DecoderSpec:
        raise NotImplementedError

    def checkpoint_layout(self) -> List[TensorLayout]:
        raise NotImplementedError

    # ---- shared ------------------------------------------------------------------------------
    def load(self, source, adapter_source: Optional[str], device, dtype: torch.dtype) -> "Model":
        from ..engine.decoder import Decoder

        self.dtype = dtype
        self.device = torch.device(device)
        self.decoder = Decoder(self.decoder_spec(), dtype)
        load_weights(self.decoder, source, self.architecture, adapter_source or self.default_source, self.device,
                     dtype, config=self.config)
        return self

    def state_dict(self):
        return self.decoder.state_dict()

    def new_engine(self, max_tokens: int, max_slots: Optional[int] = None, sampling: bool = True, **engine_options):
        """``engine_options``: further keyword arguments of ``Engine`` (``use_graphs``, ``max_graphs``)."""
        from ..engine.step import Engine

        return Engine(self, max_tokens=max_tokens, max_slots=max_slots, sampling=sampling, **engine_options)

    def cache_bytes_per_token(self) -> int:
        """Bytes of cache that one token of one sequence takes over all layers (keys and values of every layer whose
        mixer keeps them; a windowed layer counts like any other: every group of the cache is given the same number of
        blocks)."""
        from ..cache.requests import KVRequest

        itemsize = 4 if self.dtype == torch.float32 else 2
        return sum(2 * r.kvheads * r.head_dim * itemsize for r in self.decoder.cache_requests() if isinstance(r, KVRequest))

    def engine(self, min_tokens: int = 0, min_slots: int = 0):
        """The model's own engine, made on first use and made anew when it is too small."""
        e = self._engine
        if e is None or e.cache.n_blocks * 64 < min_tokens or e.cache.max_slots < min_slots:
            if e is not None and e.cache.slots.n_held:
                raise RuntimeError("the engine is too small for this call and sequences are still live in it")
            self._engine = None
            del e
            self._engine = self.new_engine(max(min_tokens, 64), max(min_slots, 1))
        return self._engine

    # ---- whole sequences in, logits out: the reference's ``model(x)`` ------------------------------
    def forward(self, x, last_n_tokens: int = 0, use_cache: bool = False, **kwargs):
        """Float32 logits of whole sequences, nothing kept afterwards (fms/models/llama.py:425-450).

        x: token ids [S], [B, S] (a tensor) or a list of sequences of any lengths.  last_n_tokens: 0 for every
        position, n for the last n of each sequence, as the reference's parameter of the same name.  Returns
        [S', V], [B, S', V] or a list of [S'_i, V].  Stepping with a cache is ``new_engine(...).step`` (or
        ``generate``), not this call: use_cache and the reference's other keywords are refused."""
        if use_cache or any(v is not None for v in kwargs.values()):
            raise NotImplementedError("model(x) scores whole sequences; to step with the cache use Engine.step or generate")
        if isinstance(x, torch.Tensor):
            if x.dim() not in (1, 2):
                raise ValueError("x must be [S] or [B, S]")
            seqs = [x.tolist()] if x.dim() == 1 else [row.tolist() for row in x]
        else:
            seqs = [[int(t) for t in s] for s in x]
        if not seqs or any(len(s) == 0 for s in seqs):
            raise ValueError("every sequence needs at least one token")
        want = [list(range(len(s) - last_n_tokens if 0 < last_n_tokens < len(s) else 0, len(s))) for s in seqs]
        engine = self.engine(min_tokens=sum((len(s) + 63) // 64 * 64 for s in seqs), min_slots=len(seqs))
        slots = engine.begin(len(seqs))
        try:
            logits = engine.step(slots, seqs, want)
        finally:
            engine.release(slots)
        parts = list(torch.split(logits, [len(w) for w in want]))
        if isinstance(x, torch.Tensor):
            return parts[0] if x.dim() == 1 else torch.stack(parts)
        return parts

    __call__ = forward
