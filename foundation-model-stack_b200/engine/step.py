"""The step function: a batch of sequences that start together, with unequal lengths; their prompts in
one step, then one token each.

``Engine.step`` runs only the tokens it is given, as one batch, against the cache that earlier steps
left, and returns float32 logits at the wanted places.  The reference's counterpart is
``LLaMA.forward(..., past_key_value_states, use_cache=True)`` (fms/models/llama.py:425-450) on a
left-padded rectangle with a mask; here rows are ragged, nothing is padded and causality is by position.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..cache.cache import Cache
from ..kernels import ops
from .batch import Batch


# Tests that replace the kernels by plain restatements clear this to drive the host logic on the CPU.
_REQUIRE_CUDA = True


class Engine:
    """A model's decoder together with a cache of a given size."""

    def __init__(self, model, max_tokens: int, max_slots: Optional[int] = None, sampling: bool = True) -> None:
        if model.decoder is None:
            raise ValueError("the model has no weights yet")
        self.model = model
        self.decoder = model.decoder
        self.device = model.device
        if _REQUIRE_CUDA and self.device.type != "cuda":
            raise RuntimeError(f"the engine runs on a CUDA device, not on {self.device}; there is no CPU path")
        self.vocab_size = self.decoder.spec.vocab_size
        if self.device.type == "cuda":
            self._compile_what_this_model_needs(sampling)
        self.cache = Cache(self.decoder.cache_requests(), max_tokens, self.decoder.spec.max_positions,
                           self.decoder.dtype, self.device, max_slots)

    def _compile_what_this_model_needs(self, sampling: bool) -> None:
        """Compiles, side by side, the kernel libraries this model will call and that are not built yet."""
        from ..kernels import build

        names = ["elementwise"]
        tensors = self.decoder.state_dict().values()
        if self.decoder.dtype == torch.float32 or any(t.dtype == torch.float32 and t.dim() == 2 for t in tensors):
            names.append("gemm_f32")
        for block in self.decoder.blocks:
            hd = getattr(block.mixer, "head_dim", None)
            if hd and getattr(block.mixer, "kvheads", None):
                names.append(f"attention_hd{hd}")
        if sampling:
            names.append("sampling")
        build.compile_many(names)

    # ---- sequences ---------------------------------------------------------------------------
    def begin(self, n: int) -> List[int]:
        """Slots for n sequences that start together."""
        return self.cache.begin(n)

    def release(self, slots: Sequence[int]) -> None:
        self.cache.release(slots)

    def length(self, slot: int) -> int:
        return self.cache.length[slot]

    # ---- one step ----------------------------------------------------------------------------
    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """Feeds ``tokens[i]`` to the sequence in ``slots[i]``.  ``want[i]`` lists the places among
        ``tokens[i]`` whose logits are returned (default: the last).  Returns [wanted, vocab] float32 on the
        device, in the order of the sequences and of ``want``."""
        if len(slots) != len(tokens) or not slots:
            raise ValueError("a step needs one token list per slot, and at least one")
        if want is None:
            want = [[len(t) - 1] for t in tokens]
        for t in tokens:
            for x in t:
                if not (0 <= int(x) < self.vocab_size):
                    raise ValueError(f"token id {x} outside the vocabulary of {self.vocab_size}")
        num_new = [len(t) for t in tokens]
        before = self.cache.prepare(slots, num_new)
        batch = Batch.from_lists(slots, before, tokens, want, self.device)
        logits = self.decoder.forward(batch, self.cache)
        self.cache.commit(slots, num_new)
        return logits

    def check(self) -> None:
        """Raises if a kernel met something the host should have prevented (synchronises)."""
        ops.check_error_flag(self.device)
