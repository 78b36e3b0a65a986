"""The decoder: embedding, the scheduled layers, final norm, output head — built from a ``DecoderSpec``.

It knows no architecture.  ``forward(batch, cache)`` runs the tokens of one step through the layers in
the order of ``spec.schedule`` and returns float32 logits at the rows the batch asks for
(fms/models/llama.py:318-357 for the body, :425-450 for gather and head).
"""
from __future__ import annotations

import torch

from ..config.specs import DecoderSpec
from ..kernels import ops
from ..parts.base import Part
from ..parts import block as _blocks  # noqa: F401  (registers the built-in arrangement)
from ..parts.registry import build_block, build_norm


def _add_path(root: Part, path: str, part: Part) -> Part:
    names = path.split(".")
    node = root
    for n in names[:-1]:
        node = node._children[n] if n in node._children else node.add(n, Part())
    return node.add(names[-1], part)


class Decoder(Part):
    def __init__(self, spec: DecoderSpec, dtype: torch.dtype) -> None:
        super().__init__()
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute dtype {dtype} is not supported: bfloat16 and float32 are")
        self.spec = spec
        self.dtype = dtype
        emb_name, layers_name, norm_name, head_name = spec.names
        self.embedding = _add_path(self, emb_name, Part())
        self.embedding.declare("weight", (spec.vocab_size, spec.dim), role="matrix")
        layer_list = _add_path(self, layers_name, Part())
        self.blocks = [layer_list.add(str(i), build_block(b)) for i, b in enumerate(spec.layers)]
        self.final_norm = _add_path(self, norm_name, build_norm(spec.final_norm))
        self.head = _add_path(self, head_name, Part())
        if not spec.tie_head:
            self.head.declare("weight", (spec.vocab_size, spec.dim), role="matrix")
        self.device = None

    def cache_requests(self):
        """Per layer, what its mixer asks of the cache."""
        return [b.cache_request() for b in self.blocks]

    def finalize(self, device, dtype=None) -> None:
        self.device = torch.device(device)
        super().finalize(self.device, self.dtype)

    def kernel_libraries(self, dtype):
        head = ["gemm_f32"] if dtype == torch.float32 or self.head_weight().dtype == torch.float32 else \
            ["gemm_bf16_skinny", "gemm_bf16_tc"] + (["gemm_bf16_mid"] if ops.USE_MID_GEMM else [])
        return ["elementwise"] + head + super().kernel_libraries(dtype)

    def head_weight(self):
        return self.embedding.tensor("weight") if self.spec.tie_head else self.head.tensor("weight")

    def forward(self, batch, cache):
        if getattr(batch, "scratch", None) is not None:
            batch.scratch.clear()  # nothing of an earlier step with the same arrays (a decode step) is kept
        residual = ops.embed(self.embedding.tensor("weight"), batch.tokens, self.spec.embedding_scale)
        pending = None
        for call in self.spec.schedule:
            view = cache.layer_view(call.cache_layer)
            pending = self.blocks[call.layer].forward(residual, pending, batch, view, call.writes_cache, self.dtype)
        h = self.final_norm.apply(residual, pending, self.dtype, rows=batch.want_rows)
        logits = ops.linear(h, self.head_weight(), None, torch.float32)
        if self.spec.logit_scale != 1.0:
            logits.mul_(self.spec.logit_scale)
        return logits
