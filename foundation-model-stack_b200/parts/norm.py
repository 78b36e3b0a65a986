"""Norms.  ``RMSNorm``: y = gain * x * rsqrt(mean(x^2) + eps), statistics in float32, eps inside the
root, no mean subtraction, no bias — the reference's ``LayerNormParameterized`` as Llama configures it
(fms/modules/layernorm.py:56-69; fms/models/llama.py:72-87).

Interface of a norm (what a block and the decoder call):

    apply(residual, delta, out_dtype, rows=None) -> normed

``residual`` is the float32 residual stream ``[tokens, dim]``.  ``delta`` (or None) is the previous
sublayer's output, which the norm first adds to the stream in place, in float32: the residual sum and
the norm are one pass over the row.  With ``rows`` only those rows are normed and returned and the
stream is left as it is (used before the output head).
"""
from __future__ import annotations

from ..config.specs import NormSpec
from ..kernels import ops
from .base import Part
from .registry import register_norm


class RMSNorm(Part):
    def __init__(self, spec: NormSpec) -> None:
        super().__init__()
        self.dim = spec.dim
        self.eps = float(spec.eps)
        self.declare("weight", (spec.dim,), role="vector")

    def apply(self, residual, delta, out_dtype, rows=None):
        return ops.add_rmsnorm(residual, delta, self.tensor("weight"), self.eps, out_dtype, rows)

    def kernel_libraries(self, dtype):
        return ["elementwise"]


register_norm("rmsnorm", RMSNorm)
