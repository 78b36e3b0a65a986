"""Feed-forwards.  ``GatedLinearUnit``: y = W2 (act(Wg x) * (W1 x)) with the gate and up rows fused into
one matrix, gate first (fms/modules/feedforward.py:227-240 for the sizes, :288-297 for the formula).

Interface of a feed-forward (what a block calls):

    forward(x) -> y          x, y: [tokens, dim] in the compute dtype

A feed-forward with routing would implement the same call and keep router and experts inside.
"""
from __future__ import annotations

from ..config.specs import FeedForwardSpec
from ..kernels import ops
from .base import Part
from .linear import Linear
from .registry import register_feed_forward

ACTIVATIONS = {"silu": 0, "swish": 0, "gelu": 1, "gelu-tanh": 2, "gelu_pytorch_tanh": 2, "relu": 3}


class GatedLinearUnit(Part):
    def __init__(self, spec: FeedForwardSpec) -> None:
        super().__init__()
        act = spec.activation.lower()
        if act not in ACTIVATIONS:
            raise ValueError(f"activation {spec.activation!r} is not supported; supported: {sorted(ACTIVATIONS)}")
        self.activation = ACTIVATIONS[act]
        self.hidden = spec.hidden
        self.gate_up = self.add("wg1_fused", Linear(spec.dim, 2 * spec.hidden, spec.bias))
        self.down = self.add("w2", Linear(spec.hidden, spec.dim, spec.bias))

    def forward(self, x):
        h = ops.gated_linear(x, self.gate_up.tensor("weight"), self.gate_up.tensor("bias"), self.activation)
        return self.down.forward(h)

    def kernel_libraries(self, dtype):
        return super().kernel_libraries(dtype) + ["elementwise"]


register_feed_forward("glu", GatedLinearUnit)
