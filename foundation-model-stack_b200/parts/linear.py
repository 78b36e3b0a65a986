"""A linear map y = x W^T (+ b) with W stored [out, in] as checkpoints store it
(the reference's ``get_linear`` default, fms/modules/linear.py:119-156)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part


class Linear(Part):
    def __init__(self, in_features: int, out_features: int, bias: bool = False) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.declare("weight", (out_features, in_features), role="matrix")
        if bias:
            self.declare("bias", (out_features,), role="vector")

    def forward(self, x, out_dtype=None):
        return ops.linear(x, self.tensor("weight"), self.tensor("bias"), out_dtype)

    def kernel_libraries(self, dtype):
        w = self.tensor("weight")
        if dtype == torch.float32 or (w is not None and w.dtype == torch.float32):
            return ["gemm_f32"]
        return ["gemm_bf16_skinny", "gemm_bf16_tc"] + (["gemm_bf16_mid"] if ops.USE_MID_GEMM else [])
