"""A weight matrix in ``nn.Linear`` layout ([out, in], optional float32 bias) and the matrix
products the parts need from it.  In a float32 run every product is the plain CUDA-core kernel
(true float32).  In a bfloat16 run products go to the tensor-core kernel when it takes the
sizes, else to the same plain kernel with bfloat16 operands."""

from __future__ import annotations

import torch

from .. import ops
from ..ops import gemm as gemm_ops


class Linear:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None) -> None:
        self.weight = weight
        self.bias = bias
        self.out_features, self.in_features = weight.shape

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        """x [M, K] -> [M, N] in x's dtype."""
        return gemm_ops.linear(x, self.weight, self.bias)

    def add_into(self, x: torch.Tensor, residual: torch.Tensor, stream=None) -> None:
        """residual (float32 [M, N]) += x W^T (+ bias), the sum done in float32.  With the residual
        stream given, the product also begins the norm that the stream says comes next, when it can."""
        begin = stream.norm_weight_to_begin() if stream is not None else None
        half = gemm_ops.linear_add_into(x, self.weight, self.bias, residual, begin_norm=begin)
        if stream is not None:
            stream.half_norm = None if half is None else (begin, *half)

    def add_or_defer(self, x: torch.Tensor, stream):
        """The product's contribution to the residual stream: added into the residual here (returns None),
        or, when the product is better split with its splits kept apart and the norm that reads the
        residual next can add them up, returned as ``ops.PartialSums`` for the stream to hold."""
        norm = stream.next_norm
        if self.bias is None and norm is not None and getattr(norm, "takes_partial_sums", False):
            parts = gemm_ops.linear_partial_sums(x, self.weight)
            if parts is not None:
                return parts
        self.add_into(x, stream.residual_after_flush(), stream)
        return None

    def to_float32(self, x: torch.Tensor) -> torch.Tensor:
        """x W^T as float32 (logits)."""
        return gemm_ops.linear_f32(x, self.weight, self.bias)
