"""RMSNorm over the float32 residual stream, fused with the pending residual add.

Reference: ``clockwork/engine/model.py:38-49`` (float32 statistics, ``x * rsqrt(mean(x^2) +
eps)``, then the weight) and ``:150``/``:154`` (the residual sums the norm kernel absorbs).
Parameters: ``size``, ``eps``.  Tensor: ``<prefix>.weight`` [size], kept in float32.
"""

from __future__ import annotations

import torch

from .. import ops
from ..ops.gemm import RowScaled
from ..weights.decl import TensorDecl
from .base import Norm, ResidualStream
from .registry import register_norm


class RMSNorm(Norm):
    graph_safe = True
    graph_safe_portions = True
    takes_partial_sums = True  # ``forward`` hands whatever the stream holds to ``ops.add_rmsnorm``, slabs included

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight: torch.Tensor | None = None

    def tensor_decls(self):
        yield TensorDecl(self.name("weight"), (self.size,), role="vector", init="norm")

    def load_weights(self, fetch) -> None:
        self.weight = fetch(self.name("weight"))

    def split_weight(self) -> torch.Tensor | None:
        """The weight a preceding product multiplies into the residual when it begins this norm."""
        return self.weight if self.dtype == torch.bfloat16 else None

    def forward(self, stream: ResidualStream, status: torch.Tensor, lazy: bool = False):
        half, stream.half_norm = stream.half_norm, None
        if lazy and half is not None and stream.pending is None and half[0] is self.weight:
            # the product that wrote the residual began this norm; the product that reads it finishes it
            residual, weight, eps, dtype = stream.residual, self.weight, self.eps, self.dtype
            return RowScaled(half[1], half[2], eps, self.size,
                             lambda: ops.add_rmsnorm(residual, None, weight, eps, dtype, status))
        delta, stream.pending = stream.pending, None
        return ops.add_rmsnorm(stream.residual, delta, self.weight, self.eps, self.dtype, status)

    def forward_rows(self, stream: ResidualStream, rows: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
        stream.flush()
        return ops.rmsnorm_rows(stream.residual, rows, self.weight, self.eps, self.dtype, status)


register_norm("rmsnorm", RMSNorm, replace=True)
