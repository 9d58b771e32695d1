"""SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))``, no biases.

Reference: ``clockwork/engine/model.py:52-63``.  Parameters: ``hidden_size, intermediate_size``.
Tensors: ``gate_proj.weight`` [I, H], ``up_proj.weight`` [I, H], ``down_proj.weight`` [H, I].
The gate and up products and the activation run as one kernel; the down product adds into the
float32 residual.
"""

from __future__ import annotations

from ..ops import gemm as gemm_ops
from ..weights.decl import TensorDecl
from .base import FeedForward, ResidualStream, StepContext
from .linear import Linear
from .registry import register_ffn


class SwiGLU(FeedForward):
    graph_safe = True
    graph_safe_portions = True
    takes_half_normed = True  # x only feeds the gate/up product

    def __init__(self, spec, prefix, dtype, device) -> None:
        super().__init__(spec, prefix, dtype, device)
        self.hidden_size = int(spec["hidden_size"])
        self.intermediate_size = int(spec["intermediate_size"])
        self.w_gate = self.w_up = None
        self.down: Linear | None = None

    def tensor_decls(self):
        h, i = self.hidden_size, self.intermediate_size
        yield TensorDecl(self.name("gate_proj.weight"), (i, h), "matrix", "linear")
        yield TensorDecl(self.name("up_proj.weight"), (i, h), "matrix", "linear")
        yield TensorDecl(self.name("down_proj.weight"), (h, i), "matrix", "linear")

    def load_weights(self, fetch) -> None:
        self.w_gate = fetch(self.name("gate_proj.weight"))
        self.w_up = fetch(self.name("up_proj.weight"))
        self.down = Linear(fetch(self.name("down_proj.weight")))

    def forward(self, ctx: StepContext, x, stream: ResidualStream):
        act = gemm_ops.swiglu(x, self.w_gate, self.w_up)
        return self.down.add_or_defer(act, stream)


register_ffn("swiglu", SwiGLU, replace=True)
