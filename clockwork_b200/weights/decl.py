"""What a part says about each tensor it owns: checkpoint name, shape, what it is used as
(which decides the precision it is kept in) and how the random-weights mode draws it."""

from __future__ import annotations

from dataclasses import dataclass

# role -> how the tensor is kept on the device
#   "matrix": operand of a matrix product; kept in the run's compute dtype
#             (bfloat16 for a bfloat16 run, float32 for a float32 run)
#   "table":  embedding rows; kept like a matrix
#   "vector": norm weights and biases; always kept in float32 (exact for bfloat16 and
#             float32 storage alike), so a tensor stored in 32-bit stays 32-bit
#   "index":  integer tables; kept as int32
#   "state32": anything an architecture stores in 32-bit on purpose; kept in float32
ROLES = ("matrix", "table", "vector", "index", "state32")

# init -> distribution of the random-weights mode
#   "linear"/"bias"/"embedding": N(0, 0.02);  "norm": 1 + N(0, 0.1);  "zeros"; "index": arange
INITS = ("linear", "bias", "embedding", "norm", "zeros", "index")


@dataclass(frozen=True)
class TensorDecl:
    name: str
    shape: tuple[int, ...]
    role: str = "matrix"
    init: str = "linear"
    optional: bool = False  # may be absent from (or present in) the checkpoint without error

    def __post_init__(self) -> None:
        if self.role not in ROLES:
            raise ValueError(f"tensor {self.name!r}: unknown role {self.role!r}")
        if self.init not in INITS:
            raise ValueError(f"tensor {self.name!r}: unknown init {self.init!r}")
