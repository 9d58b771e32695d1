"""Weights by tensor name: compare what the model declares with what the checkpoint holds,
report every difference in one error, then hand tensors to the parts in the precision their
role asks for.

The reference's rule (``clockwork/engine/loader.py:57-64``): Hugging Face names unchanged;
any missing or unexpected key is ``RuntimeError("state dict mismatch: missing=… unexpected=…")``
except a missing ``lm_head.weight`` of a tied model.  Added here: wrong shapes are listed in
the same error, and truncated files are reported by the reader.
"""

from __future__ import annotations

from pathlib import Path
from typing import Callable, Iterable

import torch

from .decl import TensorDecl
from .safetensors_io import CheckpointIndex


class WeightMismatchError(RuntimeError):
    """The checkpoint and the model disagree; ``missing``, ``unexpected`` and ``wrong_shape``
    hold the full lists."""

    def __init__(self, missing, unexpected, wrong_shape, where: str) -> None:
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        shapes = [f"{n}: checkpoint {list(got)} != model {list(want)}" for n, got, want in self.wrong_shape]
        super().__init__(
            f"state dict mismatch in {where}: missing={self.missing} "
            f"unexpected={self.unexpected} wrong_shape={shapes}"
        )


def check_declarations(decls: Iterable[TensorDecl], shapes: dict[str, tuple[int, ...]], where: str) -> None:
    """Raise one ``WeightMismatchError`` that lists everything that is wrong."""
    decls = list(decls)
    by_name = {d.name: d for d in decls}
    if len(by_name) != len(decls):
        seen, dup = set(), []
        for d in decls:
            if d.name in seen:
                dup.append(d.name)
            seen.add(d.name)
        raise ValueError(f"model declares tensors twice: {sorted(set(dup))}")
    missing = sorted(n for n, d in by_name.items() if n not in shapes and not d.optional)
    unexpected = sorted(n for n in shapes if n not in by_name)
    wrong = sorted(
        (n, tuple(shapes[n]), tuple(d.shape))
        for n, d in by_name.items()
        if n in shapes and not d.optional and tuple(shapes[n]) != tuple(d.shape)
    )
    if missing or unexpected or wrong:
        raise WeightMismatchError(missing, unexpected, wrong, where)


def kept_dtype(role: str, compute_dtype: torch.dtype) -> torch.dtype:
    if role in ("matrix", "table"):
        return compute_dtype
    if role == "index":
        return torch.int32
    return torch.float32  # "vector", "state32"


Fetch = Callable[[str], torch.Tensor]


def make_fetch(
    source: Callable[[str], torch.Tensor],
    decls: dict[str, TensorDecl],
    compute_dtype: torch.dtype,
    device: torch.device | str,
) -> Fetch:
    """``fetch(name)`` returns the named tensor on ``device`` in the dtype its role keeps."""

    def fetch(name: str) -> torch.Tensor:
        decl = decls[name]
        t = source(name)
        return t.to(device=device, dtype=kept_dtype(decl.role, compute_dtype)).contiguous()

    return fetch


def load_checkpoint_into(model, model_dir: str | Path) -> None:
    """Check and load ``model_dir``'s safetensors into ``model`` (a ``DecoderModel``)."""
    index = CheckpointIndex(model_dir)
    try:
        decls = {d.name: d for d in model.tensor_decls()}
        check_declarations(decls.values(), {n: index.shape(n) for n in index.names()}, str(model_dir))
        model.load_weights(make_fetch(index.tensor, decls, model.dtype, model.device))
    finally:
        index.close()
