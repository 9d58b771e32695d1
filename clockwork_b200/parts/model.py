"""The decoder model: embedding, the layers in their run order, final norm, output head.

Reference: ``clockwork/engine/model.py:157-233`` (embedding, layer stack, final norm, logits
only at the requested rows, output head tied to the embedding when ``tie_word_embeddings``).
Built from a ``ModelSpec`` alone.  ``forward`` runs one flat batch of tokens (whatever mixture
of prompt portions and decoded tokens the step function assembled) and returns float32 logits
for the requested rows.
"""

from __future__ import annotations

import torch

from .. import ops
from ..config.model_spec import ModelSpec
from ..weights.decl import TensorDecl
from .base import PagedKVNeed, ResidualStream, SlotStateNeed, StepContext
from .linear import Linear
from .registry import build_block, build_part


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device) -> None:
        spec.validate()
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"run dtype must be float32 or bfloat16, got {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.blocks = [build_block(layer, dtype, self.device) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, spec.final_norm_prefix, dtype, self.device)
        self.embedding: torch.Tensor | None = None
        self.head: Linear | None = None

    # ---- what the cache manager needs to know -------------------------------------------
    def cache_needs(self) -> dict[int, PagedKVNeed | SlotStateNeed]:
        """Per cache layer (a layer some schedule entry writes): what its mixer keeps."""
        needs: dict[int, PagedKVNeed | SlotStateNeed] = {}
        for step in self.spec.schedule:
            need = self.blocks[step.layer].mixer.cache_need()
            if need is None:
                continue
            cache_layer = step.resolved_cache_layer()
            if step.write_cache:
                needs[cache_layer] = need
            elif needs.get(cache_layer) != need:
                raise ValueError(
                    f"layer {step.layer} reads cache layer {cache_layer}, whose contents have another shape"
                )
        return needs

    def graph_safe(self) -> bool:
        """Whether a step of this model may be captured in a CUDA graph."""
        return all(block.graph_safe for block in self.blocks) and self.final_norm.graph_safe

    def graph_safe_portions(self) -> bool:
        """Whether a step of this model that holds prompt portions may be captured in a CUDA graph."""
        return all(part.graph_safe_portions for part in self.all_parts())

    def all_parts(self):
        """Every part of every block, and the final norm."""
        for block in self.blocks:
            yield from block.parts()
        yield self.final_norm

    def step_scalars(self) -> dict:
        """The per-step device scalars that the model's parts declare (``Part.step_scalars``), by name."""
        scalars: dict = {}
        for part in self.all_parts():
            for name, rule in part.step_scalars().items():
                scalars.setdefault(name, rule)
        return scalars

    def step_arrays(self, max_tokens: int, max_seqs: int, page_size: int, max_portions: int | None = None,
                    max_ctx: int | None = None) -> dict:
        """The per-step device arrays that the model's parts declare (``Part.step_arrays``), by key."""
        arrays: dict = {}
        for part in self.all_parts():
            for key, decl in part.step_arrays(max_tokens, max_seqs, page_size, max_portions, max_ctx).items():
                arrays.setdefault(key, decl)
        return arrays

    def reserve_for_steps(self, max_seqs: int, max_ctx: int) -> None:
        for part in self.all_parts():
            part.reserve_for_steps(max_seqs, max_ctx)

    # ---- weights ---------------------------------------------------------------------------
    def tensor_decls(self) -> list[TensorDecl]:
        spec = self.spec
        decls = [TensorDecl(spec.embedding_name, (spec.vocab_size, spec.hidden_size), "table", "embedding")]
        for block in self.blocks:
            decls.extend(block.tensor_decls())
        decls.extend(self.final_norm.tensor_decls())
        # a tied model's checkpoint may omit the head (clockwork/engine/loader.py:57-62)
        decls.append(TensorDecl(spec.head_name, (spec.vocab_size, spec.hidden_size), "matrix", "linear",
                                optional=spec.tie_word_embeddings))
        return decls

    def load_weights(self, fetch) -> None:
        self.embedding = fetch(self.spec.embedding_name)
        for block in self.blocks:
            block.load_weights(fetch)
        self.final_norm.load_weights(fetch)
        self.head = Linear(self.embedding if self.spec.tie_word_embeddings else fetch(self.spec.head_name))

    def weight_bytes(self) -> int:
        """Bytes of distinct weight storage a step reads when every weight is used once."""
        seen: dict[int, int] = {}

        def visit(obj) -> None:
            if isinstance(obj, torch.Tensor):
                seen[obj.data_ptr()] = obj.numel() * obj.element_size()
            elif isinstance(obj, Linear):
                visit(obj.weight)
                visit(obj.bias)
            elif isinstance(obj, (list, tuple)):
                for o in obj:
                    visit(o)
            elif hasattr(obj, "__dict__") and not isinstance(obj, (ModelSpec, torch.dtype, torch.device)):
                for key, value in vars(obj).items():
                    if key in ("spec", "layer"):
                        continue
                    visit(value)

        visit(self.blocks)
        visit(self.final_norm)
        visit(self.head)
        return sum(seen.values())

    # ---- one step --------------------------------------------------------------------------
    def forward(self, ctx: StepContext, token_ids: torch.Tensor, logit_rows: torch.Tensor | None) -> torch.Tensor | None:
        """token_ids int32 [N]; logit_rows int32 [R] (rows of the flat batch whose logits are
        wanted).  Returns float32 [R, vocab], or None when no row is wanted."""
        # (kernels of a step read its inputs before they wait for their predecessors; when a kernel has
        # only just written those inputs, the first kernel here must not start before it has finished)
        stream = ResidualStream(ops.embed(self.embedding, token_ids, ctx.status, serial=ctx.inputs_from_device))
        schedule = self.spec.schedule
        for i, step in enumerate(schedule):
            view = ctx.views.get(step.resolved_cache_layer())
            if view is not None and hasattr(view, "write"):
                view.write = step.write_cache
            block = self.blocks[step.layer]
            # the norm that reads the residual next, for blocks that can fuse its first half into their
            # last product (the final norm reads selected rows only and is left alone)
            following = self.blocks[schedule[i + 1].layer].first_norm() if i + 1 < len(schedule) else None
            if following is not None:
                block.forward(ctx, stream, view, following_norm=following)
            else:
                block.forward(ctx, stream, view)
        if logit_rows is None or logit_rows.numel() == 0:
            stream.flush()
            return None
        x = self.final_norm.forward_rows(stream, logit_rows, ctx.status)
        return self.head.to_float32(x)


def tensor_decls_for_spec(spec: ModelSpec) -> list[TensorDecl]:
    """Declarations without building anything on a GPU (parts are built on the meta-free CPU
    path: no tensor is allocated until weights load)."""
    return DecoderModel(spec, torch.float32, "cpu").tensor_decls()


def build_model(spec: ModelSpec, dtype: torch.dtype, device) -> DecoderModel:
    return DecoderModel(spec, dtype, device)
