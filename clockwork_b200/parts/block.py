"""Pre-norm residual block: ``h += mixer(norm1(h)); h += ffn(norm2(h))``.

Reference: ``clockwork/engine/model.py:131-154``.  The block owns the arrangement only; its
mixer, feed-forward and norms are whatever the layer's spec names.  Tensor prefixes follow the
Hugging Face layout: ``<layer>.self_attn``, ``<layer>.mlp``, ``<layer>.input_layernorm``,
``<layer>.post_attention_layernorm``.
"""

from __future__ import annotations

from ..config.model_spec import LayerSpec
from .base import Block, ResidualStream, StepContext
from .registry import build_part, register_block


class PreNormResidualBlock(Block):
    def __init__(self, layer: LayerSpec, dtype, device) -> None:
        self.layer = layer
        self.prefix = layer.prefix
        self.dtype, self.device = dtype, device
        self.mixer_norm = build_part("norm", layer.mixer_norm, f"{layer.prefix}.input_layernorm", dtype, device)
        self.mixer = build_part("mixer", layer.mixer, f"{layer.prefix}.self_attn", dtype, device)
        self.ffn_norm = build_part("norm", layer.ffn_norm, f"{layer.prefix}.post_attention_layernorm", dtype, device)
        self.ffn = build_part("ffn", layer.ffn, f"{layer.prefix}.mlp", dtype, device)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for part in self.parts())

    def tensor_decls(self):
        for part in self.parts():
            yield from part.tensor_decls()

    def load_weights(self, fetch) -> None:
        for part in self.parts():
            part.load_weights(fetch)

    def first_norm(self):
        return self.mixer_norm

    @staticmethod
    def _normed(norm, consumer, stream: ResidualStream, status):
        if getattr(consumer, "takes_half_normed", False) and hasattr(norm, "split_weight"):
            return norm.forward(stream, status, lazy=True)
        return norm.forward(stream, status)

    def forward(self, ctx: StepContext, stream: ResidualStream, view, following_norm=None) -> None:
        x = self._normed(self.mixer_norm, self.mixer, stream, ctx.status)
        stream.next_norm = self.ffn_norm  # what the mixer's output product may begin
        stream.push(self.mixer.forward(ctx, x, view, stream))
        x = self._normed(self.ffn_norm, self.ffn, stream, ctx.status)
        stream.next_norm = following_norm
        stream.push(self.ffn.forward(ctx, x, stream))
        stream.next_norm = None


register_block("prenorm_residual", PreNormResidualBlock, replace=True)
