"""Interfaces of the parts a layer is put together from, and what a step hands to them.

A *part* owns some named tensors and one piece of the layer's arithmetic.  Parts are built
from a ``PartSpec`` (kind + parameters); they never see the model's configuration and do not
know which model they are in.  The kinds:

* **Norm**      ``forward(stream) -> x``: adds the stream's pending delta into the float32
  residual, returns the normalised activations in the run's dtype.
* **PositionEncoding**  ``apply_and_store(ctx, qkv, view, ...)``: encodes positions into q and k
  and stores k, v into the cache view.
* **Mixer**     ``forward(ctx, x, view, stream) -> delta | None``: mixes tokens of a request
  (attention here).  It says what per-request memory it needs with ``cache_need()``: pages
  (``PagedKVNeed``), a fixed-size state slot (``SlotStateNeed``) or nothing.
* **FeedForward** ``forward(ctx, x, stream) -> delta | None``.
* **Block**     ``forward(ctx, stream, view)``: the arrangement of the above in one layer.

A mixer or feed-forward returns its contribution to the residual stream as a tensor in the
run's dtype (the next norm adds it), or ``None`` when it has already added it into
``stream.residual`` itself (a fused epilogue).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Iterable

import torch

from ..config.model_spec import PartSpec
from ..weights.decl import TensorDecl

Fetch = Callable[[str], torch.Tensor]


@dataclass(frozen=True)
class PagedKVNeed:
    """The mixer keeps keys and values per token, in pages.  ``window``: only the last
    ``window`` tokens are ever read (pages behind it can be given back); None: all."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class SlotStateNeed:
    """The mixer keeps a state of fixed size per request (``shape`` per layer), float32
    unless said otherwise.  It is zero when a request starts."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class PagedView:
    """One cache layer of a paged group as a step sees it."""

    k_cache: torch.Tensor  # [pages, page_size, kv_heads, head_dim]
    v_cache: torch.Tensor
    block_tables: torch.Tensor  # int32 [S, max_blocks] of this step's requests (-1: no page)
    slots: torch.Tensor  # int32 [N]: where each token's k/v go (page*page_size + offset)
    write: bool = True

    @property
    def page_size(self) -> int:
        return self.k_cache.shape[1]


@dataclass
class StateView:
    """One layer's fixed-size states: ``state[slots[s]]`` belongs to request ``s`` of the step."""

    state: torch.Tensor  # [num_slots + 1, *shape] (the last row: scratch for padding rows)
    slots: torch.Tensor  # int64 [S] on the device
    slots_host: list[int] = field(default_factory=list)  # the same on the host (empty in a captured step)


@dataclass
class StepContext:
    """Everything a part may ask about the step it runs in.  Tokens of all requests are one
    flat batch of ``num_tokens`` rows; request ``s`` owns rows ``q_start[s]:q_start[s+1]``."""

    dtype: torch.dtype
    device: torch.device
    status: torch.Tensor  # int32 status words that kernels report into
    num_tokens: int
    num_seqs: int
    positions: torch.Tensor  # int32 [N] absolute position of each token in its request
    tok_seq: torch.Tensor  # int32 [N] index of the token's request within this step (-1: padding)
    q_start: torch.Tensor  # int32 [S+1]
    ctx_lens: torch.Tensor  # int32 [S] tokens of the request that are in the cache after this step
    q_lens_host: list[int]   # per request: tokens it brings / tokens in the cache after the step, on the host; the
    ctx_lens_host: list[int]  # capture's placeholders in a captured step (empty in one that holds portions)
    max_q_len: int
    max_ctx_len: int
    views: dict[int, PagedView | StateView] = field(default_factory=dict)  # by cache layer
    inputs_from_device: bool = False  # a kernel launched just before the forward pass wrote the arrays above
    extras: dict = field(default_factory=dict)  # scratch that kernels share within a step

    @property
    def all_single_token(self) -> bool:
        return self.max_q_len <= 1


class ResidualStream:
    """The float32 residual [N, H] plus at most one contribution not yet added to it.

    A norm between two matrix products can be split over them (``ops.gemm.RowScaled``): the block
    names the norm that comes next in ``next_norm``; a product that adds into the residual may then
    begin that norm in its epilogue and leave the result in ``half_norm``; the norm hands it on to a
    consumer that can finish it, or ignores it.  Whoever changes the residual drops ``half_norm``."""

    def __init__(self, residual: torch.Tensor) -> None:
        self.residual = residual
        self.pending = None     # a tensor [N, H], or the ``ops.PartialSums`` of a product (for norms that take them)
        self.next_norm = None   # the Norm part that will read the residual next, if the block knows it
        self.half_norm = None   # (norm weight, x * weight in bfloat16, per-row partial sums of squares)

    def push(self, delta: torch.Tensor | None) -> None:
        if delta is None:
            return
        if self.pending is not None:
            self.flush()
        self.pending = delta
        self.half_norm = None

    def flush(self) -> None:
        if self.pending is not None:
            from .. import ops

            ops.add_to_residual(self.residual, self.pending)
            self.pending = None
            self.half_norm = None

    def residual_after_flush(self) -> torch.Tensor:
        """The float32 residual with nothing pending: what a fused epilogue adds into."""
        self.flush()
        self.half_norm = None  # the caller is about to change the residual
        return self.residual

    def norm_weight_to_begin(self) -> torch.Tensor | None:
        """The weight of the norm that follows, if that norm can be split over two products."""
        norm = self.next_norm
        return norm.split_weight() if norm is not None and hasattr(norm, "split_weight") else None


class Part:
    """Base of all parts: a name prefix for its tensors, declarations, and loading."""

    def __init__(self, spec: PartSpec, prefix: str, dtype: torch.dtype, device: torch.device) -> None:
        self.spec = spec
        self.prefix = prefix
        self.dtype = dtype
        self.device = device

    def name(self, suffix: str) -> str:
        return f"{self.prefix}.{suffix}" if self.prefix else suffix

    graph_safe = False  # True when, in a step in which every request brings one token, forward only launches
    # kernels on the current stream (no host reads of device data, no Python-side use of the step's
    # host-side lists, which hold the capture's placeholders): such a step may be captured in a CUDA graph

    def tensor_decls(self) -> Iterable[TensorDecl]:
        return ()

    def load_weights(self, fetch: Fetch) -> None:
        pass

    # ---- optional hooks for steps that are captured in CUDA graphs ------------------------------
    def step_scalars(self) -> dict[str, Callable[[int, int], int]]:
        """int32 values that the part's kernels read from device memory and that change from step to
        step: ``name -> f(live requests, longest live context)``.  A captured step keeps one word per
        name in its input buffer, refreshes it before every replay and hands the word's device view to
        the parts as ``ctx.extras[name]``; in an uncaptured step the name is absent and the part
        computes the value on the host.  Parts that want the same value use the same name."""
        return {}

    graph_safe_portions = False  # True when forward, in a step that holds prompt portions, also only launches
    # kernels on the current stream and takes what it needs about the portions from device memory (the
    # step's arrays and ``step_arrays`` below), never from the host-side lists: such a step may be captured too

    def step_arrays(self, max_tokens: int, max_seqs: int, page_size: int, max_portions: int | None = None,
                    max_ctx: int | None = None) -> dict:
        """int32 arrays that the part's kernels read from device memory in a step of prompt portions and
        that depend on how the step's tokens are divided among its requests: ``key -> (words,
        fill(q_lens, ctx_lens) -> numpy int32 [words], present(device view) -> object)``.  A captured
        step of up to ``max_tokens`` tokens of up to ``max_seqs`` requests with contexts up to ``max_ctx``
        (None: any), of which at most ``max_portions`` (None: all) bring more than one token, keeps ``words`` words per key
        in its input buffer, fills them before every replay and hands ``present(view)`` to the parts as
        ``ctx.extras[key]``; ``ctx.extras["captured_portions"]`` then holds ``{"singles": bool}``
        (whether the steps that replay this graph hold requests that bring a single token).  In an
        uncaptured step the key is absent and the part builds the array from the step's host-side
        lists."""
        return {}

    def reserve_for_steps(self, max_seqs: int, max_ctx: int) -> None:
        """Called once before steps are captured: set up whatever scratch memory a single-token step
        of up to ``max_seqs`` requests with contexts up to ``max_ctx`` needs, so that no buffer a
        captured graph points at is replaced later."""


class Norm(Part):
    def forward(self, stream: ResidualStream, status: torch.Tensor, lazy: bool = False):
        """The normalised activations.  ``lazy``: the consumer also takes an ``ops.gemm.RowScaled``."""
        raise NotImplementedError

    def forward_rows(self, stream: ResidualStream, rows: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
        """Normalised activations of the selected residual rows only."""
        raise NotImplementedError


class PositionEncoding(Part):
    pass


class Mixer(Part):
    takes_half_normed = False  # True: ``x`` may be an ``ops.gemm.RowScaled`` (it only feeds matrix products)

    def cache_need(self) -> PagedKVNeed | SlotStateNeed | None:
        return None

    def forward(self, ctx: StepContext, x: torch.Tensor, view, stream: ResidualStream) -> torch.Tensor | None:
        raise NotImplementedError


class FeedForward(Part):
    takes_half_normed = False

    def forward(self, ctx: StepContext, x: torch.Tensor, stream: ResidualStream) -> torch.Tensor | None:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer

    def forward(self, ctx: StepContext, stream: ResidualStream, view, following_norm=None) -> None:
        """``following_norm``: the norm that reads the residual after this block (the next block's
        first norm), when the model knows it; a hint for fusion, never needed for correctness."""
        raise NotImplementedError

    def first_norm(self):
        """The norm this block applies to the incoming residual first, or None."""
        return None

    def parts(self) -> tuple:
        """The parts the block is made of (for hooks that are collected over a whole model)."""
        return ()
