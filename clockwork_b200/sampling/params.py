"""Per-request sampling parameters, with the reference's names, defaults and meanings
(``clockwork/engine/sequence.py:28-41``)."""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class SamplingParams:
    max_tokens: int = 64
    temperature: float = 0.0  # 0 means greedy
    top_p: float = 1.0
    top_k: int = -1  # <= 0 or >= vocabulary: disabled
    stop: list[str] = field(default_factory=list)  # stop strings; need a tokenizer
    stop_token_ids: list[int] = field(default_factory=list)
    ignore_eos: bool = False
    seed: int | None = None  # None: the engine's model seed

    def __post_init__(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if self.temperature < 0:
            raise ValueError("temperature must be non-negative")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0
