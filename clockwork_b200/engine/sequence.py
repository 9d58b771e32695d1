"""Per-request state shared by the scheduler and the engine.

Same fields and meanings as the reference's ``clockwork/engine/sequence.py:10-96``; the block
table lives in the cache manager (``clockwork_b200/cache/manager.py``) instead of here.
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from enum import Enum

from ..sampling.params import SamplingParams


class SequenceStatus(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    PREEMPTED = "preempted"
    FINISHED_STOPPED = "finished_stopped"
    FINISHED_LENGTH = "finished_length"
    FINISHED_ABORTED = "finished_aborted"


_FINISHED = frozenset(
    {SequenceStatus.FINISHED_STOPPED, SequenceStatus.FINISHED_LENGTH, SequenceStatus.FINISHED_ABORTED}
)


class Sequence:
    """One request's tokens and its progress through the cache."""

    def __init__(self, seq_id: str, prompt_token_ids: list[int], sampling_params: SamplingParams | None = None,
                 arrival_time: float | None = None) -> None:
        self.seq_id = seq_id
        self.prompt_token_ids = list(prompt_token_ids)
        self.output_token_ids: list[int] = []
        self.sampling_params = sampling_params if sampling_params is not None else SamplingParams()
        self.status = SequenceStatus.WAITING
        self.num_computed_tokens = 0  # tokens whose keys/values are in the cache
        self.num_cached_tokens = 0  # of those, how many came from the prefix cache at admission
        self.arrival_time = time.monotonic() if arrival_time is None else arrival_time
        # set by the engine when the request is added: the token ids that end it (None: none does) and
        # the number of generated tokens at which it ends by length
        self.stop_ids: frozenset[int] | None = None
        self.length_limit: int | None = None

    def token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.output_token_ids

    def __len__(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    def tokens_between(self, start: int, end: int) -> list[int]:
        n_prompt = len(self.prompt_token_ids)
        if end <= n_prompt:
            return self.prompt_token_ids[start:end]
        if start >= n_prompt:
            return self.output_token_ids[start - n_prompt : end - n_prompt]
        return self.prompt_token_ids[start:] + self.output_token_ids[: end - n_prompt]

    def append_token(self, token_id: int) -> None:
        self.output_token_ids.append(token_id)

    def is_finished(self) -> bool:
        return self.status in _FINISHED

    def num_uncomputed_tokens(self) -> int:
        return len(self) - self.num_computed_tokens

    def reset_for_recompute(self) -> None:
        """Preemption by recompute keeps the tokens and drops the cache progress
        (``clockwork/engine/sequence.py:79-82``)."""
        self.num_computed_tokens = 0


class RequestOutput:
    """What ``LLMEngine.step`` reports for a request that sampled a token (the reference's
    ``clockwork/engine/sequence.py`` RequestOutput: ids, text, finish state, counts).

    An output holds what was true when it was made (how many tokens were generated, whether and why
    the request finished, the text) and reads the rest from its sequence: ``prompt_token_ids`` is the
    request's own prompt list and ``token_ids`` a view of its output list as long as it was then (the
    list only ever grows), so that a step costs the same however long the prompt and the output are.
    Treat both as read-only."""

    __slots__ = ("_seq", "num_generated_tokens", "finished", "finish_reason", "text", "delta_text")

    def __init__(self, seq: Sequence, num_generated_tokens: int, finished: bool, finish_reason: str | None,
                 text: str = "", delta_text: str = "") -> None:
        self._seq = seq
        self.num_generated_tokens = num_generated_tokens
        self.finished = finished
        self.finish_reason = finish_reason
        self.text = text
        self.delta_text = delta_text

    @property
    def request_id(self) -> str:
        return self._seq.seq_id

    @property
    def prompt_token_ids(self) -> list[int]:
        return self._seq.prompt_token_ids

    @property
    def num_prompt_tokens(self) -> int:
        return len(self._seq.prompt_token_ids)

    @property
    def num_cached_tokens(self) -> int:
        return self._seq.num_cached_tokens

    @property
    def token_ids(self) -> list[int]:
        out = self._seq.output_token_ids
        return out if len(out) == self.num_generated_tokens else out[: self.num_generated_tokens]

    def __repr__(self) -> str:
        return (f"RequestOutput(request_id={self.request_id!r}, token_ids={self.token_ids!r}, text={self.text!r}, "
                f"finished={self.finished}, finish_reason={self.finish_reason!r})")
