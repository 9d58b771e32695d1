"""A request as the scheduler and the engine see it, and what the engine reports about it.

The field names and the states are those of the reference's request object
(``clockwork/engine/sequence.py:10-96``), because the scheduler's rules, the tests and the users of
``RequestOutput`` speak in them; the block table is not here but in the cache manager
(``clockwork_b200/cache/manager.py``), and progress is kept as one number that only three verbs
change: ``admit`` (a prefix came from the cache), ``advance`` (a step computed tokens) and
``rewind`` (preemption by recompute)."""

from __future__ import annotations

import time
from enum import Enum

from ..sampling.params import SamplingParams


class SequenceStatus(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    PREEMPTED = "preempted"
    FINISHED_STOPPED = "finished_stopped"
    FINISHED_LENGTH = "finished_length"
    FINISHED_ABORTED = "finished_aborted"

    @property
    def finished(self) -> bool:
        return self.name.startswith("FINISHED")

    @property
    def finish_reason(self) -> str | None:
        return {"FINISHED_STOPPED": "stop", "FINISHED_LENGTH": "length", "FINISHED_ABORTED": "abort"}.get(self.name)


class Sequence:
    """One request: its prompt, what it has generated, and how far the cache has got with it."""

    __slots__ = ("seq_id", "prompt_token_ids", "output_token_ids", "sampling_params", "status", "arrival_time",
                 "num_computed_tokens", "num_cached_tokens", "stop_ids", "length_limit", "state_slot")

    def __init__(self, seq_id: str, prompt_token_ids: list[int], sampling_params: SamplingParams | None = None,
                 arrival_time: float | None = None) -> None:
        self.seq_id = seq_id
        self.prompt_token_ids = list(prompt_token_ids)
        self.output_token_ids: list[int] = []
        self.sampling_params = sampling_params or SamplingParams()
        self.status = SequenceStatus.WAITING
        self.arrival_time = time.monotonic() if arrival_time is None else arrival_time
        self.num_computed_tokens = 0  # tokens whose keys and values are in the cache
        self.num_cached_tokens = 0    # how many of them the prefix cache supplied at the last admission
        # filled in by the engine: the token ids that end the request (None: none does), and the number
        # of generated tokens at which it ends by length
        self.stop_ids: frozenset[int] | None = None
        self.length_limit: int | None = None
        self.state_slot: int | None = None  # the request's row in the engine's per-request device state

    # ---- tokens ------------------------------------------------------------------------------------
    def __len__(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    def token_ids(self) -> list[int]:
        return [*self.prompt_token_ids, *self.output_token_ids]

    def tokens_between(self, start: int, end: int) -> list[int]:
        """Tokens at positions [start, end), wherever the border between prompt and output lies."""
        border = len(self.prompt_token_ids)
        head = self.prompt_token_ids[start:end] if start < border else []
        tail = self.output_token_ids[max(start - border, 0) : end - border] if end > border else []
        return head + tail if head and tail else (head or tail)

    def append_token(self, token_id: int) -> None:
        self.output_token_ids.append(token_id)

    # ---- progress ----------------------------------------------------------------------------------
    def num_uncomputed_tokens(self) -> int:
        return len(self) - self.num_computed_tokens

    def admit(self, cached_tokens: int) -> None:
        """The request starts (or starts again) running with this many leading tokens already cached."""
        self.num_cached_tokens = self.num_computed_tokens = cached_tokens
        self.status = SequenceStatus.RUNNING

    def rewind(self) -> None:
        """Preemption by recompute: the tokens stay, the cache's progress is dropped, so the next
        admission computes prompt and output so far again (``clockwork/engine/sequence.py:79-82``)."""
        self.num_computed_tokens = self.num_cached_tokens = 0
        self.status = SequenceStatus.PREEMPTED

    reset_for_recompute = rewind

    def is_finished(self) -> bool:
        return self.status.finished


class RequestOutput:
    """What ``LLMEngine.step`` reports for a request that sampled a token: ids, text, whether and why
    it finished, counts (the fields of the reference's ``RequestOutput``).

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
