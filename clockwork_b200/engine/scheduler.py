"""Continuous-batching scheduler: decode first, first-come-first-served admission, prompts cut
into portions under a token budget, preemption by recompute when pages run out.

Rules taken from the reference's ``clockwork/scheduler/scheduler.py``:

* priority is (arrival, order of adding) and nothing else, so the same inputs give the same
  schedule (``:57-58``);
* every running sequence that has a token to decode gets its slot before anything is admitted
  (``:149-155``); if a slot needs a page and none is free, the latest-arrived running sequence
  not yet granted a slot this step is preempted, and if none is left the sequence preempts
  itself (``:98-118``).  Preemption frees its pages, resets its progress, keeps its tokens, and
  puts it at the front of the waiting queue, first come first served among the preempted
  (``:79-96``);
* admission looks at the head of the waiting queue only (``:159-166``): the prefix cache is
  consulted first, then the sequence needs room in the token budget and pages for all its
  tokens with the watermark left free; a refused admission undoes the prefix match
  (``:120-147``);
* finished and aborted sequences give everything back (``:172-197``).

What differs: the reference admits a prompt whole or not at all, so a prompt longer than the
budget can never run.  Here a prompt is cut into portions: an admitted sequence takes as many
of its uncomputed tokens as the step's remaining budget (and ``prefill_chunk_size``) allows, and
stays running with the rest, which later steps take, before new admissions, in priority order.
A sequence produces a token only in the step that computes its last uncomputed token.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from ..cache.manager import CacheManager
from ..cache.prefix import PrefixCache
from ..config.engine import SchedulerConfig
from .sequence import Sequence, SequenceStatus


@dataclass
class ScheduledPortion:
    seq: Sequence
    start: int  # first position computed this step
    num_tokens: int
    samples: bool  # whether the step computes the sequence's last token, so a token is sampled


@dataclass
class SchedulerOutput:
    portions: list[ScheduledPortion] = field(default_factory=list)
    prefill_seqs: list[Sequence] = field(default_factory=list)  # sequences given a prompt portion
    decode_seqs: list[Sequence] = field(default_factory=list)  # sequences given one decode token
    preempted: list[Sequence] = field(default_factory=list)
    num_batched_tokens: int = 0

    def is_empty(self) -> bool:
        return not (self.portions or self.preempted)


@dataclass
class SchedulerStats:
    num_waiting: int = 0
    num_running: int = 0
    num_preempted_total: int = 0
    num_scheduled_batches: int = 0
    total_prompt_tokens: int = 0
    total_cached_tokens: int = 0


class Scheduler:
    def __init__(self, cfg: SchedulerConfig, cache: CacheManager, prefix_cache: PrefixCache | None = None) -> None:
        self.cfg = cfg
        self.cache = cache
        self.prefix_cache = prefix_cache
        self.waiting: list[Sequence] = []
        self.running: list[Sequence] = []
        self.stats = SchedulerStats()
        self._arrival_order: dict[str, int] = {}
        self._arrival_counter = 0

    # ---- queues -------------------------------------------------------------------------------
    def _priority(self, seq: Sequence) -> tuple[float, int]:
        return (seq.arrival_time, self._arrival_order.get(seq.seq_id, 0))

    def add_seq(self, seq: Sequence) -> None:
        self._arrival_order[seq.seq_id] = self._arrival_counter
        self._arrival_counter += 1
        seq.status = SequenceStatus.WAITING
        self.waiting.append(seq)
        self._refresh_counts()

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def _refresh_counts(self) -> None:
        self.stats.num_waiting = len(self.waiting)
        self.stats.num_running = len(self.running)

    # ---- giving memory back ----------------------------------------------------------------------
    def _free_resources(self, seq: Sequence) -> None:
        if seq.seq_id not in self.cache.requests:
            return
        shared = self.cache.close(seq.seq_id)
        if shared and self.prefix_cache is not None:
            self.prefix_cache.release(shared)

    def _preempt(self, seq: Sequence) -> None:
        self._free_resources(seq)
        seq.reset_for_recompute()
        seq.num_cached_tokens = 0
        seq.status = SequenceStatus.PREEMPTED
        key = self._priority(seq)
        i = 0
        while (i < len(self.waiting) and self.waiting[i].status is SequenceStatus.PREEMPTED
               and self._priority(self.waiting[i]) < key):
            i += 1
        self.waiting.insert(i, seq)
        self.stats.num_preempted_total += 1

    # ---- one step's plan -------------------------------------------------------------------------
    def _chunk(self, uncomputed: int, budget_left: int) -> int:
        n = min(uncomputed, budget_left)
        if self.cfg.prefill_chunk_size:
            n = min(n, self.cfg.prefill_chunk_size)
        return max(n, 0)

    def _all_decode(self, ordered: list[Sequence], out: SchedulerOutput) -> bool:
        """The common step of a running batch, decided without the general machinery: every running
        sequence decodes one token, and the pages for that are there (mostly the token's slot lies in
        a page the sequence already owns alone; the others get their page here).  Makes the plan the
        general path would make; returns False, with nothing planned, when a sequence is in the
        middle of its prompt or the pages run out (the general path then decides whom to preempt;
        reservations made here stay and are what it would have made first)."""
        cache = self.cache
        requests = cache.requests
        portions = []
        for seq in ordered:
            n = len(seq.prompt_token_ids) + len(seq.output_token_ids)
            req = requests.get(seq.seq_id)
            if req is None or seq.status is not SequenceStatus.RUNNING or n - seq.num_computed_tokens != 1:
                return False
            if n <= req.writable_len:
                if n > req.num_tokens:
                    req.num_tokens = n  # what CacheManager.reserve does when nothing has to be allocated
            elif cache.can_reserve(req, n):
                cache.reserve(req, n)
            else:
                return False
            portions.append(ScheduledPortion(seq, n - 1, 1, True))
        out.portions.extend(portions)
        out.decode_seqs.extend(ordered)
        out.num_batched_tokens += len(ordered)
        return True

    def plan_next_decode(self, max_model_len: int) -> SchedulerOutput | None:
        """Called while a decode step of every running sequence is in flight and its tokens are not
        known yet: the plan of the step after it, under the assumption that no sequence ends and
        nothing arrives, with the pages it needs reserved; None when that assumption is known to fail
        (a sequence ends by length, something waits, a sequence is in its prompt, pages run out).
        The engine drops the plan if the assumption fails after all; the reservations are then
        what the general path would have made, or belong to sequences that are freed."""
        if self.waiting or not self.running:
            return None
        ordered = sorted(self.running, key=self._priority)
        cache = self.cache
        out = SchedulerOutput()
        for seq in ordered:
            n = len(seq.prompt_token_ids) + len(seq.output_token_ids)  # without the token in flight
            req = cache.requests.get(seq.seq_id)
            if (req is None or seq.status is not SequenceStatus.RUNNING or n - seq.num_computed_tokens != 1
                    or len(seq.output_token_ids) + 1 >= seq.sampling_params.max_tokens or n + 1 >= max_model_len):
                return None
            if n + 1 > req.writable_len:
                if not cache.can_reserve(req, n + 1):
                    return None
                cache.reserve(req, n + 1)
            elif n + 1 > req.num_tokens:
                req.num_tokens = n + 1
            out.portions.append(ScheduledPortion(seq, n, 1, True))
        out.decode_seqs.extend(ordered)
        out.num_batched_tokens = len(ordered)
        return out

    def accept_plan(self, out: SchedulerOutput) -> None:
        """Bookkeeping of a plan made by ``plan_next_decode`` that the engine now runs as a step."""
        self.stats.num_scheduled_batches += 1
        self._refresh_counts()

    def _schedule_running(self, out: SchedulerOutput) -> list[Sequence]:
        ordered = sorted(self.running, key=self._priority)
        if ordered and self._all_decode(ordered, out):
            return ordered
        kept: list[Sequence] = []
        # pass 1: decodes, in priority order, each reserving its slot at once so that a later
        # sequence sees the true pool
        pending = [s for s in ordered]
        decodes = [s for s in pending if s.num_uncomputed_tokens() == 1]
        others = [s for s in pending if s.num_uncomputed_tokens() != 1]
        victims_pool = list(ordered)  # candidates for preemption, latest arrival last
        granted: set[str] = set()
        for seq in decodes:
            if seq.status is SequenceStatus.PREEMPTED:
                continue
            req = self.cache.get(seq.seq_id)
            while not self.cache.can_reserve(req, len(seq)):
                victim = None
                for cand in reversed(victims_pool):
                    if cand.seq_id not in granted and cand is not seq and cand.status is SequenceStatus.RUNNING:
                        victim = cand
                        break
                if victim is None:
                    victim = seq
                victims_pool.remove(victim)
                self._preempt(victim)
                out.preempted.append(victim)
                if victim is seq:
                    break
            if seq.status is SequenceStatus.PREEMPTED:
                continue
            self.cache.reserve(req, len(seq))
            granted.add(seq.seq_id)
            out.portions.append(ScheduledPortion(seq, seq.num_computed_tokens, 1, True))
            out.decode_seqs.append(seq)
            out.num_batched_tokens += 1
        # pass 2: sequences in the middle of their prompt take portions of the remaining budget
        for seq in others:
            if seq.status is SequenceStatus.PREEMPTED:
                continue
            n = self._chunk(seq.num_uncomputed_tokens(), self.cfg.max_num_batched_tokens - out.num_batched_tokens)
            if n > 0:
                out.portions.append(ScheduledPortion(seq, seq.num_computed_tokens, n,
                                                     n == seq.num_uncomputed_tokens()))
                out.prefill_seqs.append(seq)
                out.num_batched_tokens += n
        for seq in ordered:
            if seq.status is SequenceStatus.RUNNING:
                kept.append(seq)
        return kept

    def _try_admit(self, seq: Sequence, out: SchedulerOutput) -> bool:
        matched_pages: list[int] = []
        matched_tokens = 0
        if self.prefix_cache is not None:
            match = self.prefix_cache.match(seq.token_ids())
            matched_pages, matched_tokens = match.pages, match.num_tokens
        uncomputed = len(seq) - matched_tokens
        n = self._chunk(uncomputed, self.cfg.max_num_batched_tokens - out.num_batched_tokens)
        fits = n > 0 and self.cache.can_open(len(seq), len(matched_pages))
        if not fits:
            if matched_pages and self.prefix_cache is not None:
                self.prefix_cache.release(matched_pages)
            return False
        req = self.cache.open(seq.seq_id, shared_prefix=matched_pages)
        self.cache.reserve(req, len(seq))
        seq.num_cached_tokens = matched_tokens
        seq.num_computed_tokens = matched_tokens
        seq.status = SequenceStatus.RUNNING
        self.stats.total_prompt_tokens += len(seq)
        self.stats.total_cached_tokens += matched_tokens
        out.portions.append(ScheduledPortion(seq, matched_tokens, n, n == uncomputed))
        out.prefill_seqs.append(seq)
        out.num_batched_tokens += n
        return True

    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput()
        self.running = self._schedule_running(out)
        while self.waiting and len(self.running) < self.cfg.max_num_seqs:
            seq = self.waiting[0]
            if not self._try_admit(seq, out):
                break
            self.waiting.pop(0)
            self.running.append(seq)
        if not out.is_empty():
            self.stats.num_scheduled_batches += 1
        self._refresh_counts()
        return out

    # ---- after a step -----------------------------------------------------------------------------
    def free_finished(self) -> None:
        for seq in self.running:
            if seq.is_finished():
                self._free_resources(seq)
                self._arrival_order.pop(seq.seq_id, None)
        self.running = [s for s in self.running if not s.is_finished()]
        self._refresh_counts()

    def abort(self, seq_id: str) -> None:
        for queue in (self.waiting, self.running):
            for i, seq in enumerate(queue):
                if seq.seq_id == seq_id:
                    if queue is self.running:
                        self._free_resources(seq)
                    queue.pop(i)
                    seq.status = SequenceStatus.FINISHED_ABORTED
                    self._arrival_order.pop(seq_id, None)
                    self._refresh_counts()
                    return
