"""Continuous batching: which requests run in the next step, and with how many tokens each.

The rules are the reference's (``clockwork/scheduler/scheduler.py``), plus portions:

* A request's rank is (arrival, order of adding) and nothing else, so equal inputs give equal
  schedules (``:57-58``).
* Requests that are running come first (``:149-155``).  One that has a single token left to compute
  (a decode) gets the slot for it before anything else is decided; if that slot needs a page and
  the pool has none, the running request of the latest rank that has not been granted its slot yet
  in this step is preempted, and if no such request is left, the request itself (``:98-118``).
* Preemption gives the request's pages back, drops its progress, keeps its tokens, and lets it wait
  in front of every request that has never run, in rank order among the preempted (``:79-96``).
* Admission is strictly in order: only the first waiting request is looked at (``:159-166``).  The
  prefix cache is asked first; the request then needs room in the step's token budget and pages for
  all of its tokens with the watermark left free; if it does not get in, what the prefix cache lent
  is handed back (``:120-147``).
* A request that finishes or is aborted gives everything back (``:172-197``).

What the reference does not have: it admits a prompt whole or not at all, so a prompt longer than
the budget never runs.  Here a request takes as many of its uncomputed tokens as the rest of the
budget (and ``prefill_chunk_size``) allows and keeps running with the remainder, which later steps
take before anybody new is admitted.  A token is sampled only in the step that computes a request's
last uncomputed token.

How it is kept: ``running`` is always in rank order (a request is inserted at its place when it is
admitted), requests that wait to be resumed after a preemption are a rank-ordered list of their
own in front of the first-come queue of requests that have never run, and a dictionary finds a
request by its id; counters are plain integers read into a ``SchedulerStats`` on demand.
"""

from __future__ import annotations

from bisect import insort
from collections import deque
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
        return len(self.portions) + len(self.preempted) == 0

    def give(self, seq: Sequence, start: int, count: int, decode: bool) -> None:
        self.portions.append(ScheduledPortion(seq, start, count, start + count == len(seq)))
        (self.decode_seqs if decode else self.prefill_seqs).append(seq)
        self.num_batched_tokens += count


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
        self.running: list[Sequence] = []                     # in rank order
        self._resuming: list[tuple[tuple, Sequence]] = []     # preempted, waiting to run again: (rank, request), sorted
        self._arrivals: deque[Sequence] = deque()             # never ran yet, first come first
        self._rank: dict[str, tuple[float, int]] = {}         # by request id, for everything queued or running
        self._added = 0
        self._preemptions = self._batches = self._prompt_tokens = self._cached_tokens = 0

    # ---- what the outside reads ----------------------------------------------------------------------
    @property
    def waiting(self) -> list[Sequence]:
        """Everything that waits, in the order in which it will be looked at."""
        return [seq for _, seq in self._resuming] + list(self._arrivals)

    @property
    def stats(self) -> SchedulerStats:
        return SchedulerStats(len(self._resuming) + len(self._arrivals), len(self.running), self._preemptions,
                              self._batches, self._prompt_tokens, self._cached_tokens)

    def has_unfinished(self) -> bool:
        return bool(self.running or self._arrivals or self._resuming)

    def add_seq(self, seq: Sequence) -> None:
        self._rank[seq.seq_id] = (seq.arrival_time, self._added)
        self._added += 1
        seq.status = SequenceStatus.WAITING
        self._arrivals.append(seq)

    # ---- letting go ----------------------------------------------------------------------------------
    def _release(self, seq: Sequence) -> None:
        """Everything the request holds goes back: its own pages to the pool, borrowed ones to the prefix cache."""
        if seq.seq_id in self.cache.requests:
            borrowed = self.cache.close(seq.seq_id)
            if borrowed and self.prefix_cache is not None:
                self.prefix_cache.release(borrowed)

    def _preempt(self, seq: Sequence, plan: SchedulerOutput) -> None:
        self._release(seq)
        seq.rewind()
        insort(self._resuming, (self._rank[seq.seq_id], seq), key=lambda entry: entry[0])
        self._preemptions += 1
        plan.preempted.append(seq)

    def free_finished(self) -> None:
        still = []
        for seq in self.running:
            if seq.status.finished:
                self._release(seq)
                self._rank.pop(seq.seq_id, None)
            else:
                still.append(seq)
        self.running = still

    def abort(self, seq_id: str) -> None:
        if seq_id not in self._rank:
            return
        del self._rank[seq_id]
        for i, seq in enumerate(self.running):
            if seq.seq_id == seq_id:
                self._release(seq)
                del self.running[i]
                seq.status = SequenceStatus.FINISHED_ABORTED
                return
        for i, (_, seq) in enumerate(self._resuming):
            if seq.seq_id == seq_id:
                del self._resuming[i]
                seq.status = SequenceStatus.FINISHED_ABORTED
                return
        for seq in self._arrivals:
            if seq.seq_id == seq_id:
                self._arrivals.remove(seq)
                seq.status = SequenceStatus.FINISHED_ABORTED
                return

    # ---- one step's plan -------------------------------------------------------------------------------
    def _portion(self, uncomputed: int, plan: SchedulerOutput) -> int:
        """How many of a request's uncomputed tokens this step can still take."""
        room = self.cfg.max_num_batched_tokens - plan.num_batched_tokens
        if self.cfg.prefill_chunk_size:
            room = min(room, self.cfg.prefill_chunk_size)
        return max(0, min(uncomputed, room))

    def _decode_slot(self, seq: Sequence, total: int) -> bool:
        """Make sure position ``total - 1`` of a running request has its slot.  Most steps it lies in a
        page the request owns alone and nothing has to be looked up."""
        req = self.cache.requests[seq.seq_id]
        if total <= req.writable_len:
            if total > req.num_tokens:
                req.num_tokens = total  # what CacheManager.reserve does when nothing has to be allocated
            return True
        if not self.cache.can_reserve(req, total):
            return False
        self.cache.reserve(req, total)
        return True

    def _all_decode(self, plan: SchedulerOutput) -> bool:
        """The common step of a running batch: every running request has exactly one token to compute and
        the pages for it are there.  Plans what the general path would plan; False, with nothing planned,
        when a request is in the middle of its prompt or a page is missing (the general path then decides
        whom to preempt; slots granted here stay granted and are what it would have granted first)."""
        grants = []
        for seq in self.running:
            total = len(seq)
            if (seq.status is not SequenceStatus.RUNNING or total - seq.num_computed_tokens != 1
                    or seq.seq_id not in self.cache.requests or not self._decode_slot(seq, total)):
                return False
            grants.append((seq, total - 1))
        for seq, position in grants:
            plan.give(seq, position, 1, decode=True)
        return True

    def _plan_running(self, plan: SchedulerOutput) -> None:
        if self.running and self._all_decode(plan):
            return
        # decodes first, in rank order; each takes its slot at once, so that the next sees the true pool
        granted: set[str] = set()
        for seq in list(self.running):
            if seq.status is not SequenceStatus.RUNNING or seq.num_uncomputed_tokens() != 1:
                continue
            while not self._decode_slot(seq, len(seq)):
                victim = next((other for other in reversed(self.running)
                               if other is not seq and other.status is SequenceStatus.RUNNING and other.seq_id not in granted), seq)
                self._preempt(victim, plan)
                if victim is seq:
                    break
            if seq.status is SequenceStatus.RUNNING:
                granted.add(seq.seq_id)
                plan.give(seq, seq.num_computed_tokens, 1, decode=True)
        # then the requests that are in the middle of their prompts share what is left of the budget
        for seq in self.running:
            if seq.status is SequenceStatus.RUNNING and seq.seq_id not in granted:
                count = self._portion(seq.num_uncomputed_tokens(), plan)
                if count:
                    plan.give(seq, seq.num_computed_tokens, count, decode=False)
        self.running = [seq for seq in self.running if seq.status is SequenceStatus.RUNNING]

    def _admit_first_waiting(self, plan: SchedulerOutput) -> bool:
        seq = self._resuming[0][1] if self._resuming else self._arrivals[0]
        total = len(seq)
        borrowed, cached = [], 0
        if self.prefix_cache is not None:
            hit = self.prefix_cache.match(seq.token_ids())
            borrowed, cached = hit.pages, hit.num_tokens
        count = self._portion(total - cached, plan)
        if count == 0 or not self.cache.can_open(total, len(borrowed)):
            if borrowed:
                self.prefix_cache.release(borrowed)  # not admitted: nothing of the look-up stays
            return False
        self.cache.reserve(self.cache.open(seq.seq_id, shared_prefix=borrowed), total)
        seq.admit(cached)
        self._prompt_tokens += total
        self._cached_tokens += cached
        plan.give(seq, cached, count, decode=False)
        if self._resuming:
            self._resuming.pop(0)
        else:
            self._arrivals.popleft()
        insort(self.running, seq, key=lambda s: self._rank[s.seq_id])
        return True

    def schedule(self) -> SchedulerOutput:
        plan = SchedulerOutput()
        self._plan_running(plan)
        while (self._resuming or self._arrivals) and len(self.running) < self.cfg.max_num_seqs:
            if not self._admit_first_waiting(plan):
                break
        if not plan.is_empty():
            self._batches += 1
        return plan

    # ---- planning one step ahead -------------------------------------------------------------------------
    def plan_next_decode(self, max_model_len: int) -> SchedulerOutput | None:
        """Called while a step in which every running request decodes is in flight and its tokens are not
        known yet: the plan of the step after it, if no request ends and nothing arrives, with the slots it
        needs granted; None when that cannot be (a request ends by length, something waits, a request is
        in its prompt, a page is missing).  The engine drops the plan if a request ends after all; the
        slots granted here are then what the general path would have granted, or belong to requests
        that are being freed."""
        if self._arrivals or self._resuming or not self.running:
            return None
        plan = SchedulerOutput()
        for seq in self.running:
            total = len(seq) + 1  # with the token that is in flight
            if (seq.status is not SequenceStatus.RUNNING or total - 1 - seq.num_computed_tokens != 1
                    or seq.seq_id not in self.cache.requests
                    or len(seq.output_token_ids) + 1 >= seq.sampling_params.max_tokens or total >= max_model_len
                    or not self._decode_slot(seq, total)):
                return None
            plan.portions.append(ScheduledPortion(seq, total - 1, 1, True))
        plan.decode_seqs.extend(self.running)
        plan.num_batched_tokens = len(self.running)
        return plan

    def accept_plan(self, plan: SchedulerOutput) -> None:
        """A plan made by ``plan_next_decode`` is now run as a step."""
        self._batches += 1
