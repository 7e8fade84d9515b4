"""Continuous batching: every step a new batch, chosen under a token budget and a sequence limit.

What is decided, and what the tests pin (the behaviour of src/llmserve/scheduler.py:94-173):

* A step spends at most ``max_num_batched_tokens`` new tokens on at most ``max_num_seqs``
  sequences. Sequences that already run come first, in the order they were admitted: a sequence
  that decodes takes its one token, a sequence still inside its prompt takes as much of the prompt
  as the budget has left (a *portion*). What is then left of the budget goes to the waiting queue,
  strictly first come first served: only its head is looked at, and it is admitted if a state slot
  is free and the pages for its first portion are.
* Pages are asked for per portion, from every cache group at once (``CacheManager.try_allocate``:
  all groups or nothing). When a running sequence cannot get its pages, the sequence admitted last
  is evicted: everything it holds goes back, its computed count returns to zero and it goes to the
  *front* of the queue, to be recomputed later (prompt and the tokens it has generated). If the
  sequence that needs pages is itself the newest, it is the one evicted, and no running sequence
  behind it is looked at in this step. A step that evicted somebody admits nobody.
* Without chunked prefill a prompt is never cut: one that is longer than the budget runs in a step
  of its own while the running sequences pause (src/llmserve/scheduler.py:99-120).

A request that could not fit with the whole cache to itself is refused at intake
(``LLMEngine.add_request``), so evicting always ends.
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field

from ..cache.manager import CacheManager
from .sequence import SeqStatus, Sequence


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 1024
    enable_chunked_prefill: bool = True
    max_model_len: int = 4096


@dataclass
class ScheduledSeq:
    seq: Sequence
    num_new_tokens: int


@dataclass
class SchedulerOutput:
    scheduled: list[ScheduledSeq] = field(default_factory=list)
    preempted: list[Sequence] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(s.num_new_tokens for s in self.scheduled)

    @property
    def is_empty(self) -> bool:
        return not self.scheduled


class _Step:
    """The batch under construction: what is left of the budget, who is in, who was evicted."""

    def __init__(self, budget: int) -> None:
        self.left = budget
        self.out = SchedulerOutput()

    def take(self, seq: Sequence, n: int) -> None:
        self.out.scheduled.append(ScheduledSeq(seq, n))
        self.left -= n

    @property
    def started(self) -> bool:
        return bool(self.out.scheduled)


class Scheduler:
    def __init__(self, cfg: SchedulerConfig, manager: CacheManager) -> None:
        self.cfg = cfg
        self.cm = manager
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.num_preemptions = 0

    # ------------------------------------------------------------------ queue
    def add(self, seq: Sequence) -> None:
        seq.status = SeqStatus.WAITING
        self.waiting.append(seq)

    def has_unfinished(self) -> bool:
        return bool(self.running) or bool(self.waiting)

    def finish(self, seq: Sequence) -> None:
        """Take ``seq`` out, wherever it is, and give back what it holds at once."""
        for queue in (self.running, self.waiting):
            if seq in queue:
                queue.remove(seq)
                break
        seq.status = SeqStatus.FINISHED
        if self.cm.is_live(seq.seq_id):
            self.cm.release(seq.seq_id)

    # ------------------------------------------------------------------ one step
    def schedule(self) -> SchedulerOutput:
        step = _Step(self.cfg.max_num_batched_tokens)
        if self._uncut_prompt_alone(step):
            return step.out
        self._advance_running(step)
        if not step.out.preempted:
            self._admit_waiting(step)
        return step.out

    def _want(self, seq: Sequence, step: _Step) -> int:
        """Tokens ``seq`` would run now: all it has left, cut to the budget if prompts may be cut."""
        left = seq.num_tokens - seq.num_computed_tokens
        return min(left, step.left) if self.cfg.enable_chunked_prefill else left

    def _uncut_prompt_alone(self, step: _Step) -> bool:
        """Without chunked prefill: the queue's head, if longer than the budget, gets this step."""
        if self.cfg.enable_chunked_prefill or not self.waiting or not self.running:
            return False
        head = self.waiting[0]
        n = self._want(head, step)
        if n <= step.left or len(self.running) >= self.cfg.max_num_seqs:
            return False
        if not self.cm.can_allocate(head.seq_id, n):
            return False
        self._admit(head, n, step)
        return True

    def _advance_running(self, step: _Step) -> None:
        at = 0
        while at < len(self.running) and step.left > 0:
            seq = self.running[at]
            n = self._want(seq, step)
            if n > step.left and step.started:
                return  # an uncut prompt that does not fit beside what is already in the step
            if not self._pages_or_evict(seq, n, step):
                return  # seq itself was evicted: it was the newest, nobody behind it
            step.take(seq, n)
            at += 1

    def _pages_or_evict(self, seq: Sequence, n: int, step: _Step) -> bool:
        """Pages for ``n`` more tokens of ``seq``, evicting from the back of the running list
        until they are there. False if ``seq`` had to go itself."""
        while not self.cm.try_allocate(seq.seq_id, n):
            newest = self.running[-1]
            self._evict(newest, step)
            if newest is seq:
                return False
        return True

    def _evict(self, seq: Sequence, step: _Step) -> None:
        self.running.pop()  # seq is the last one
        self.cm.release(seq.seq_id)
        seq.num_computed_tokens = 0
        seq.num_preemptions += 1
        seq.status = SeqStatus.WAITING
        self.waiting.appendleft(seq)
        self.num_preemptions += 1
        step.out.preempted.append(seq)

    def _admit_waiting(self, step: _Step) -> None:
        while self.waiting and step.left > 0 and len(self.running) < self.cfg.max_num_seqs:
            head = self.waiting[0]
            n = self._want(head, step)
            if n > step.left and step.started:
                return
            if not self.cm.can_allocate(head.seq_id, n):
                return
            self._admit(head, n, step)

    def _admit(self, seq: Sequence, n: int, step: _Step) -> None:
        self.waiting.popleft()
        self.cm.admit(seq.seq_id)
        self.cm.allocate(seq.seq_id, n)
        seq.status = SeqStatus.RUNNING
        self.running.append(seq)
        metrics = seq.request.metrics
        if metrics.first_scheduled_time is None:
            metrics.first_scheduled_time = time.monotonic()
        step.take(seq, n)
