"""Iteration-level ("continuous") batching (behaviour of src/llmserve/scheduler.py:94-173).

Every step a fresh batch is built under two limits, ``max_num_seqs`` running sequences and
``max_num_batched_tokens`` new tokens:

1. running sequences first, in admission order: a decoding sequence gets its one token, a
   sequence still in its prompt gets as much of it as the budget allows (a portion);
2. then waiting sequences, first come first served, while budget, sequence slots and pages last.
   Only the head of the queue is looked at; a portion needs pages for that portion only.

When pages run out for a running sequence, the most recently admitted running sequence is
preempted: everything it holds is given back, its computed count returns to zero and it goes to
the *front* of the waiting queue, to be recomputed (prompt and the tokens generated so far) later.
If the sequence that needs pages is itself the newest, it is the one preempted and scheduling of
running sequences stops. After a preemption nothing is admitted in that step. A request that could
not fit even with the whole cache to itself is refused at intake, so preemption always ends.
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


class Scheduler:
    def __init__(self, cfg: SchedulerConfig, manager: CacheManager) -> None:
        self.cfg = cfg
        self.cm = manager
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.num_preemptions = 0

    def add(self, seq: Sequence) -> None:
        seq.status = SeqStatus.WAITING
        self.waiting.append(seq)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def finish(self, seq: Sequence) -> None:
        seq.status = SeqStatus.FINISHED
        if seq in self.running:
            self.running.remove(seq)
        elif seq in self.waiting:
            self.waiting.remove(seq)
        if self.cm.is_live(seq.seq_id):
            self.cm.release(seq.seq_id)

    def _preempt(self, seq: Sequence, out: SchedulerOutput) -> None:
        self.running.remove(seq)
        self.cm.release(seq.seq_id)
        seq.num_computed_tokens = 0
        seq.num_preemptions += 1
        seq.status = SeqStatus.WAITING
        self.waiting.appendleft(seq)
        self.num_preemptions += 1
        out.preempted.append(seq)

    def _admit(self, seq: Sequence, n: int, out: SchedulerOutput) -> None:
        self.waiting.popleft()
        self.cm.admit(seq.seq_id)
        self.cm.allocate(seq.seq_id, n)
        seq.status = SeqStatus.RUNNING
        if seq.request.metrics.first_scheduled_time is None:
            seq.request.metrics.first_scheduled_time = time.monotonic()
        self.running.append(seq)
        out.scheduled.append(ScheduledSeq(seq, n))

    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput()
        budget = self.cfg.max_num_batched_tokens
        chunked = self.cfg.enable_chunked_prefill

        # Without chunked prefill a prompt larger than the budget can never share a step with
        # decodes: run it in a step of its own (src/llmserve/scheduler.py:99-120).
        if not chunked and self.waiting and self.running:
            head = self.waiting[0]
            n = head.num_tokens - head.num_computed_tokens
            if (n > budget and len(self.running) < self.cfg.max_num_seqs
                    and self.cm.can_allocate(head.seq_id, n)):
                self._admit(head, n, out)
                return out

        # 1) running sequences, oldest first
        i = 0
        while i < len(self.running) and budget > 0:
            seq = self.running[i]
            remaining = seq.num_tokens - seq.num_computed_tokens
            n = min(remaining, budget) if chunked else remaining
            if n > budget and out.scheduled:
                break
            while not self.cm.try_allocate(seq.seq_id, n):
                victim = self.running[-1]
                if victim is seq:
                    self._preempt(seq, out)
                    seq = None
                    break
                self._preempt(victim, out)
            if seq is None:
                break
            out.scheduled.append(ScheduledSeq(seq, n))
            budget -= n
            i += 1

        # 2) waiting sequences, first come first served; none after a preemption
        if not out.preempted:
            while self.waiting and budget > 0 and len(self.running) < self.cfg.max_num_seqs:
                seq = self.waiting[0]
                remaining = seq.num_tokens - seq.num_computed_tokens
                if chunked:
                    n = min(remaining, budget)
                else:
                    n = remaining
                    if n > budget and out.scheduled:
                        break
                if not self.cm.can_allocate(seq.seq_id, n):
                    break
                self._admit(seq, n, out)
                budget -= n
        return out
