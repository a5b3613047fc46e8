"""Continuous-batching scheduler: which tokens of which requests the next step runs.

Bookkeeping only (no tensors), one owner, not thread-safe -- like the reference's
scheduler (worker/src/inference/scheduler.py:1-17), whose order of work each step
is kept:

1. requests that were aborted are dropped and their pages returned
   (scheduler.py:168-180);
2. running requests get the pages their known tokens need; when the pool is short
   the NEWEST running request is preempted: its pages are returned, it forgets what
   it cached and goes to the FRONT of the waiting queue, to be recomputed later as
   prompt + tokens generated so far (scheduler.py:182-194, 213-225);
3. waiting requests are admitted first-in-first-out -- never skipping the head --
   while a seat, budget and pages for all their known tokens are available
   (scheduler.py:196-211);
4. the plan: one token for every request that is decoding, then the rest of the
   token budget is dealt, in admission order, to requests that still have prompt
   tokens to cache, as portions.

Step 4 is where this scheduler goes beyond the reference, which always runs an
admitted prompt whole (scheduler.py:145-147): here a prompt may be cut anywhere,
down to one token, by the budget or by ``prefill_chunk``.  A request whose portion
does not reach its last known token gets no sampled token in that step.
``complete`` appends sampled tokens; tokens are appended nowhere else, so a
preempted request never emits a token twice (scheduler.py:15-16).
"""

from __future__ import annotations

import enum
import logging
from collections import deque
from dataclasses import dataclass, field
from typing import Sequence as SequenceT

from ..cache.manager import CacheExhausted

_log = logging.getLogger(__name__)


class SeqState(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass(eq=False)
class Sequence:
    request_id: str
    prompt_ids: list[int]
    max_new_tokens: int
    temperature: float = 0.0
    eos_id: int | None = None
    seed: int = 0
    output_ids: list[int] = field(default_factory=list)
    seat: int | None = None
    num_cached: int = 0  # tokens whose keys and values are in the cache
    state: SeqState = SeqState.WAITING
    preemptions: int = 0
    finish_reason: str | None = None

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def num_pending(self) -> int:
        return self.num_tokens - self.num_cached

    def tokens(self, start: int, stop: int) -> list[int]:
        n = len(self.prompt_ids)
        if stop <= n:
            return self.prompt_ids[start:stop]
        if start >= n:
            return self.output_ids[start - n : stop - n]
        return self.prompt_ids[start:] + self.output_ids[: stop - n]


@dataclass(frozen=True)
class ScheduledSeq:
    seq: Sequence
    token_ids: list[int]
    past_len: int
    samples: bool  # the portion reaches the request's last known token


@dataclass(frozen=True)
class StepPlan:
    items: tuple[ScheduledSeq, ...]

    @property
    def num_tokens(self) -> int:
        return sum(len(item.token_ids) for item in self.items)

    @property
    def kind(self) -> str:
        return "decode" if all(len(item.token_ids) == 1 for item in self.items) else "prefill"


@dataclass(frozen=True)
class Emission:
    seq: Sequence
    token_id: int
    finished: bool


class Scheduler:
    def __init__(self, cache, max_seqs: int = 32, token_budget: int = 2048, prefill_chunk: int | None = None) -> None:
        if max_seqs < 1 or token_budget < 1:
            raise ValueError("max_seqs and token_budget must be >= 1")
        if prefill_chunk is not None and prefill_chunk < 1:
            raise ValueError("prefill_chunk must be >= 1")
        self._cache = cache
        self._max_seqs = max_seqs
        self._budget = token_budget
        self._chunk = prefill_chunk
        self._waiting: deque[Sequence] = deque()
        self._running: list[Sequence] = []
        self._aborted: set[str] = set()
        self._ids: dict[str, Sequence] = {}

    # -- queries ------------------------------------------------------------
    @property
    def num_waiting(self) -> int:
        return len(self._waiting)

    @property
    def num_running(self) -> int:
        return len(self._running)

    def has_work(self) -> bool:
        return bool(self._waiting or self._running or self._aborted)

    # -- requests in and out ------------------------------------------------
    def submit(self, seq: Sequence) -> None:
        if not seq.prompt_ids:
            raise ValueError("prompt_ids must be non-empty")
        if seq.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
        if seq.request_id in self._ids:
            raise ValueError(f"duplicate request_id {seq.request_id}")
        # Worst case the request holds every page it will ever need at once (scheduler.py:125-131).
        total = len(seq.prompt_ids) + seq.max_new_tokens
        if not self._cache.fits_ever(total):
            raise CacheExhausted(
                f"out of KV blocks: request of {total} tokens can never fit "
                f"(pool has {self._cache.total_pages()} pages per group)"
            )
        seq.state = SeqState.WAITING
        self._waiting.append(seq)
        self._ids[seq.request_id] = seq

    def abort(self, request_id: str) -> None:
        """Takes effect at the next ``schedule()``; results in flight for it are discarded."""
        if request_id in self._ids:
            self._aborted.add(request_id)

    def force_preempt(self, request_id: str) -> bool:
        """Preempt a running request now (for tests and experiments)."""
        seq = self._ids.get(request_id)
        if seq is None or seq.state is not SeqState.RUNNING:
            return False
        self._preempt(seq)
        return True

    # -- the step -----------------------------------------------------------
    def schedule(self) -> StepPlan:
        self._reap_aborted()
        self._grow_running()
        self._admit()
        return StepPlan(items=tuple(self._deal()))

    def complete(self, plan: StepPlan, sampled: SequenceT[int]) -> list[Emission]:
        """``sampled`` holds one token for every item of the plan with ``samples``, in order."""
        wanted = sum(1 for item in plan.items if item.samples)
        if len(sampled) != wanted:
            raise ValueError(f"the plan samples {wanted} tokens, got {len(sampled)}")
        out: list[Emission] = []
        tokens = iter(sampled)
        for item in plan.items:
            token = int(next(tokens)) if item.samples else None
            seq = item.seq
            if seq.request_id in self._aborted or seq.state is not SeqState.RUNNING:
                continue  # aborted, preempted or finished while the step was in flight
            seq.num_cached = item.past_len + len(item.token_ids)
            self._cache.trim(seq.seat, seq.num_cached)
            if token is None:
                continue
            seq.output_ids.append(token)
            if seq.eos_id is not None and token == seq.eos_id:
                seq.finish_reason = "eos"
            elif len(seq.output_ids) >= seq.max_new_tokens:
                seq.finish_reason = "length"
            finished = seq.finish_reason is not None
            if finished:
                self._finish(seq)
            out.append(Emission(seq=seq, token_id=token, finished=finished))
        return out

    # -- a step ahead ---------------------------------------------------------
    # A decode step may be launched before the tokens of the step ahead of it have reached the host: the
    # device feeds them to it directly.  The scheduler then books the earlier step provisionally
    # (``assume``: one more cached token, a placeholder for the token nobody has seen yet), plans the next
    # step as usual, and fills the tokens in when they arrive (``resolve``).  A request that turns out to
    # have ended with that token is finished then; its row in the step already launched is ignored.
    PLACEHOLDER = -1

    def can_look_ahead(self, plan: StepPlan) -> bool:
        """True when the step after ``plan`` can be planned without ``plan``'s tokens: decoding only,
        nobody waiting or aborted, and no request that this step ends by length."""
        if self._waiting or self._aborted or not plan.items:
            return False
        for item in plan.items:
            seq = item.seq
            if len(item.token_ids) != 1 or not item.samples or seq.state is not SeqState.RUNNING:
                return False
            if len(seq.output_ids) + 1 >= seq.max_new_tokens:
                return False
        return len(plan.items) == len(self._running)

    def assume(self, plan: StepPlan) -> None:
        for item in plan.items:
            seq = item.seq
            seq.num_cached = item.past_len + len(item.token_ids)
            self._cache.trim(seq.seat, seq.num_cached)
            seq.output_ids.append(self.PLACEHOLDER)

    def resolve(self, plan: StepPlan, sampled: SequenceT[int]) -> list[Emission]:
        """The tokens of a step booked with ``assume``: replaces the placeholders, finishes what ended."""
        if len(sampled) != len(plan.items):
            raise ValueError(f"the plan samples {len(plan.items)} tokens, got {len(sampled)}")
        out: list[Emission] = []
        for item, token in zip(plan.items, sampled):
            seq = item.seq
            index = item.past_len + 1 - len(seq.prompt_ids)  # where this step's token sits among the outputs
            if seq.state is SeqState.FINISHED or index >= len(seq.output_ids) or seq.output_ids[index] != self.PLACEHOLDER:
                continue
            token = int(token)
            seq.output_ids[index] = token
            if seq.request_id in self._aborted:
                continue
            if seq.eos_id is not None and token == seq.eos_id:
                seq.finish_reason = "eos"
            elif index + 1 >= seq.max_new_tokens:
                seq.finish_reason = "length"
            finished = seq.finish_reason is not None
            if finished:
                del seq.output_ids[index + 1 :]  # a placeholder of the step launched meanwhile
                if seq.state is SeqState.RUNNING:
                    self._finish(seq)
                else:  # preempted meanwhile: it waits, holding nothing
                    self._waiting.remove(seq)
                    seq.state = SeqState.FINISHED
                    self._ids.pop(seq.request_id, None)
            out.append(Emission(seq=seq, token_id=token, finished=finished))
        return out

    # -- internals ------------------------------------------------------------
    def _reap_aborted(self) -> None:
        for request_id in list(self._aborted):
            seq = self._ids.pop(request_id, None)
            if seq is None:
                continue
            if seq.state is SeqState.WAITING:
                self._waiting.remove(seq)
            elif seq.state is SeqState.RUNNING:
                self._running.remove(seq)
                self._release(seq)
            seq.state = SeqState.FINISHED
            seq.finish_reason = "aborted"
            _log.info("sequence aborted request_id=%s", request_id)
        self._aborted.clear()

    def _grow_running(self) -> None:
        index = 0
        while index < len(self._running):
            seq = self._running[index]
            while seq.state is SeqState.RUNNING and not self._cache.grow(seq.seat, seq.num_tokens):
                self._preempt(self._running[-1])  # the newest; may be seq itself
            if seq.state is SeqState.RUNNING:
                index += 1

    def _planned_tokens(self) -> int:
        """Tokens the running requests will take of this step's budget."""
        left = self._budget
        for seq in self._running:
            if seq.num_pending == 1:
                left -= 1
        for seq in self._running:
            if seq.num_pending > 1 and left > 0:
                left -= min(seq.num_pending, left, self._chunk or left)
        return self._budget - left

    def _admit(self) -> None:
        tokens = self._planned_tokens()
        while self._waiting and len(self._running) < self._max_seqs and self._cache.free_seats > 0:
            seq = self._waiting[0]
            if tokens >= self._budget and self._running:
                break  # no budget left for even one of its tokens; a lone request is always admitted
            if not self._cache.can_grow(None, seq.num_tokens):
                break
            self._waiting.popleft()
            seq.seat = self._cache.open_seat()
            if not self._cache.grow(seq.seat, seq.num_tokens):  # cannot happen after can_grow; stay safe
                self._cache.close_seat(seq.seat)
                seq.seat = None
                self._waiting.appendleft(seq)
                break
            seq.num_cached = 0
            seq.state = SeqState.RUNNING
            self._running.append(seq)
            room = max(0, self._budget - tokens)
            tokens += min(seq.num_pending, room, self._chunk or room) if room else 0

    def _deal(self) -> list[ScheduledSeq]:
        items: list[ScheduledSeq] = []
        left = self._budget
        for seq in self._running:  # decoding requests first: one token each, whatever the budget
            if seq.num_pending == 1:
                items.append(ScheduledSeq(seq, seq.tokens(seq.num_cached, seq.num_tokens), seq.num_cached, True))
                left -= 1
        for seq in self._running:  # then portions of prompts, in admission order
            pending = seq.num_pending
            if pending <= 1:
                continue
            room = max(left, 0)
            count = min(pending, room, self._chunk or room)
            if count <= 0:
                continue
            stop = seq.num_cached + count
            items.append(ScheduledSeq(seq, seq.tokens(seq.num_cached, stop), seq.num_cached, stop == seq.num_tokens))
            left -= count
        return items

    def _preempt(self, seq: Sequence) -> None:
        self._running.remove(seq)
        self._release(seq)
        seq.num_cached = 0
        seq.state = SeqState.WAITING
        seq.preemptions += 1
        self._waiting.appendleft(seq)
        _log.info(
            "sequence preempted request_id=%s tokens=%s preemptions=%s", seq.request_id, seq.num_tokens, seq.preemptions
        )

    def _finish(self, seq: Sequence) -> None:
        self._running.remove(seq)
        self._release(seq)
        seq.state = SeqState.FINISHED
        self._ids.pop(seq.request_id, None)

    def _release(self, seq: Sequence) -> None:
        if seq.seat is not None:
            self._cache.close_seat(seq.seat)
            seq.seat = None
