"""Continuous-batching scheduler: which tokens of which requests the next step runs.

Bookkeeping only (no tensors), one owner, not thread-safe.  The policy is the
reference's (worker/src/inference/scheduler.py:141-236), in its order of work:

1. requests that were aborted leave and give their pages back (scheduler.py:168-180);
2. every running request gets the pages its known tokens need; when the pool is
   short the NEWEST running request is sent back: it gives up its pages, forgets
   what it cached and goes to the FRONT of the line, to be recomputed later as
   prompt + tokens generated so far (scheduler.py:182-194, 213-225);
3. the line is admitted head first, never skipping, while a seat, budget and the
   pages for all known tokens are there (scheduler.py:196-211);
4. the plan: one token for every request that is decoding, then the rest of the
   token budget dealt, in admission order, to requests with prompt tokens still to
   cache, as portions.

Step 4 goes beyond the reference, which always runs an admitted prompt whole
(scheduler.py:145-147): here a prompt may be cut anywhere, down to one token, by
the budget or by ``prefill_chunk``; a request whose portion does not reach its last
known token samples nothing in that step.  Tokens are appended in one place only
(``_take_token``), so a request that was sent back never emits a token twice
(scheduler.py:15-16).

How a request moves: ``submit`` puts it in the line (WAITING); ``_admit`` gives it a
seat (RUNNING); ``_leave_running`` is the one way out of RUNNING, either back to the
line (preemption) or for good (finished, aborted).
"""

from __future__ import annotations

import enum
import logging
from collections import deque
from typing import Iterable, NamedTuple, Sequence as SequenceT

from ..cache.manager import CacheExhausted

_log = logging.getLogger(__name__)


class SeqState(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


class Sequence:
    """One request as the scheduler sees it: what is known of it and how much of that is cached."""

    def __init__(self, request_id: str, prompt_ids, max_new_tokens: int, temperature: float = 0.0,
                 eos_id: int | None = None, seed: int = 0) -> None:
        self.request_id = request_id
        self.prompt_ids = list(prompt_ids)
        self.max_new_tokens = max_new_tokens
        self.temperature = temperature
        self.eos_id = eos_id
        self.seed = seed
        self.output_ids: list[int] = []
        self.seat: int | None = None
        self.num_cached = 0  # tokens whose keys and values are in the cache
        self.state = SeqState.WAITING
        self.preemptions = 0
        self.finish_reason: str | None = None  # "eos" | "length" | "aborted"

    def __repr__(self) -> str:
        return (f"Sequence({self.request_id!r}, prompt={len(self.prompt_ids)}, outputs={len(self.output_ids)}, "
                f"cached={self.num_cached}, {self.state.value})")

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def num_pending(self) -> int:
        return self.num_tokens - self.num_cached

    @property
    def is_running(self) -> bool:
        return self.state is SeqState.RUNNING

    def tokens(self, start: int, stop: int) -> list[int]:
        """Known tokens ``[start, stop)``, prompt and outputs read as one sequence."""
        split = len(self.prompt_ids)
        head = self.prompt_ids[start:min(stop, split)] if start < split else []
        tail = self.output_ids[max(start, split) - split : stop - split] if stop > split else []
        return head + tail


class ScheduledSeq(NamedTuple):
    seq: Sequence
    token_ids: list[int]
    past_len: int
    samples: bool  # the portion reaches the request's last known token


class Emission(NamedTuple):
    seq: Sequence
    token_id: int
    finished: bool


class StepPlan:
    def __init__(self, items: Iterable[ScheduledSeq]) -> None:
        self.items = tuple(items)

    @property
    def num_tokens(self) -> int:
        return sum(len(item.token_ids) for item in self.items)

    @property
    def num_samples(self) -> int:
        return sum(1 for item in self.items if item.samples)

    @property
    def kind(self) -> str:
        """``decode`` when every request brings one token, else ``prefill`` (the step statistics' groups)."""
        return "decode" if all(len(item.token_ids) == 1 for item in self.items) else "prefill"


class Scheduler:
    PLACEHOLDER = -1  # stands for a token that was sampled on the device and has not reached the host

    def __init__(self, cache, max_seqs: int = 32, token_budget: int = 2048, prefill_chunk: int | None = None) -> None:
        if max_seqs < 1 or token_budget < 1:
            raise ValueError("max_seqs and token_budget must be >= 1")
        if prefill_chunk is not None and prefill_chunk < 1:
            raise ValueError("prefill_chunk must be >= 1")
        self._cache = cache
        self._max_seqs = max_seqs
        self._budget = token_budget
        self._chunk = prefill_chunk
        self._book: dict[str, Sequence] = {}   # every request that has not left for good
        self._line: deque[Sequence] = deque()  # WAITING, head first
        self._live: list[Sequence] = []        # RUNNING, in admission order (the last one is the newest)
        self._cancelled: set[str] = set()

    # -- queries ------------------------------------------------------------
    @property
    def num_waiting(self) -> int:
        return len(self._line)

    @property
    def num_running(self) -> int:
        return len(self._live)

    def running(self) -> tuple[Sequence, ...]:
        """Running requests, oldest first."""
        return tuple(self._live)

    def waiting(self) -> tuple[Sequence, ...]:
        """The line, head first."""
        return tuple(self._line)

    def has_work(self) -> bool:
        return bool(self._line or self._live or self._cancelled)

    # -- requests in and out ------------------------------------------------
    def validate(self, seq: Sequence) -> None:
        """Raises what ``submit`` would raise, without taking the request."""
        if not seq.prompt_ids:
            raise ValueError("prompt_ids must be non-empty")
        if seq.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
        if seq.request_id in self._book:
            raise ValueError(f"duplicate request_id {seq.request_id}")
        # At worst the request holds every page it will ever need at the same time (scheduler.py:125-131).
        most = len(seq.prompt_ids) + seq.max_new_tokens
        if not self._cache.fits_ever(most):
            raise CacheExhausted(
                f"out of KV blocks: request of {most} tokens can never fit "
                f"(pool has {self._cache.total_pages()} pages per group)"
            )

    def submit(self, seq: Sequence) -> None:
        self.validate(seq)
        seq.state = SeqState.WAITING
        self._book[seq.request_id] = seq
        self._line.append(seq)

    def abort(self, request_id: str) -> None:
        """Takes effect at the next ``schedule()``; results in flight for the request are dropped."""
        if request_id in self._book:
            self._cancelled.add(request_id)

    def force_preempt(self, request_id: str) -> bool:
        """Send a running request back to the line now (for tests and experiments)."""
        seq = self._book.get(request_id)
        if seq is None or not seq.is_running:
            return False
        self._leave_running(seq, requeue=True)
        return True

    # -- the step -----------------------------------------------------------
    def schedule(self) -> StepPlan:
        self._drop_cancelled()
        self._make_room()
        self._admit()
        return StepPlan(self._deal())

    def complete(self, plan: StepPlan, sampled: SequenceT[int]) -> list[Emission]:
        """``sampled`` holds one token for every item of the plan with ``samples``, in order."""
        if len(sampled) != plan.num_samples:
            raise ValueError(f"the plan samples {plan.num_samples} tokens, got {len(sampled)}")
        feed = iter(sampled)
        emissions = []
        for item in plan.items:
            token = int(next(feed)) if item.samples else None
            seq = item.seq
            if seq.request_id in self._cancelled or not seq.is_running:
                continue  # aborted, sent back or finished while the step was in flight
            self._mark_cached(seq, item)
            if token is not None:
                seq.output_ids.append(token)
                emissions.append(self._take_token(seq, len(seq.output_ids) - 1))
        return emissions

    # -- a step ahead ---------------------------------------------------------
    # A decode step may be launched before the tokens of the step ahead of it have reached the host: the
    # device feeds them to it directly.  The earlier step is then booked provisionally (``assume``: one more
    # cached token and a placeholder where the unseen token will stand), the next step is planned as usual,
    # and the tokens are filled in when they arrive (``resolve``).  A request that turns out to have ended
    # with that token ends then; its row in the step launched meanwhile is ignored.
    def can_look_ahead(self, plan: StepPlan) -> bool:
        """True when the step after ``plan`` can be planned without ``plan``'s tokens: decoding only,
        nobody waiting or aborted, and no request that this step ends by length."""
        if self._line or self._cancelled or len(plan.items) != len(self._live) or not plan.items:
            return False
        return all(
            len(item.token_ids) == 1 and item.samples and item.seq.is_running
            and len(item.seq.output_ids) + 1 < item.seq.max_new_tokens
            for item in plan.items
        )

    def assume(self, plan: StepPlan) -> None:
        for item in plan.items:
            self._mark_cached(item.seq, item)
            item.seq.output_ids.append(self.PLACEHOLDER)

    def resolve(self, plan: StepPlan, sampled: SequenceT[int]) -> list[Emission]:
        """The tokens of a step booked with ``assume``: replaces the placeholders, ends what ended."""
        if len(sampled) != len(plan.items):
            raise ValueError(f"the plan samples {len(plan.items)} tokens, got {len(sampled)}")
        emissions = []
        for item, token in zip(plan.items, sampled):
            seq = item.seq
            index = item.past_len + 1 - len(seq.prompt_ids)  # where this step's token stands among the outputs
            stale = seq.state is SeqState.FINISHED or index >= len(seq.output_ids) or seq.output_ids[index] != self.PLACEHOLDER
            if stale:
                continue
            seq.output_ids[index] = int(token)
            if seq.request_id not in self._cancelled:
                emissions.append(self._take_token(seq, index))
        return emissions

    # -- internals ------------------------------------------------------------
    def _mark_cached(self, seq: Sequence, item: ScheduledSeq) -> None:
        seq.num_cached = item.past_len + len(item.token_ids)
        self._cache.trim(seq.seat, seq.num_cached)

    def _take_token(self, seq: Sequence, index: int) -> Emission:
        """Output ``index`` of ``seq`` is now known: decide whether the request ends with it."""
        token = seq.output_ids[index]
        if seq.eos_id is not None and token == seq.eos_id:
            seq.finish_reason = "eos"
        elif index + 1 >= seq.max_new_tokens:
            seq.finish_reason = "length"
        if seq.finish_reason is None:
            return Emission(seq, token, False)
        del seq.output_ids[index + 1 :]  # a placeholder of a step launched meanwhile
        if seq.is_running:
            self._leave_running(seq, requeue=False)
        else:  # sent back meanwhile: it waits in the line, holding nothing
            self._line.remove(seq)
            self._forget(seq)
        return Emission(seq, token, True)

    def _forget(self, seq: Sequence) -> None:
        seq.state = SeqState.FINISHED
        self._book.pop(seq.request_id, None)

    def _leave_running(self, seq: Sequence, requeue: bool) -> None:
        """The one way out of RUNNING: the seat and every page go back to the cache manager."""
        self._live.remove(seq)
        if seq.seat is not None:
            self._cache.close_seat(seq.seat)
            seq.seat = None
        if not requeue:
            self._forget(seq)
            return
        seq.num_cached = 0
        seq.preemptions += 1
        seq.state = SeqState.WAITING
        self._line.appendleft(seq)
        _log.info(
            "sequence preempted request_id=%s tokens=%s preemptions=%s", seq.request_id, seq.num_tokens, seq.preemptions
        )

    def _drop_cancelled(self) -> None:
        for request_id in self._cancelled:
            seq = self._book.get(request_id)
            if seq is None:
                continue
            seq.finish_reason = "aborted"
            if seq.is_running:
                self._leave_running(seq, requeue=False)
            else:
                self._line.remove(seq)
                self._forget(seq)
            _log.info("sequence aborted request_id=%s", request_id)
        self._cancelled.clear()

    def _make_room(self) -> None:
        """Pages for every running request's known tokens, oldest first; the newest pays when the pool is short."""
        position = 0
        while position < len(self._live):
            seq = self._live[position]
            while seq.is_running and not self._cache.grow(seq.seat, seq.num_tokens):
                self._leave_running(self._live[-1], requeue=True)  # may be seq itself
            position += seq.is_running

    def _share(self, pending: int, left: int) -> int:
        """How many of a request's ``pending`` prompt tokens fit into ``left`` tokens of budget."""
        room = max(left, 0)
        return min(pending, room, self._chunk or room)

    def _spoken_for(self) -> int:
        """Tokens of this step's budget that the running requests will take."""
        left = self._budget - sum(1 for seq in self._live if seq.num_pending == 1)
        for seq in self._live:
            if seq.num_pending > 1:
                left -= self._share(seq.num_pending, left)
        return self._budget - left

    def _admit(self) -> None:
        used = self._spoken_for()
        while self._line and len(self._live) < self._max_seqs and self._cache.free_seats > 0:
            seq = self._line[0]
            if used >= self._budget and self._live:
                break  # not one token of budget left for it; a request alone is always admitted
            if not self._cache.can_grow(None, seq.num_tokens):
                break
            seat = self._cache.open_seat()
            if not self._cache.grow(seat, seq.num_tokens):  # cannot happen after can_grow; stay safe
                self._cache.close_seat(seat)
                break
            self._line.popleft()
            seq.seat, seq.num_cached, seq.state = seat, 0, SeqState.RUNNING
            self._live.append(seq)
            used += self._share(seq.num_pending, self._budget - used)

    def _deal(self) -> list[ScheduledSeq]:
        decoding = [seq for seq in self._live if seq.num_pending == 1]
        items = [ScheduledSeq(seq, seq.tokens(seq.num_cached, seq.num_tokens), seq.num_cached, True) for seq in decoding]
        left = self._budget - len(decoding)  # decoding requests get their token whatever the budget
        for seq in self._live:  # portions of prompts, in admission order
            count = self._share(seq.num_pending, left) if seq.num_pending > 1 else 0
            if count:
                stop = seq.num_cached + count
                items.append(ScheduledSeq(seq, seq.tokens(seq.num_cached, stop), seq.num_cached, stop == seq.num_tokens))
                left -= count
        return items
