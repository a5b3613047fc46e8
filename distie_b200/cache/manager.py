"""The cache manager: pages of keys and values, block tables, seats, state slots.

Control plane and data plane are separate, as in the reference (worker/src/
inference/kv_cache.py:1-10): a native pool hands out page ids only; the keys and
values live in one device slab per group, indexed by those ids.

* A **group** is a set of cache slots (layers) with the same need: kv heads, head
  size, and either all keys or a window of them.  Each group has its own pool,
  slab and block tables, so a windowed group can give pages back while a full
  group keeps them.
* A **seat** is what a live request holds: row ``seat`` of every group's block
  table and slot ``seat`` of every per-request state tensor.  ``close_seat``
  returns the pages of all groups and the seat.
* ``grow(seat, n)`` makes sure the pages for positions ``< n`` exist in every
  group, all or nothing.  ``trim(seat, n)`` returns the pages of windowed groups
  that no position ``>= n`` can see any more.
* Slab layout per group: ``[slot, 2 (k|v), page, kv_head, page_size, head_dim]``
  with one spare page past the pool's range (id ``num_pages``) that padded rows of
  a captured decode step write to (the reference's spare page,
  worker/src/inference/torch_engine.py:439-446).  Row ``max_seats`` of each table
  is the padding seat: all its entries name the spare page.
* State slots: one tensor ``[max_seats + 1, *shape]`` per slot that declares a
  :class:`~distie_b200.parts.base.StateNeed`, zeroed when a seat is opened.  The
  Qwen2 decoder declares none; the structure is there all the same.

With ``device=None`` the manager keeps only the bookkeeping (no slabs), which is
what the scheduler tests and sizing estimates use.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Mapping

import numpy as np
import torch

from ..kernels.interface import KvSlot
from ..parts.base import CacheNeed, StateNeed


class CacheExhausted(RuntimeError):
    """No free seat, or a request that can never fit the pool."""


def pages_needed(tokens: int, page_size: int) -> int:
    if page_size < 1:
        raise ValueError("page_size must be >= 1")
    return 0 if tokens <= 0 else (tokens + page_size - 1) // page_size


def pages_that_fit(cache_needs, page_size: int, element_size: int, budget_bytes: int) -> int:
    """How many pages per group ``budget_bytes`` of device memory hold (the spare page of every slab included
    in the budget, not in the count): every cache slot keeps keys and values of its own for each page id."""
    per_page = sum(2 * need.num_kv_heads * need.head_dim * element_size * page_size for need in cache_needs.values())
    if per_page <= 0:
        raise ValueError("the model declares no cache to size")
    return int(budget_bytes // per_page) - 1


@dataclass
class _SeatPages:
    first: int = 0   # logical index of the first page still held
    ids: list | None = None  # page ids of logical pages first, first + 1, ...

    def __post_init__(self) -> None:
        if self.ids is None:
            self.ids = []


class KvGroup:
    def __init__(self, need: CacheNeed, slots: tuple[int, ...], num_pages: int, page_size: int, max_seats: int,
                 table_width: int, pool) -> None:
        self.need = need
        self.slots = slots
        self.num_pages = num_pages
        self.page_size = page_size
        self.table_width = table_width
        self.pool = pool
        self.seats: dict[int, _SeatPages] = {}
        self.host_table = np.full((max_seats + 1, table_width), -1, dtype=np.int32)
        self.host_table[max_seats, :] = num_pages  # padding seat -> spare page
        self.dirty: dict[int, int] = {}  # seat -> first column that changed since the last upload
        self.slab: torch.Tensor | None = None
        self.device_table: torch.Tensor | None = None
        self._host_tensor: torch.Tensor | None = None
        self._views: dict[int, KvSlot] = {}
        self._uploaded = None  # CUDA event after the last upload: the pinned table waits for it before it changes

    def bytes_per_token(self, element_size: int) -> int:
        return 2 * len(self.slots) * self.need.num_kv_heads * self.need.head_dim * element_size

    # -- bookkeeping --------------------------------------------------------
    def first_needed_page(self, cached: int) -> int:
        """Logical index of the first page a position >= cached can still see."""
        if self.need.window is None:
            return 0
        first_key = max(0, cached - int(self.need.window) + 1)
        return first_key // self.page_size

    def missing(self, seat: int | None, tokens: int) -> int:
        held = self.seats.get(seat) if seat is not None else None
        end = pages_needed(tokens, self.page_size)
        if held is None:
            return end
        return max(0, end - (held.first + len(held.ids)))

    def _mark(self, seat: int, column: int) -> None:
        self.dirty[seat] = min(self.dirty.get(seat, column), column)

    def _before_write(self) -> None:
        if self._uploaded is not None:
            self._uploaded.synchronize()

    def grow(self, seat: int, tokens: int) -> None:
        held = self.seats.setdefault(seat, _SeatPages())
        count = self.missing(seat, tokens)
        if count == 0:
            return
        start = held.first + len(held.ids)
        if start + count > self.table_width:
            raise CacheExhausted(
                f"{tokens} tokens need {start + count} pages per request, block tables hold {self.table_width}"
            )
        ids = list(self.pool.allocate(count))
        held.ids.extend(ids)
        self._before_write()
        self.host_table[seat, start : start + count] = ids
        self._mark(seat, start)

    def trim(self, seat: int, cached: int) -> int:
        held = self.seats.get(seat)
        if held is None or self.need.window is None:
            return 0
        keep_from = min(self.first_needed_page(cached), held.first + len(held.ids))
        drop = keep_from - held.first
        if drop <= 0:
            return 0
        self.pool.free(held.ids[:drop])
        self._before_write()
        self.host_table[seat, held.first : keep_from] = -1
        self._mark(seat, held.first)
        del held.ids[:drop]
        held.first = keep_from
        return drop

    def release(self, seat: int) -> None:
        held = self.seats.pop(seat, None)
        if held is None:
            return
        if held.ids:
            self.pool.free(held.ids)
        self._before_write()
        self.host_table[seat, :] = -1
        self._mark(seat, 0)

    def pages_of(self, seat: int) -> list[int]:
        held = self.seats.get(seat)
        return list(held.ids) if held else []

    # -- device side --------------------------------------------------------
    def allocate_device(self, dtype: torch.dtype, device: torch.device) -> None:
        shape = (len(self.slots), 2, self.num_pages + 1, self.need.num_kv_heads, self.page_size, self.need.head_dim)
        self.slab = torch.zeros(shape, dtype=dtype, device=device)
        self._host_tensor = torch.from_numpy(self.host_table)
        if device.type == "cuda":
            self._host_tensor = self._host_tensor.pin_memory()
            self.host_table = self._host_tensor.numpy()  # keep writing into the pinned copy
        self.device_table = self._host_tensor.to(device, non_blocking=False).clone()
        self.dirty.clear()

    def upload(self, seats) -> None:
        if self.device_table is None:
            return
        copied = False
        for seat in seats:
            column = self.dirty.pop(seat, None)
            if column is None:
                continue
            self.device_table[seat, column:].copy_(self._host_tensor[seat, column:], non_blocking=True)
            copied = True
        if copied and self.device_table.is_cuda:
            if self._uploaded is None:
                self._uploaded = torch.cuda.Event()
            self._uploaded.record()

    def slot_view(self, slot: int) -> KvSlot:
        view = self._views.get(slot)
        if view is None:
            index = self.slots.index(slot)
            view = KvSlot(self.slab[index, 0], self.slab[index, 1], self.device_table, self.page_size, self.num_pages + 1)
            self._views[slot] = view
        return view


class CacheManager:
    def __init__(
        self,
        cache_needs: Mapping[int, CacheNeed],
        state_needs: Mapping[int, StateNeed] | None = None,
        *,
        num_pages: int,
        page_size: int,
        max_seats: int,
        max_tokens_per_request: int,
        dtype: torch.dtype = torch.bfloat16,
        device=None,
        pool_factory: Callable[[int], object] | None = None,
    ) -> None:
        if num_pages < 1 or page_size < 1 or max_seats < 1 or max_tokens_per_request < 1:
            raise ValueError("num_pages, page_size, max_seats and max_tokens_per_request must be >= 1")
        if pool_factory is None:
            from .block_pool import BlockPool as pool_factory
        self.page_size = page_size
        self.max_seats = max_seats
        self.pad_seat = max_seats
        self.max_tokens_per_request = max_tokens_per_request
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else None
        width = pages_needed(max_tokens_per_request, page_size)
        by_need: dict[CacheNeed, list[int]] = {}
        for slot in sorted(cache_needs):
            by_need.setdefault(cache_needs[slot], []).append(slot)
        self.groups = [
            KvGroup(need, tuple(slots), num_pages, page_size, max_seats, width, pool_factory(num_pages))
            for need, slots in by_need.items()
        ]
        self._group_of = {slot: group for group in self.groups for slot in group.slots}
        self.state_needs = dict(state_needs or {})
        self.states: dict[int, torch.Tensor] = {}
        self._free_seats = list(range(max_seats - 1, -1, -1))
        self._open: set[int] = set()
        if self.device is not None:
            for group in self.groups:
                group.allocate_device(dtype, self.device)
            for slot, need in self.state_needs.items():
                self.states[slot] = torch.zeros((max_seats + 1, *need.shape), dtype=need.dtype, device=self.device)

    # -- seats --------------------------------------------------------------
    @property
    def free_seats(self) -> int:
        return len(self._free_seats)

    def open_seat(self) -> int:
        if not self._free_seats:
            raise CacheExhausted(f"all {self.max_seats} seats are taken")
        seat = self._free_seats.pop()
        self._open.add(seat)
        for state in self.states.values():
            state[seat].zero_()
        return seat

    def close_seat(self, seat: int) -> None:
        if seat not in self._open:
            raise ValueError(f"seat {seat} is not open")
        for group in self.groups:
            group.release(seat)
        self._open.remove(seat)
        self._free_seats.append(seat)

    def reset_seat(self, seat: int) -> None:
        """Give back the pages and clear the state but keep the seat (recompute from position 0)."""
        if seat not in self._open:
            raise ValueError(f"seat {seat} is not open")
        for group in self.groups:
            group.release(seat)
        for state in self.states.values():
            state[seat].zero_()

    # -- pages --------------------------------------------------------------
    def fits_ever(self, tokens: int) -> bool:
        if tokens > self.max_tokens_per_request:
            return False
        return all(pages_needed(tokens, g.page_size) <= g.num_pages for g in self.groups)

    def can_grow(self, seat: int | None, tokens: int) -> bool:
        return all(g.missing(seat, tokens) <= g.pool.num_free for g in self.groups)

    def grow(self, seat: int, tokens: int) -> bool:
        """Pages for positions < tokens in every group, all or nothing."""
        if seat not in self._open:
            raise ValueError(f"seat {seat} is not open")
        if tokens > self.max_tokens_per_request:
            raise CacheExhausted(f"{tokens} tokens exceed the longest request the tables hold ({self.max_tokens_per_request})")
        if not self.can_grow(seat, tokens):
            return False
        for group in self.groups:
            group.grow(seat, tokens)
        return True

    def trim(self, seat: int, cached: int) -> int:
        return sum(group.trim(seat, cached) for group in self.groups)

    def free_pages(self) -> int:
        return min((int(g.pool.num_free) for g in self.groups), default=0)

    def total_pages(self) -> int:
        return min((g.num_pages for g in self.groups), default=0)

    def pages_held(self, seat: int) -> dict[int, list[int]]:
        return {i: g.pages_of(seat) for i, g in enumerate(self.groups)}

    def bytes_per_token(self) -> int:
        size = torch.empty((), dtype=self.dtype).element_size()
        return sum(g.bytes_per_token(size) for g in self.groups)

    # -- what a step sees -----------------------------------------------------
    def upload_tables(self, seats) -> None:
        for group in self.groups:
            group.upload(seats)

    def kv_slot(self, slot: int) -> KvSlot | None:
        group = self._group_of.get(slot)
        return group.slot_view(slot) if group is not None else None

    def state_slot(self, slot: int):
        return self.states.get(slot)
