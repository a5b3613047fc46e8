"""Turning a step's entries into the device tensors the kernels read.

An entry is ``(seat, tokens, past_len, want)``: the next tokens of one request,
how many of its tokens are already cached, and the places among these tokens
whose logits are asked for.  Entries may be portions of prompts or single decoded
tokens, in any mix.  The layout puts single-token entries first (attention then
serves them with the split-KV kernel and the rest with the other), flattens the
tokens, and records for every token its position and its entry.

All integers of a step travel in one pinned buffer and one copy:
``token_ids [T] | positions [T] | token_seq [T] | seq_seat [B] | logit_rows [N]``
(the reference builds seven tensors per step with Python loops over every token,
worker/src/inference/qwen2/paged_attn.py:325-357).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from ..kernels.interface import Q_TILE, StepTensors
from ..parts.base import SeqSlice


@dataclass
class BatchEntry:
    seat: int
    tokens: Sequence[int]
    past_len: int
    want: Sequence[int] = field(default_factory=tuple)


@dataclass
class StepLayout:
    """Host-side result of laying a batch out; ``arrays`` is what goes to the device."""

    seqs: list[SeqSlice]
    num_tokens: int
    num_seqs: int
    num_decode_tokens: int
    num_rows: int
    max_kv_len: int
    packed: np.ndarray  # int32: token_ids | positions | token_seq | seq_seat | logit_rows | q_tiles
    num_q_tiles: int = 0


def lay_out(entries: Sequence[BatchEntry], vocab_size: int | None = None) -> StepLayout:
    if not entries:
        raise ValueError("a step needs at least one entry")
    order = sorted(range(len(entries)), key=lambda i: (len(entries[i].tokens) != 1, i))
    starts = [0] * len(entries)
    seqs: list[SeqSlice] = []
    cursor = 0
    decode_tokens = 0
    max_kv = 0
    for row, index in enumerate(order):
        entry = entries[index]
        q_len = len(entry.tokens)
        if q_len < 1 or entry.past_len < 0:
            raise ValueError("each entry needs at least one token and past_len >= 0")
        starts[index] = cursor
        seqs.append(SeqSlice(entry.seat, cursor, q_len, entry.past_len))
        if q_len == 1:
            decode_tokens += 1
        cursor += q_len
        max_kv = max(max_kv, entry.past_len + q_len)
    total = cursor
    rows = sum(len(e.want) for e in entries)
    tiles = [(s.start + at, min(Q_TILE, s.q_len - at)) for s in seqs if s.q_len > 1 for at in range(0, s.q_len, Q_TILE)]
    packed = np.empty(3 * total + len(entries) + rows + 2 * len(tiles), dtype=np.int32)
    ids, positions, token_seq = packed[:total], packed[total : 2 * total], packed[2 * total : 3 * total]
    seats = packed[3 * total : 3 * total + len(entries)]
    logit_rows = packed[3 * total + len(entries) : 3 * total + len(entries) + rows]
    if tiles:
        packed[3 * total + len(entries) + rows :] = np.asarray(tiles, dtype=np.int32).reshape(-1)
    for row, index in enumerate(order):
        entry = entries[index]
        s, n = starts[index], len(entry.tokens)
        ids[s : s + n] = entry.tokens
        positions[s : s + n] = np.arange(entry.past_len, entry.past_len + n, dtype=np.int32)
        token_seq[s : s + n] = row
        seats[row] = entry.seat
    at = 0
    for index, entry in enumerate(entries):  # rows in the caller's order of entries and of want
        for place in entry.want:
            if not 0 <= place < len(entry.tokens):
                raise ValueError(f"want {place} outside the {len(entry.tokens)} tokens of its entry")
            logit_rows[at] = starts[index] + place
            at += 1
    if vocab_size is not None and total and (ids.min() < 0 or ids.max() >= vocab_size):
        raise ValueError(f"token id outside [0, {vocab_size})")
    return StepLayout(seqs, total, len(entries), decode_tokens, rows, max_kv, packed, len(tiles))


class StepStaging:
    """Pinned host buffers (two, used in turn) and the device buffer a step's integers live in."""

    def __init__(self, capacity: int, device: torch.device) -> None:
        self.capacity = capacity
        self.device = device
        pin = device.type == "cuda"
        self._host = [torch.empty(capacity, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        # A pinned buffer is rewritten only after the copy that last read it has run.
        self._copied = [torch.cuda.Event() if pin else None for _ in range(2)]
        self._turn = 0
        self.device_buffer = torch.empty(capacity, dtype=torch.int32, device=device)

    def upload(self, layout: StepLayout) -> tuple[StepTensors, torch.Tensor]:
        n = layout.packed.shape[0]
        if n > self.capacity:
            raise ValueError(f"step needs {n} integers of staging, capacity is {self.capacity}")
        host, copied = self._host[self._turn], self._copied[self._turn]
        self._turn ^= 1
        if copied is not None:
            copied.synchronize()
        host.numpy()[:n] = layout.packed
        self.device_buffer[:n].copy_(host[:n], non_blocking=True)
        if copied is not None:
            copied.record()
        return views(self.device_buffer, layout)


def views(buffer: torch.Tensor, layout: StepLayout) -> tuple[StepTensors, torch.Tensor]:
    t, b = layout.num_tokens, layout.num_seqs
    step = StepTensors(
        token_ids=buffer[:t],
        positions=buffer[t : 2 * t],
        token_seq=buffer[2 * t : 3 * t],
        seq_seat=buffer[3 * t : 3 * t + b],
        num_tokens=t,
        num_seqs=b,
        num_decode_tokens=layout.num_decode_tokens,
        max_kv_len=layout.max_kv_len,
    )
    rows_end = 3 * t + b + layout.num_rows
    if layout.num_q_tiles:
        step.q_tiles = buffer[rows_end : rows_end + 2 * layout.num_q_tiles]
        step.num_q_tiles = layout.num_q_tiles
    return step, buffer[3 * t + b : rows_end]
