"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

``ModelRunner.step(entries)`` runs only the tokens it is given, as one batch,
against what earlier steps left in the cache, and returns float32 logits
``[wanted, vocab]`` on the device.  Trace replay and generation both go through
it; generation adds sampling on the device (``run_plan``).  A step in which every
entry is a single token replays the captured decode step of its bucket in both.

Steps in which every request decodes one token are replayed from CUDA graphs, one
per batch-size bucket, like the reference's (worker/src/inference/qwen2/
batch_decode.py:1-17): the batch is rounded up to a bucket (1, 2, 4, 8, then steps
of 8), padding rows decode token 0 at position 0 of the padding seat, whose block
table names a spare page the pool never hands out.  Everything a captured step
reads sits in fixed device buffers that are refilled before each replay.
"""

from __future__ import annotations

import bisect
import logging
from typing import Sequence

import numpy as np
import torch

from ..sampling.sampler import Sampler, uniform
from .batch import BatchEntry, StepLayout, StepStaging, lay_out, views

_log = logging.getLogger(__name__)


def decode_buckets(max_batch: int) -> tuple[int, ...]:
    """Powers of two up to 8, then steps of 8, then ``max_batch`` (batch_decode.py:42-49)."""
    if max_batch < 1:
        raise ValueError("max_batch must be >= 1")
    sizes = {b for b in (1, 2, 4, 8) if b < max_batch}
    sizes.update(range(16, max_batch, 8))
    sizes.add(max_batch)
    return tuple(sorted(sizes))


class _Bucket:
    def __init__(self, size: int, device: torch.device) -> None:
        self.size = size
        # token_ids | positions | token_seq | seq_seat | logit_rows, each `size` long
        self.ints = torch.zeros(5 * size, dtype=torch.int32, device=device)
        self.floats = torch.zeros(2 * size, dtype=torch.float32, device=device)  # temperatures | uniforms
        self.tokens = torch.zeros(size, dtype=torch.int32, device=device)
        self.logits: torch.Tensor | None = None
        self.graph: torch.cuda.CUDAGraph | None = None
        self.kernels_per_replay = 0  # own kernels inside the captured step
        pin = device.type == "cuda"
        self.host_ints = torch.zeros(5 * size, dtype=torch.int32, pin_memory=pin)
        self.host_floats = torch.zeros(2 * size, dtype=torch.float32, pin_memory=pin)
        self.layout = StepLayout([], size, size, size, size, 0, np.zeros(0, dtype=np.int32))
        self.copied = torch.cuda.Event() if pin else None  # the pinned buffers wait for it before they change
        # Sampled tokens and the kernels' error word on their way back, two sets used in turn: a step may be
        # launched before the one ahead of it has been read.
        self.result_host = [torch.zeros(size + 1, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self.result_ready = [torch.cuda.Event() if pin else None for _ in range(2)]
        self.turn = 0

    def before_write(self) -> None:
        if self.copied is not None:
            self.copied.synchronize()

    def upload(self, ids_on_device: bool = False) -> None:
        """Host staging to the device; with ``ids_on_device`` the token ids the last replay left there stay."""
        if ids_on_device:
            self.ints[self.size :].copy_(self.host_ints[self.size :], non_blocking=True)
        else:
            self.ints.copy_(self.host_ints, non_blocking=True)
        self.floats.copy_(self.host_floats, non_blocking=True)
        if self.copied is not None:
            self.copied.record()


class ModelRunner:
    def __init__(self, model, cache, max_step_tokens: int, max_seqs: int, decode_graphs: bool = True) -> None:
        self.model = model
        self.cache = cache
        self.kernels = model.kernels
        self.device = self.kernels.device
        self.sampler = Sampler(self.kernels)
        self.max_step_tokens = max_step_tokens
        self.max_seqs = max_seqs
        self.staging = StepStaging(5 * max_step_tokens + 3 * max_seqs, self.device)
        self._floats_host = [
            torch.zeros(2 * max_seqs, dtype=torch.float32, pin_memory=self.device.type == "cuda") for _ in range(2)
        ]
        self._floats_turn = 0
        self._floats_device = torch.zeros(2 * max_seqs, dtype=torch.float32, device=self.device)
        graph_safe = all(getattr(block, "graph_safe", True) for block in model.blocks)
        self.use_graphs = bool(decode_graphs) and self.device.type == "cuda" and graph_safe
        self._sizes = decode_buckets(max_seqs)
        self._buckets: dict[int, _Bucket] = {}
        self._graph_pool = None
        self.graph_replays = 0
        self.steps = 0

    # -- the step function ----------------------------------------------------
    @torch.inference_mode()
    def step(self, entries: Sequence[BatchEntry]) -> torch.Tensor | None:
        if self.use_graphs and len(entries) <= self._sizes[-1] and all(len(e.tokens) == 1 for e in entries):
            logits = self._graph_logits(entries)
            if logits is not NotImplemented:
                return logits
        layout = lay_out(entries, self.model.vocab_size)
        if layout.num_tokens > self.max_step_tokens or layout.num_seqs > self.max_seqs:
            raise ValueError(
                f"step of {layout.num_tokens} tokens / {layout.num_seqs} requests exceeds the runner's "
                f"limits ({self.max_step_tokens} / {self.max_seqs})"
            )
        self.cache.upload_tables([s.seat for s in layout.seqs])
        step, rows = self.staging.upload(layout)
        self.steps += 1
        return self.model.forward(step, layout.seqs, self.cache, rows if layout.num_rows else None)

    def _graph_logits(self, entries: Sequence[BatchEntry]):
        """A step of single tokens through the captured decode step of its bucket: the logits of the
        wanted entries, or ``NotImplemented`` when no graph could be made (every step is eager from then on)."""
        vocab = self.model.vocab_size
        for entry in entries:
            if not 0 <= entry.tokens[0] < vocab or entry.past_len < 0:
                raise ValueError(f"token id outside [0, {vocab}) or past_len < 0")
            if any(place != 0 for place in entry.want):
                raise ValueError("want outside the one token of its entry")
        rows = [(entry.tokens[0], entry.past_len, entry.seat, 0.0, 0.0) for entry in entries]
        bucket = self._replay(rows, ids_on_device=False)
        if bucket is None:
            return NotImplemented
        self.steps += 1
        wanted = [row for row, entry in enumerate(entries) for _ in entry.want]
        if not wanted:
            return None
        if wanted == list(range(len(wanted))):
            return bucket.logits[: len(wanted)].clone()
        return bucket.logits.index_select(0, torch.tensor(wanted, dtype=torch.long, device=self.device))

    def finish_step(self) -> None:
        """After the step's results reached the host: surface device-side checks."""
        self.kernels.check_errors()

    # -- generation: plan in, one token per sampling item out -----------------
    @torch.inference_mode()
    def run_plan(self, plan) -> list[int]:
        items = plan.items
        if not items:
            raise ValueError("empty step plan")
        sampling = [item for item in items if item.samples]
        if self.can_launch_decode(items):
            handle = self.launch_decode(items)
            if handle is not None:
                return self.fetch_decode(handle)  # a device-side check that fails here is the request's, not the graph's
        entries = [
            BatchEntry(i.seq.seat, i.token_ids, i.past_len, (len(i.token_ids) - 1,) if i.samples else ())
            for i in items
        ]
        logits = self.step(entries)
        if not sampling:
            self.finish_step()
            return []
        temps, uniforms = self._sampling_numbers(sampling)
        tokens = self.sampler.pick(logits, temps, uniforms).tolist()
        self.finish_step()
        return tokens

    def _sampling_numbers(self, sampling):
        if all(item.seq.temperature <= 0 for item in sampling):
            return None, None
        n = len(sampling)
        host = self._floats_host[self._floats_turn]
        self._floats_turn ^= 1
        array = host.numpy()  # rewritten two steps later at the earliest, and every sampling step ends with a sync
        for row, item in enumerate(sampling):
            array[row] = max(0.0, float(item.seq.temperature))
            array[n + row] = uniform(item.seq.seed, len(item.seq.output_ids))
        self._floats_device[: 2 * n].copy_(host[: 2 * n], non_blocking=True)
        return self._floats_device[:n], self._floats_device[n : 2 * n]

    # -- decode graphs ------------------------------------------------------
    def bucket_for(self, rows: int) -> int:
        if rows < 1 or rows > self._sizes[-1]:
            raise ValueError(f"decode batch of {rows} rows outside 1..{self._sizes[-1]}")
        return self._sizes[bisect.bisect_left(self._sizes, rows)]

    def can_launch_decode(self, items) -> bool:
        """Whether ``launch_decode`` takes these items: graphs on, one token each, a bucket large enough."""
        return bool(
            self.use_graphs and items and len(items) <= self._sizes[-1] and all(len(i.token_ids) == 1 for i in items)
        )

    @torch.inference_mode()
    def launch_decode(self, items, ids_on_device: bool = False):
        """Starts a decode step (graph replay) and returns a handle for ``fetch_decode``; does not wait.
        Returns None when the bucket's graph could not be captured: graphs are off from then on and the
        caller runs the step eagerly (which rewrites the same slots).

        With ``ids_on_device`` the rows' token ids are the tokens that the previous replay of
        the same bucket sampled for the same rows (they never left the device); everything
        else -- positions, seats, block tables, sampling numbers -- comes from the host as usual.
        """
        rows = [
            (
                max(0, item.token_ids[0]), item.past_len, item.seq.seat,
                float(item.seq.temperature) if item.seq.temperature > 0 else 0.0,
                uniform(item.seq.seed, len(item.seq.output_ids)) if item.seq.temperature > 0 else 0.0,
            )
            for item in items
        ]
        bucket = self._replay(rows, ids_on_device)
        if bucket is None:
            return None
        size = bucket.size
        self.steps += 1
        turn = bucket.turn
        bucket.turn ^= 1
        host = bucket.result_host[turn]
        host[:size].copy_(bucket.tokens, non_blocking=True)
        flag = getattr(self.kernels, "error_flag", None)
        if flag is not None:
            host[size:].copy_(flag, non_blocking=True)
        else:
            host[size:] = 0
        if bucket.result_ready[turn] is not None:
            bucket.result_ready[turn].record()
        return bucket, turn, [item.samples for item in items]

    def _replay(self, rows, ids_on_device: bool):
        """Stage ``rows`` of (token, past_len, seat, temperature, uniform) into their bucket and replay its
        captured step (capturing it first when new).  None: capture or replay failed, graphs are now off."""
        size = self.bucket_for(len(rows))
        bucket = self._buckets.get(size)
        if bucket is None:
            bucket = _Bucket(size, self.device)
            self._buckets[size] = bucket
        bucket.before_write()
        ints = bucket.host_ints.numpy()
        floats = bucket.host_floats.numpy()
        ids, positions, token_seq = ints[:size], ints[size : 2 * size], ints[2 * size : 3 * size]
        seats, logit_rows = ints[3 * size : 4 * size], ints[4 * size :]
        ids[:] = 0
        positions[:] = 0
        seats[:] = self.cache.pad_seat
        token_seq[:] = np.arange(size, dtype=np.int32)
        logit_rows[:] = np.arange(size, dtype=np.int32)
        floats[:] = 0.0
        for row, (token, past_len, seat, temperature, draw) in enumerate(rows):
            ids[row] = token
            positions[row] = past_len
            seats[row] = seat
            floats[row] = temperature
            floats[size + row] = draw
        self.cache.upload_tables([row[2] for row in rows])
        bucket.upload(ids_on_device and bucket.graph is not None)
        if bucket.graph is None and ids_on_device:
            raise RuntimeError("token ids on the device need a replay of the same bucket before")
        try:
            if bucket.graph is None:
                self._capture(bucket)
            else:
                bucket.graph.replay()
                self.graph_replays += 1
        except Exception:  # noqa: BLE001  (capture and replay only; device-side checks surface in fetch_decode)
            _log.exception("decode graph failed; every step stays eager from now on")
            self.use_graphs = False
            self._buckets.pop(size, None)
            return None
        return bucket

    def fetch_decode(self, handle) -> list[int]:
        """The sampled tokens of a launched decode step (waits for them), after the device-side checks."""
        bucket, turn, samples = handle
        if bucket.result_ready[turn] is not None:
            bucket.result_ready[turn].synchronize()
        host = bucket.result_host[turn].tolist()
        if host[bucket.size]:
            self.kernels.check_errors()  # raises with the code's text and clears the word
        return [token for token, wanted in zip(host, samples) if wanted]

    def _forward_bucket(self, bucket: _Bucket) -> None:
        layout = bucket.layout
        layout.max_kv_len = self.cache.max_tokens_per_request  # a fixed bound: the graph must not depend on lengths
        step, rows = views(bucket.ints, layout)
        bucket.logits = self.model.forward(step, (), self.cache, rows)
        size = bucket.size
        self.sampler.pick(bucket.logits, bucket.floats[:size], bucket.floats[size:], bucket.tokens)
        # The sampled tokens are also the next step's token ids, should it be launched before they reach the host.
        bucket.ints[:size].copy_(bucket.tokens)

    def _capture(self, bucket: _Bucket) -> None:
        # Warm up on a side stream (library workspaces, lazy kernel loading), then capture.
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ids = bucket.ints[: bucket.size].clone()
            # The warm-up runs the step for real.  Keys and values it writes are the ones the replay writes
            # again; per-request state is not idempotent, so it is put back as it was.
            states = {slot: state.clone() for slot, state in self.cache.states.items()}
            self._forward_bucket(bucket)
            for slot, state in states.items():
                self.cache.states[slot].copy_(state)
            bucket.ints[: bucket.size].copy_(ids)  # the warm-up fed its tokens back; the replay starts from the step's own ids
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(self.device)
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        graph = torch.cuda.CUDAGraph()
        before = self.kernels.launches
        with torch.cuda.graph(graph, pool=self._graph_pool):
            self._forward_bucket(bucket)
        bucket.kernels_per_replay = self.kernels.launches - before
        bucket.graph = graph
        graph.replay()
        _log.info("decode graph captured bucket=%s", bucket.size)
