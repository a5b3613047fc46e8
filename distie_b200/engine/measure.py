"""Measuring helpers.  Nothing here is on the path of generation or of trace replay.

``DecodeBurst`` times the decode step itself: K steps of a batch back to back on
the device, each feeding the next, with no trip to the host in between.  It drives
the runner's own captured decode step (the same model, cache, kernels and bucket
buffers that generation replays) inside a graph of its own that also moves the
positions on by one, which generation does on the host.
"""

from __future__ import annotations

import torch

from .runner import ModelRunner


class DecodeBurst:
    def __init__(self, runner: ModelRunner) -> None:
        self.runner = runner
        self._graphs: dict[int, tuple[torch.cuda.CUDAGraph, torch.Tensor]] = {}  # bucket size -> (graph, advance)

    @torch.inference_mode()
    def run(self, items, steps: int) -> torch.Tensor:
        """``steps`` greedy decode steps for ``items`` (one token each, as a scheduler plans them).

        The caller has grown every request's pages for ``past_len + steps`` tokens beforehand and
        does its own bookkeeping afterwards (the scheduler never sees the tokens).  Returns the
        sampled tokens ``[steps, rows]`` (int32, on the device).
        """
        runner = self.runner
        if any(item.seq.temperature > 0 or len(item.token_ids) != 1 for item in items):
            raise ValueError("a burst decodes greedily, one token per request and step")
        if not runner.use_graphs:
            raise RuntimeError("a burst replays captured decode steps: the runner has its graphs switched off")
        if runner.cache.states:
            raise RuntimeError("a burst runs its first step twice, which per-request state does not survive")
        rows = [(item.token_ids[0], item.past_len, item.seq.seat, 0.0, 0.0) for item in items]
        # Stage the rows and make sure the bucket's step is captured (this runs the first step once more than
        # asked: same tokens, same slots), then stage again, because the step fed its tokens back as ids.
        bucket = runner._replay(rows, ids_on_device=False)
        if bucket is None:
            raise RuntimeError("the decode step could not be captured")
        bucket.upload()
        size = bucket.size
        if size not in self._graphs:
            advance = torch.zeros(size, dtype=torch.int32, device=runner.device)
            advance[: len(rows)] = 1
            torch.cuda.synchronize(runner.device)
            graph = torch.cuda.CUDAGraph()
            logits = bucket.logits  # the runner's own graph keeps writing these; the burst's graph gets its own
            with torch.cuda.graph(graph, pool=runner._graph_pool):
                runner._forward_bucket(bucket)                      # the step; leaves its tokens as the next ids
                bucket.ints[size : 2 * size].add_(advance)          # and every live row moves on by one position
            bucket.logits = logits
            self._graphs[size] = (graph, advance)
        graph, advance = self._graphs[size]
        advance.zero_()
        advance[: len(rows)] = 1
        out = torch.empty((steps, size), dtype=torch.int32, device=runner.device)
        for k in range(steps):
            graph.replay()
            out[k].copy_(bucket.tokens)
        runner.graph_replays += steps
        runner.steps += steps
        return out[:, : len(rows)]

    def kernels_per_step(self, rows: int) -> int:
        """Own kernels inside the captured step of the bucket that ``rows`` requests use."""
        bucket = self.runner._buckets.get(self.runner.bucket_for(rows))
        return bucket.kernels_per_replay if bucket is not None else 0
