"""Greedy and temperature sampling, reproducible per request.

The reference takes the arg-max of float32 logits for ``temperature <= 0`` and
otherwise draws from ``softmax(logits / temperature)`` with the process-wide
generator, row by row (worker/src/inference/model_runner.py:122-130).  It has no
top-k, top-p or repetition penalty (the fields of its wire format are never
forwarded, worker/src/worker/servicer.py:74-80), so neither has this engine.

Here the draw inverts the cumulative distribution at a uniform number that is a
pure function of ``(seed, output index)`` of the request, so a request's tokens do
not depend on what else was in the batch, on how its prompt was cut, or on a
preemption in between.  The selection itself runs on the device; only token ids
come back.
"""

from __future__ import annotations

import torch

_MASK = (1 << 64) - 1


def uniform(seed: int, index: int) -> float:
    """A float32-exact uniform in [0, 1) from a 64-bit mix of (seed, index) (SplitMix64 finaliser)."""
    x = (int(seed) * 0x9E3779B97F4A7C15 + (int(index) + 1) * 0xD1B54A32D192ED03) & _MASK
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & _MASK
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _MASK
    x ^= x >> 31
    return (x >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, kernels) -> None:
        self.kernels = kernels

    def pick(self, logits: torch.Tensor, temperatures, uniforms, out: torch.Tensor | None = None) -> torch.Tensor:
        """Token ids (int32, on the device) for float32 ``logits [rows, vocab]``.

        ``temperatures`` and ``uniforms`` are float32 device tensors ``[rows]`` or
        ``None`` for all-greedy.
        """
        if out is None:
            out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        self.kernels.sample(logits, temperatures, uniforms, out)
        return out

    def pick_host(self, logits: torch.Tensor, temperatures, seeds, indices) -> list[int]:
        """Convenience for callers with Python lists: uploads the per-row numbers, returns ids."""
        rows = logits.shape[0]
        if all(t <= 0 for t in temperatures):
            return self.pick(logits, None, None).tolist()
        numbers = torch.tensor(
            [list(map(float, temperatures)), [uniform(s, i) for s, i in zip(seeds, indices)]],
            dtype=torch.float32,
        ).to(logits.device)
        return self.pick(logits, numbers[0], numbers[1]).tolist()[:rows]
