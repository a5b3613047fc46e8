"""Where each scheduler step spends its time, logged every N steps.

The split follows the reference's (worker/src/inference/step_stats.py:1-19):
``sched`` (planning the step), ``gpu`` (the forward and sampling, ending with the
copy of the token ids to the host), ``emit`` (appending tokens, finishing
requests, callbacks); ``gpu`` is further split into ``kernel`` (between two CUDA
events around the launches) and ``host = gpu - kernel``.  Steps are grouped by
kind: ``decode`` (every request decodes one token) and ``prefill`` (any other).
There is no ``wait`` part: this engine has no event loop between the parts.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass, field

_log = logging.getLogger(__name__)

PARTS = ("sched", "gpu", "emit")


@dataclass
class _Group:
    steps: int = 0
    rows: int = 0
    tokens: int = 0
    ms: dict = field(default_factory=lambda: dict.fromkeys(PARTS, 0.0))
    kernel_ms: float = 0.0
    kernel_steps: int = 0
    kernel_gpu_ms: float = 0.0

    def total_ms(self) -> float:
        return sum(self.ms.values())


class StepStats:
    def __init__(self, every: int) -> None:
        if every < 1:
            raise ValueError("step stats interval must be >= 1")
        self.every = every
        self._groups: dict[str, _Group] = {}
        self._steps = 0
        self.lines: list[str] = []

    def record(self, kind: str, rows: int, tokens: int, kernel: float | None = None, **parts_ms: float) -> None:
        missing = set(PARTS) - set(parts_ms)
        if missing:
            raise ValueError(f"missing step parts: {sorted(missing)}")
        group = self._groups.setdefault(kind, _Group())
        group.steps += 1
        group.rows += rows
        group.tokens += tokens
        for name in PARTS:
            group.ms[name] += parts_ms[name]
        if kernel is not None:
            group.kernel_ms += kernel
            group.kernel_steps += 1
            group.kernel_gpu_ms += parts_ms["gpu"]
        self._steps += 1
        if self._steps >= self.every:
            self.flush()

    def flush(self) -> str | None:
        if self._steps == 0:
            return None
        line = self.format()
        _log.info("%s", line)
        self.lines.append(line)
        self._groups.clear()
        self._steps = 0
        return line

    def format(self) -> str:
        wall = sum(g.total_ms() for g in self._groups.values()) or 1.0
        pieces = [f"step stats steps={self._steps}"]
        for kind in sorted(self._groups):
            g = self._groups[kind]
            n = g.steps
            avg = " ".join(f"{name}={g.ms[name] / n:.2f}" for name in PARTS)
            if g.kernel_steps:
                kernel = g.kernel_ms / g.kernel_steps
                host = (g.kernel_gpu_ms - g.kernel_ms) / g.kernel_steps
                avg += f" (kernel={kernel:.2f} host={host:.2f})"
            pieces.append(
                f"{kind} n={n} rows={g.rows / n:.1f} tok={g.tokens / n:.0f} "
                f"ms/step[{avg}] share={100 * g.total_ms() / wall:.0f}%"
            )
        totals = {name: sum(g.ms[name] for g in self._groups.values()) for name in PARTS}
        pieces.append("wall " + " ".join(f"{name}={100 * totals[name] / wall:.0f}%" for name in PARTS))
        return " | ".join(pieces)
