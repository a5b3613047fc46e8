"""Where each scheduler step spends its time, logged every N steps.

The parts of a step are the reference's (worker/src/inference/step_stats.py:1-19):
``sched`` (planning the step), ``gpu`` (the forward and sampling, ending with the
copy of the token ids to the host) and ``emit`` (appending tokens, ending requests,
callbacks); ``gpu`` divides into ``kernel`` (between two CUDA events around the
launches) and ``host = gpu - kernel``.  Steps are grouped by kind: ``decode`` (every
request brings one token) and ``prefill`` (any other).  The reference's fourth part,
``wait``, is the time its event loop takes to resume; this engine has no event loop.

A window keeps one record per step; ``summary`` reduces the window to plain numbers
per kind (which measuring code reads) and ``format`` renders them as the log line,
laid out like the reference's (step_stats.py:82-100).
"""

from __future__ import annotations

import logging
from typing import NamedTuple

_log = logging.getLogger(__name__)

PARTS = ("sched", "gpu", "emit")


class StepRecord(NamedTuple):
    kind: str
    rows: int
    tokens: int
    sched: float
    gpu: float
    emit: float
    kernel: float | None  # None: the step was not bracketed by events


def _mean(values) -> float:
    values = list(values)
    return sum(values) / len(values) if values else 0.0


class StepStats:
    def __init__(self, every: int) -> None:
        if every < 1:
            raise ValueError("step stats interval must be >= 1")
        self.every = every
        self._window: list[StepRecord] = []
        self.lines: list[str] = []          # every line logged so far
        self.summaries: list[dict] = []     # and the numbers behind it

    def record(self, kind: str, rows: int, tokens: int, kernel: float | None = None, *, sched: float, gpu: float, emit: float) -> None:
        self._window.append(StepRecord(kind, rows, tokens, sched, gpu, emit, kernel))
        if len(self._window) >= self.every:
            self.flush()

    def summary(self) -> dict:
        """Per kind: steps, mean rows and tokens, mean milliseconds of each part, kernel/host where timed,
        and the kind's share of the window's wall time; under ``"wall"`` each part's share of it."""
        wall = sum(r.sched + r.gpu + r.emit for r in self._window) or 1.0
        out: dict = {"steps": len(self._window), "kinds": {}, "wall": {}}
        for kind in sorted({r.kind for r in self._window}):
            steps = [r for r in self._window if r.kind == kind]
            entry = {
                "n": len(steps),
                "rows": _mean(r.rows for r in steps),
                "tok": _mean(r.tokens for r in steps),
                **{part: _mean(getattr(r, part) for r in steps) for part in PARTS},
                "share": sum(r.sched + r.gpu + r.emit for r in steps) / wall,
            }
            timed = [r for r in steps if r.kernel is not None]
            if timed:
                entry["kernel"] = _mean(r.kernel for r in timed)
                entry["host"] = _mean(r.gpu - r.kernel for r in timed)
            out["kinds"][kind] = entry
        for part in PARTS:
            out["wall"][part] = sum(getattr(r, part) for r in self._window) / wall
        return out

    def format(self, summary: dict | None = None) -> str:
        summary = summary or self.summary()
        fields = [f"step stats steps={summary['steps']}"]
        for kind, e in summary["kinds"].items():
            parts = " ".join(f"{part}={e[part]:.2f}" for part in PARTS)
            if "kernel" in e:
                parts += f" (kernel={e['kernel']:.2f} host={e['host']:.2f})"
            fields.append(
                f"{kind} n={e['n']} rows={e['rows']:.1f} tok={e['tok']:.0f} ms/step[{parts}] share={100 * e['share']:.0f}%"
            )
        fields.append("wall " + " ".join(f"{part}={100 * summary['wall'][part]:.0f}%" for part in PARTS))
        return " | ".join(fields)

    def flush(self) -> str | None:
        """Log the window and start a new one; None when the window is empty."""
        if not self._window:
            return None
        summary = self.summary()
        line = self.format(summary)
        _log.info("%s", line)
        self.lines.append(line)
        self.summaries.append(summary)
        self._window.clear()
        return line
