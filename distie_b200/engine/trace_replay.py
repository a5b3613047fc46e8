"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and owns no forward pass, cache or loader: it drives the same
model, step function (:class:`~distie_b200.engine.runner.ModelRunner`), cache
manager and kernels that generation uses.  The reference's analogue is the
teacher-forced ``trace`` of its engine (worker/src/inference/torch_engine.py:
295-338).

Input, one JSON object per line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose
logits are wanted.  All entries of a step are one batch.  ``end``: requests that
are finished after the step; their pages and seat are given back.  For a step in
which something is wanted ``<out>/<step>.f32`` receives the logits
``[wanted, vocab]`` as little-endian float32, in the order of the entries and of
``want``.  After every step ``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import json
import os
import sys
from typing import IO, Iterable

import numpy as np
import torch

from ..cache.manager import CacheExhausted, pages_needed
from ..config.engine_config import EngineConfig
from .batch import BatchEntry
from .engine import Engine

LIVE_REQUESTS = 8  # the protocol keeps up to four live; seats for twice that


class TraceSession:
    def __init__(self, engine: Engine) -> None:
        self.engine = engine
        self.live: dict[str, list[int]] = {}  # id -> [seat, cached tokens]

    @classmethod
    def open(cls, model: str, dtype: str, max_tokens: int, page_size: int = 16, device: str = "cuda",
             decode_graphs: bool = True) -> "TraceSession":
        """``max_tokens``: the most tokens live requests hold at any time, each request's count
        rounded up to a multiple of 64; the pool is made for exactly this many, so pages are reused.
        With ``decode_graphs`` a step in which every request brings one token replays the captured
        decode step of its batch bucket, as generation does."""
        rounded = -(-int(max_tokens) // 64) * 64
        engine = Engine.load(
            model,
            device=device,
            dtype=dtype,
            num_blocks=pages_needed(rounded, page_size),
            page_size=page_size,
            max_seqs=LIVE_REQUESTS,
            token_budget=rounded,
            max_model_len=rounded,
            decode_graphs=decode_graphs,
        )
        return cls(engine)

    def run_step(self, entries: list[dict], end: Iterable[str] = ()) -> np.ndarray | None:
        cache, runner = self.engine.cache, self.engine.runner
        batch: list[BatchEntry] = []
        seen: set[str] = set()
        for entry in entries:
            rid = str(entry["id"])
            tokens = [int(t) for t in entry["tokens"]]
            if rid in seen:
                raise ValueError(f"request {rid!r} appears twice in one step")
            seen.add(rid)
            if not tokens:
                raise ValueError(f"request {rid!r} brings no tokens")
            if rid not in self.live:
                self.live[rid] = [cache.open_seat(), 0]
            seat, cached = self.live[rid]
            if not cache.grow(seat, cached + len(tokens)):
                raise CacheExhausted(
                    f"out of pages: request {rid!r} needs {cached + len(tokens)} tokens, "
                    f"{cache.free_pages()} pages of {cache.page_size} tokens are free"
                )
            batch.append(BatchEntry(seat, tokens, cached, tuple(int(w) for w in entry.get("want", ()))))
        result = None
        if batch:
            logits = runner.step(batch)
            if logits is not None:
                result = logits.float().cpu().numpy()
            runner.finish_step()
            for entry, item in zip(entries, batch):
                state = self.live[str(entry["id"])]
                state[1] += len(item.tokens)
                cache.trim(state[0], state[1])
        for rid in end:
            state = self.live.pop(str(rid), None)
            if state is not None:
                cache.close_seat(state[0])
        return result


def replay(session: TraceSession, lines: IO[str], out_dir: str, report: IO[str] = sys.stdout) -> int:
    os.makedirs(out_dir, exist_ok=True)
    steps = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        logits = session.run_step(record.get("entries", []), record.get("end", []))
        if logits is not None and logits.size:
            logits.astype("<f4", copy=False).tofile(os.path.join(out_dir, f"{step}.f32"))
        report.write(f"done {step}\n")
        report.flush()
        steps += 1
    return steps


def main(argv=None) -> int:
    import argparse

    parser = argparse.ArgumentParser(
        prog="trace_run",
        description="Feed token ids from standard input through the model step by step and write logits.",
    )
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True, help="most tokens live requests hold at any time")
    parser.add_argument("--page-size", type=int, default=16, help="tokens per cache page (default 16)")
    parser.add_argument("--no-decode-graphs", action="store_true",
                        help="run steps of single tokens eagerly instead of replaying captured decode steps")
    args = parser.parse_args(argv)
    print(f"[distie_b200] loading {args.model} as {args.dtype}", file=sys.stderr, flush=True)
    session = TraceSession.open(args.model, args.dtype, args.max_tokens, args.page_size,
                                decode_graphs=not args.no_decode_graphs)
    print("[distie_b200] ready", file=sys.stderr, flush=True)
    replay(session, sys.stdin, args.out)
    return 0
