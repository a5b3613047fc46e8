"""The Python entry point: load a model folder, generate, trace.

In the reference's manner (worker/src/inference/torch_engine.py:117-159, 295-338):
``Engine.load(model, device=..., dtype=...)`` builds everything once;
``generate(...)`` joins requests into one scheduler loop, so concurrent requests
are batched step by step; ``trace(prompt_ids, max_new_tokens, forced_ids)`` runs
one request synchronously and returns the arg-max and the float32 logits of every
step, free-running or teacher-forced.  The reference streams events through an
asyncio loop to a gRPC servicer; without a server the loop here is synchronous and
results come back as records (an ``on_token`` callback sees every token as it is
made).  Prompts are token ids: tokenisers are not part of the engine.

Request options follow the reference's ``GenerateRequest`` (worker/src/inference/
engine.py:46-52): ``max_tokens <= 0`` means 16 (engine.py:170-173); its hard cap of
256 is not kept, the cap is what the cache can hold.
"""

from __future__ import annotations

import logging
import time
from dataclasses import dataclass, field
from typing import Callable, Sequence

import torch

from ..cache.manager import CacheExhausted, CacheManager
from ..config.engine_config import EngineConfig
from ..config.registry import read_config
from ..kernels import make_kernels
from ..models.decoder import DecoderModel, model_tensor_specs, slot_needs
from ..weights.loader import open_weights
from .batch import BatchEntry
from .runner import ModelRunner
from .scheduler import Emission, Scheduler, Sequence as Seq
from .step_stats import StepStats

_log = logging.getLogger(__name__)

DEFAULT_MAX_TOKENS = 16
_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


@dataclass(frozen=True)
class GenerateRequest:
    request_id: str
    prompt_ids: Sequence[int]
    max_tokens: int = DEFAULT_MAX_TOKENS
    temperature: float = 0.0
    seed: int = 0


@dataclass
class GenerationResult:
    request_id: str
    token_ids: list[int] = field(default_factory=list)
    finish_reason: str | None = None  # "eos" | "length" | "aborted"
    prompt_tokens: int = 0
    completion_tokens: int = 0
    time_to_first_token_ms: float = 0.0
    total_latency_ms: float = 0.0
    preemptions: int = 0


@dataclass(frozen=True)
class Trace:
    """``token_ids[t]`` is the arg-max at step t; ``logits`` is ``[steps, vocab]`` float32 on the CPU."""

    token_ids: list[int]
    logits: torch.Tensor


def clamp_max_tokens(max_tokens: int) -> int:
    return DEFAULT_MAX_TOKENS if max_tokens <= 0 else int(max_tokens)


class Engine:
    def __init__(self, model: DecoderModel, cache: CacheManager, config: EngineConfig, model_config=None) -> None:
        self.model = model
        self.cache = cache
        self.config = config
        self.model_config = model_config
        self.runner = ModelRunner(
            model, cache, max(config.token_budget, config.max_seqs), config.max_seqs, config.decode_graphs
        )
        self.scheduler = Scheduler(cache, config.max_seqs, config.token_budget, config.prefill_chunk)
        self.stats = StepStats(config.step_stats) if config.step_stats else None
        self._serial = 0
        self.steps = 0
        self._in_flight = None  # (plan, handle) of a launched decode step whose tokens are still on the device
        self._planned = None    # a plan made by the pipelined path for the plain path to run

    # -- construction ---------------------------------------------------------
    @classmethod
    def load(cls, model: str, device: str = "cuda", dtype: str = "auto", **knobs) -> "Engine":
        """Build an engine for the model folder ``model`` (``config.json`` + safetensors).

        ``knobs``: ``num_blocks``, ``page_size``, ``max_seqs``, ``token_budget``,
        ``prefill_chunk``, ``max_model_len``, ``decode_graphs``, ``decode_ahead``, ``step_stats``; the
        reference's ``WORKER_*`` environment variables give the defaults.
        """
        if device == "cuda":
            device = "cuda:0"
        config = EngineConfig.from_env(dtype=dtype, device=device, **knobs)
        arch, model_config = read_config(model)
        kernels = make_kernels(_TORCH_DTYPE[config.dtype], config.device)
        return cls.assemble(arch, model_config, model, kernels, config)

    @classmethod
    def assemble(cls, arch, model_config, source, kernels, config: EngineConfig) -> "Engine":
        """Put an engine together from a registry entry, its typed configuration, a weight source
        (a model folder or a dict of tensors by checkpoint name) and a kernel set."""
        spec = arch.recipe(model_config)
        started = time.perf_counter()
        weights = open_weights(source, model_tensor_specs(spec), spec.tolerated, kernels.dtype, kernels.device)
        decoder = DecoderModel(spec, kernels, weights)
        cache = build_cache(spec, config, kernels.dtype, kernels.device)
        _log.info(
            "model ready architecture=%s dtype=%s pages=%s page_size=%s seats=%s load_s=%.1f",
            spec.architecture, config.dtype, config.num_blocks, config.page_size, config.max_seqs,
            time.perf_counter() - started,
        )
        return cls(decoder, cache, config, model_config)

    # -- generation -----------------------------------------------------------
    def generate(
        self,
        prompts,
        max_new_tokens: int = DEFAULT_MAX_TOKENS,
        temperature: float = 0.0,
        seed: int = 0,
        eos_id: int | None | str = "config",
        ignore_eos: bool = False,
        on_token: Callable[[str, int, bool], None] | None = None,
    ) -> list[GenerationResult]:
        """Generate for one prompt (a list of ids) or several (a list of lists), batched together.

        Every request gets ``seed + its index`` as sampling seed.  ``eos_id="config"``
        stops at the model configuration's ``eos_token_id``; ``ignore_eos`` never stops early.
        """
        single = bool(prompts) and isinstance(prompts[0], int)
        batch = [list(prompts)] if single else [list(p) for p in prompts]
        requests = []
        for index, prompt in enumerate(batch):
            self._serial += 1
            requests.append(
                GenerateRequest(f"gen-{self._serial}", prompt, max_new_tokens, temperature, seed + index)
            )
        return self.run(requests, eos_id=eos_id, ignore_eos=ignore_eos, on_token=on_token)

    def run(self, requests: Sequence[GenerateRequest], eos_id="config", ignore_eos=False, on_token=None) -> list[GenerationResult]:
        if eos_id == "config":
            eos_id = getattr(self.model_config, "eos_token_id", None)
        if ignore_eos:
            eos_id = None
        started = time.perf_counter()
        results: dict[str, GenerationResult] = {}
        seqs: dict[str, Seq] = {}
        for req in requests:
            result = GenerationResult(req.request_id, prompt_tokens=len(req.prompt_ids))
            results[req.request_id] = result
            if not req.prompt_ids:  # the reference answers an empty prompt with one finished, empty event
                result.finish_reason = "length"
                continue
            seq = Seq(
                request_id=req.request_id,
                prompt_ids=list(req.prompt_ids),
                max_new_tokens=clamp_max_tokens(req.max_tokens),
                temperature=req.temperature,
                eos_id=eos_id,
                seed=req.seed,
            )
            self.scheduler.submit(seq)
            seqs[req.request_id] = seq
        try:
            while self.has_work():
                for emission in self.step():
                    self._deliver(emission, results, started, on_token)
        except BaseException:
            for request_id in seqs:  # a failed step drops every request and returns their pages
                self.scheduler.abort(request_id)
            self._in_flight = self._planned = None
            self.scheduler.schedule()
            raise
        for request_id, seq in seqs.items():
            result = results[request_id]
            result.finish_reason = seq.finish_reason
            result.preemptions = seq.preemptions
        if self.stats is not None:
            self.stats.flush()
        return [results[req.request_id] for req in requests]

    def step(self) -> list[Emission]:
        """One scheduler step: plan, run, sample, complete.

        Decode steps run a step ahead when they can (``EngineConfig.decode_ahead``): the step is
        launched, the next one is planned and launched on the strength of it, and only then are its
        tokens waited for, so the host's share of a step and the launch of the graph overlap the
        GPU's work on the step before.  A call still returns the emissions of exactly one step.
        """
        if self._in_flight is not None or (self.config.decode_ahead and self.stats is None):
            ahead = self._step_ahead()
            if ahead is not None:
                return ahead
        t0 = time.perf_counter()
        plan, self._planned = self._planned or self.scheduler.schedule(), None
        if not plan.items:
            if self.scheduler.has_work():
                raise CacheExhausted("no request can run: waiting requests do not fit the free pages and nothing is running")
            return []
        t1 = time.perf_counter()
        kernel_ms = None
        if self.stats is not None:
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            tokens = self.runner.run_plan(plan)
            end.record()
            end.synchronize()
            kernel_ms = begin.elapsed_time(end)
        else:
            tokens = self.runner.run_plan(plan)
        t2 = time.perf_counter()
        emissions = self.scheduler.complete(plan, tokens)
        t3 = time.perf_counter()
        self.steps += 1
        if self.stats is not None:
            self.stats.record(
                plan.kind, len(plan.items), plan.num_tokens, kernel_ms,
                sched=(t1 - t0) * 1e3, gpu=(t2 - t1) * 1e3, emit=(t3 - t2) * 1e3,
            )
        return emissions

    def _step_ahead(self) -> list[Emission] | None:
        """The pipelined form of ``step`` for decode steps; None when this step has to run the plain way."""
        runner, scheduler = self.runner, self.scheduler
        if self._in_flight is None:
            plan = scheduler.schedule()
            if not plan.items:
                if scheduler.has_work():
                    raise CacheExhausted("no request can run: waiting requests do not fit the free pages and nothing is running")
                return []
            if not runner.can_launch_decode(plan.items):
                self._planned = plan  # a step with prompt portions: the plain path runs this very plan
                return None
            self._in_flight = (plan, runner.launch_decode(plan.items))
        plan, handle = self._in_flight
        self._in_flight = None
        if scheduler.can_look_ahead(plan):
            scheduler.assume(plan)
            following = scheduler.schedule()
            same_rows = len(following.items) == len(plan.items) and all(
                a.seq is b.seq and len(b.token_ids) == 1 for a, b in zip(plan.items, following.items)
            )
            if same_rows and runner.can_launch_decode(following.items):
                self._in_flight = (following, runner.launch_decode(following.items, ids_on_device=True))
            # otherwise the step after this one is planned again once these tokens are known
            emissions = scheduler.resolve(plan, runner.fetch_decode(handle))
        else:
            emissions = scheduler.complete(plan, runner.fetch_decode(handle))
        self.steps += 1
        return emissions

    def drain(self) -> None:
        """Waits for a launched step, if any, and drops its tokens (after requests were aborted)."""
        if self._in_flight is not None:
            _, handle = self._in_flight
            self._in_flight = None
            self.runner.fetch_decode(handle)
        self._planned = None

    def has_work(self) -> bool:
        """Requests waiting or running, or a launched step whose tokens have not been collected."""
        return self.scheduler.has_work() or self._in_flight is not None

    def _deliver(self, emission: Emission, results, started: float, on_token) -> None:
        result = results.get(emission.seq.request_id)
        if result is None:
            return
        now = time.perf_counter()
        result.token_ids.append(emission.token_id)
        result.completion_tokens = len(result.token_ids)
        if result.completion_tokens == 1:
            result.time_to_first_token_ms = (now - started) * 1e3
        if emission.finished:
            result.total_latency_ms = (now - started) * 1e3
        if on_token is not None:
            on_token(emission.seq.request_id, emission.token_id, emission.finished)

    # -- trace ----------------------------------------------------------------
    def trace(self, prompt_ids: Sequence[int], max_new_tokens: int, forced_ids: Sequence[int] | None = None) -> Trace:
        """One request through the step function, synchronously (torch_engine.py:295-338).

        Free-running (``forced_ids=None``) feeds back the arg-max and stops after the
        configuration's EOS; teacher-forced feeds ``forced_ids[step]`` whatever was picked.
        """
        if not prompt_ids:
            raise ValueError("prompt_ids must be non-empty")
        if max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
        if forced_ids is not None and len(forced_ids) < max_new_tokens:
            raise ValueError("forced_ids shorter than max_new_tokens")
        eos_id = getattr(self.model_config, "eos_token_id", None)
        seat = self.cache.open_seat()
        picks: list[int] = []
        rows: list[torch.Tensor] = []
        try:
            if not self.cache.grow(seat, len(prompt_ids) + max_new_tokens):
                raise CacheExhausted("out of KV blocks for the trace")
            current = list(prompt_ids)
            cached = 0
            for step in range(max_new_tokens):
                logits = self.runner.step([BatchEntry(seat, current, cached, (len(current) - 1,))])
                row = logits[0].float().cpu()
                self.runner.finish_step()
                cached += len(current)
                pick = int(torch.argmax(row))
                picks.append(pick)
                rows.append(row)
                if forced_ids is None:
                    if eos_id is not None and pick == eos_id:
                        break
                    current = [pick]
                else:
                    current = [int(forced_ids[step])]
        finally:
            self.cache.close_seat(seat)
        return Trace(token_ids=picks, logits=torch.stack(rows))


def build_cache(spec, config: EngineConfig, torch_dtype, device) -> CacheManager:
    cache_needs, state_needs = slot_needs(spec)
    longest = config.max_model_len or config.num_blocks * config.page_size
    if spec.max_positions:
        longest = min(longest, spec.max_positions)
    return CacheManager(
        cache_needs,
        state_needs,
        num_pages=config.num_blocks,
        page_size=config.page_size,
        max_seats=config.max_seqs,
        max_tokens_per_request=longest,
        dtype=torch_dtype,
        device=device,
    )
