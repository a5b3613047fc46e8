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

from ..cache.manager import CacheExhausted, CacheManager, pages_that_fit
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

        ``knobs``: ``num_blocks`` or ``gpu_mem_fraction``, ``page_size``, ``max_seqs``, ``token_budget``,
        ``prefill_chunk``, ``max_model_len``, ``decode_graphs``, ``decode_ahead``, ``step_stats``,
        ``float32_weights``; the reference's ``WORKER_*`` environment variables give the defaults.
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
        weights = open_weights(source, model_tensor_specs(spec), spec.tolerated, kernels.dtype, kernels.device,
                               config.float32_weights)
        decoder = DecoderModel(spec, kernels, weights)
        if config.gpu_mem_fraction is not None:
            config = config.sized(pages_from_free_memory(spec, config, kernels.dtype, kernels.device))
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
            if req.request_id in results:
                raise ValueError(f"duplicate request_id {req.request_id}")
            result = GenerationResult(req.request_id, prompt_tokens=len(req.prompt_ids))
            results[req.request_id] = result
            if not req.prompt_ids:  # the reference answers an empty prompt with one finished, empty event
                result.finish_reason = "length"
                continue
            seqs[req.request_id] = Seq(
                request_id=req.request_id,
                prompt_ids=list(req.prompt_ids),
                max_new_tokens=clamp_max_tokens(req.max_tokens),
                temperature=req.temperature,
                eos_id=eos_id,
                seed=req.seed,
            )
        for seq in seqs.values():  # every request is checked before any is taken: a refusal leaves nothing behind
            self.scheduler.validate(seq)
        for seq in seqs.values():
            self.scheduler.submit(seq)
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
        if self._in_flight is not None or self.config.decode_ahead:
            ahead = self._step_ahead()
            if ahead is not None:
                return ahead
        clock = time.perf_counter
        t0 = clock()
        plan, self._planned = self._planned or self.scheduler.schedule(), None
        if not plan.items:
            return self._nothing_to_run()
        t1 = clock()
        events = self._bracket()
        tokens = self.runner.run_plan(plan)
        kernel_ms = self._elapsed(events)
        t2 = clock()
        emissions = self.scheduler.complete(plan, tokens)
        self.steps += 1
        if self.stats is not None:
            self.stats.record(plan.kind, len(plan.items), plan.num_tokens, kernel_ms,
                              sched=(t1 - t0) * 1e3, gpu=(t2 - t1) * 1e3, emit=(clock() - t2) * 1e3)
        return emissions

    def _nothing_to_run(self) -> list[Emission]:
        if self.scheduler.has_work():
            raise CacheExhausted("no request can run: waiting requests do not fit the free pages and nothing is running")
        return []

    def _bracket(self):
        """With step statistics on: a CUDA event recorded now, to be paired with one after the launches."""
        if self.stats is None or self.runner.device.type != "cuda":
            return None
        begin = torch.cuda.Event(enable_timing=True)
        begin.record()
        return [begin, None]

    @staticmethod
    def _elapsed(events) -> float | None:
        if events is None:
            return None
        if events[1] is None:
            events[1] = torch.cuda.Event(enable_timing=True)
            events[1].record()
        events[1].synchronize()
        return events[0].elapsed_time(events[1])

    def _launch(self, plan, ids_on_device: bool = False):
        """Launch a decode step; ``(plan, handle, events, host milliseconds)`` or None when no graph could be made."""
        started = time.perf_counter()
        events = self._bracket()
        handle = self.runner.launch_decode(plan.items, ids_on_device=ids_on_device)
        if handle is None:
            return None
        if events is not None:
            events[1] = torch.cuda.Event(enable_timing=True)
            events[1].record()
        return plan, handle, events, (time.perf_counter() - started) * 1e3

    def _step_ahead(self) -> list[Emission] | None:
        """The pipelined form of ``step`` for decode steps; None when this step has to run the plain way."""
        runner, scheduler, clock = self.runner, self.scheduler, time.perf_counter
        sched_ms = 0.0
        if self._in_flight is None:
            t0 = clock()
            plan = scheduler.schedule()
            sched_ms += (clock() - t0) * 1e3
            if not plan.items:
                return self._nothing_to_run()
            launched = self._launch(plan) if runner.can_launch_decode(plan.items) else None
            if launched is None:
                self._planned = plan  # prompt portions, or no graph could be made: the plain path runs this very plan
                return None
            self._in_flight = launched
        plan, handle, events, gpu_ms = self._in_flight
        self._in_flight = None
        look_ahead = scheduler.can_look_ahead(plan)
        if look_ahead:
            t0 = clock()
            scheduler.assume(plan)
            following = scheduler.schedule()
            sched_ms += (clock() - t0) * 1e3
            same_rows = len(following.items) == len(plan.items) and all(
                a.seq is b.seq and len(b.token_ids) == 1 for a, b in zip(plan.items, following.items)
            )
            if same_rows and runner.can_launch_decode(following.items):
                self._in_flight = self._launch(following, ids_on_device=True)
            # otherwise the step after this one is planned again once these tokens are known
        t1 = clock()
        tokens = runner.fetch_decode(handle)
        kernel_ms = self._elapsed(events)
        t2 = clock()
        emissions = scheduler.resolve(plan, tokens) if look_ahead else scheduler.complete(plan, tokens)
        self.steps += 1
        if self.stats is not None:
            # gpu: launching this step plus waiting for its tokens; the launch of the next step, done in between,
            # is booked on the next step.
            self.stats.record(plan.kind, len(plan.items), plan.num_tokens, kernel_ms,
                              sched=sched_ms, gpu=gpu_ms + (t2 - t1) * 1e3, emit=(clock() - t2) * 1e3)
        return emissions

    def drain(self) -> None:
        """Waits for a launched step, if any, and drops its tokens (after requests were aborted)."""
        if self._in_flight is not None:
            handle = self._in_flight[1]
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


def pages_from_free_memory(spec, config: EngineConfig, torch_dtype, device) -> int:
    """Pages that ``config.gpu_mem_fraction`` of the device memory free right now (the weights are loaded)
    holds, keys and values of every cache slot counted.  What is left over serves activations, the captured
    decode steps and the library's workspaces."""
    cache_needs, _ = slot_needs(spec)
    device = torch.device(device)
    if device.type != "cuda":
        raise ValueError("gpu_mem_fraction sizes the cache from a CUDA device's free memory; give num_blocks on other devices")
    torch.cuda.empty_cache()
    free, _total = torch.cuda.mem_get_info(device)
    element = torch.empty((), dtype=torch_dtype).element_size()
    pages = pages_that_fit(cache_needs, config.page_size, element, int(free * float(config.gpu_mem_fraction)))
    if pages < 1:
        raise CacheExhausted(f"{config.gpu_mem_fraction} of the {free >> 20} MiB that are free hold not one page of cache")
    _log.info("cache sized from free memory free_mib=%s fraction=%s pages=%s", free >> 20, config.gpu_mem_fraction, pages)
    return pages


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
