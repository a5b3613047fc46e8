"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--shape 1.5b|7b|14b] [--dtype bf16|fp32] [--only decode|prefill|serving]

A "step" is one decode step.  The default run has the layer sizes of the third
configuration in ``BASELINE.json`` (the Qwen2.5-1.5B shape) with random
``N(0, 0.02)`` weights in bfloat16, a batch of 8 requests, each with a 1,024-token
random prompt in the cache, and a 4,096-token context limit.

* ``value``: decoded tokens per second at batch 8.  K steps run back to back on the
  device (each step's sampled tokens feed the next step there), bracketed by CUDA
  events and a synchronise on both sides, after W untimed steps.
* ``e2e``: the same through the Python entry point (``Engine.step``): every step
  plans on the host, copies its inputs from pinned memory, replays the step and
  reads the sampled token ids back.
* ``points``: ``value`` at batch 1 and 64.
* ``prefill``: one 2,048-token prompt through the step function; ``frac`` is the
  step's FLOPs / time / the measured bf16 peak.
* ``roofline``: bytes a decode step has to read (every weight once, the cache of the
  live requests) / its time, against the measured copy bandwidth.

Every step reads about 3 GB of weights, far more than the 126 MB L2, so nothing
stays cached between timed iterations.  This engine runs on one GPU: for
``--gpus N`` with N > 1 a line says so and the exit code is 2.

Other runs, each printing one line of the same form (none of them is the default):
``--shape 14b`` is ``BASELINE.json`` ``configs[4]`` (decode at batch 1/8/64 at 2,048-token
contexts, prefill of 2,048 tokens); ``--shape 7b`` is ``configs[3]``, the mixed
continuous-batching run through ``Engine.generate`` (64 requests, prompts of 64 to 2,048
tokens, 256 outputs each, 2,048-token step budget, 32 seats) with time to first token,
time per output token, preemptions and the step-time split; ``--dtype fp32`` times the
true 32-bit engine.  Their caches are sized from free device memory.
"""

from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The Qwen2.5-1.5B shape, used when BASELINE.json cannot be read.
FALLBACK_SHAPE = {
    "num_hidden_layers": 28, "hidden_size": 1536, "num_attention_heads": 12, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 8960, "vocab_size": 151936, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
}
PROMPT_LEN, GEN_LEN, CONTEXT, PAGE, PREFILL_TOKENS = 1024, 256, 4096, 16, 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


FALLBACK_SHAPES = {
    "1.5b": FALLBACK_SHAPE,
    "7b": {
        "num_hidden_layers": 28, "hidden_size": 3584, "num_attention_heads": 28, "num_key_value_heads": 4,
        "head_dim": 128, "intermediate_size": 18944, "vocab_size": 152064, "rope_theta": 1000000.0,
        "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    },
    "14b": {
        "num_hidden_layers": 48, "hidden_size": 5120, "num_attention_heads": 40, "num_key_value_heads": 8,
        "head_dim": 128, "intermediate_size": 13824, "vocab_size": 152064, "rope_theta": 1000000.0,
        "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
    },
}
SHAPE_CONFIG = {"1.5b": 2, "7b": 3, "14b": 4}  # index into BASELINE.json "configs"
SHAPE_NAME = {"1.5b": "Qwen2.5-1.5B", "7b": "Qwen2.5-7B", "14b": "Qwen2.5-14B"}


def shape_from_baseline(which: str = "1.5b") -> dict:
    """Layer sizes parsed from the prose of the shape's entry in ``BASELINE.json`` ``configs``."""
    try:
        with open(os.path.join(ROOT, "BASELINE.json"), "r", encoding="utf-8") as handle:
            text = json.load(handle)["configs"][SHAPE_CONFIG[which]]
        number = lambda pattern: re.search(pattern, text).group(1).replace(",", "")  # noqa: E731
        return {
            "num_hidden_layers": int(number(r"(\d+) layers")),
            "hidden_size": int(number(r"hidden (\d[\d,]*)")),
            "num_attention_heads": int(number(r"(\d+) q heads")),
            "num_key_value_heads": int(number(r"(\d+) kv heads")),
            "head_dim": int(number(r"head_dim (\d+)")),
            "intermediate_size": int(number(r"intermediate (\d[\d,]*)")),
            "vocab_size": int(number(r"vocab (\d[\d,]*)")),
            "rope_theta": float(number(r"rope_theta (\d+)")),
            "rms_norm_eps": float(number(r"rms_norm_eps ([\d.e-]+)")),
            "tie_word_embeddings": "tied embeddings" in text,
        }
    except Exception:
        return dict(FALLBACK_SHAPES[which])


def measured_peaks() -> tuple[dict, str]:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json"), "r", encoding="utf-8") as handle:
            raw = json.load(handle)
        flat = {}

        def walk(node):
            if isinstance(node, dict):
                for key, value in node.items():
                    if isinstance(value, (int, float)) and key not in flat:
                        flat[key] = float(value)
                    else:
                        walk(value)

        walk(raw)
        if "hbm_gbs" in flat and "bf16_tflops" in flat:
            return flat, "measured"
    except Exception:
        pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """``nvidia-smi`` clocks and throttle reasons, sampled every 200 ms while the timed regions run."""

    FIELDS = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __enter__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=self.file, stderr=subprocess.DEVNULL,
            )
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()

    def summary(self) -> dict:
        self.file.seek(0)
        clocks, peak, reasons = [], 0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.file:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6 or not parts[0].isdigit():
                continue
            clocks.append(int(parts[0]))
            peak = max(peak, int(parts[1])) if parts[1].isdigit() else peak
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.file.name)
        busy = [c for c in clocks if c > 0]
        return {"sm_mhz": int(statistics.median(busy)) if busy else None, "sm_max_mhz": peak or None, "reasons": sorted(reasons), "samples": len(clocks)}


def build_engine(shape: dict, layers: int, max_seqs: int, num_blocks: int | None, max_model_len: int = CONTEXT,
                 dtype: str = "bfloat16", gpu_mem_fraction: float | None = None, step_stats: int = 0,
                 token_budget: int = 2048):
    """The engine with random weights made on the device; the cache from a page count or from free memory."""
    import torch

    from distie_b200.config import EngineConfig, get_architecture
    from distie_b200.engine.engine import Engine
    from distie_b200.kernels import make_kernels
    from distie_b200.models import model_tensor_specs
    from distie_b200.weights import RandomSource

    torch_dtype = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    raw = {"architectures": ["Qwen2ForCausalLM"], **shape, "num_hidden_layers": layers, "max_position_embeddings": 32768}
    arch = get_architecture("Qwen2ForCausalLM")
    typed = arch.config_cls.from_dict(raw)
    kernels = make_kernels(torch_dtype, "cuda:0")
    source = RandomSource(model_tensor_specs(arch.recipe(typed)), seed=0, std=0.02, dtype=torch_dtype, device="cuda:0")
    config = EngineConfig(
        num_blocks=num_blocks or 1, gpu_mem_fraction=None if num_blocks else gpu_mem_fraction, page_size=PAGE,
        max_seqs=max_seqs, token_budget=token_budget, max_model_len=max_model_len, dtype=dtype, decode_graphs=True,
        device="cuda:0", step_stats=step_stats,
    )
    return Engine.assemble(arch, typed, source, kernels, config)


def random_prompt(vocab: int, length: int, seed: int) -> list[int]:
    import torch

    return torch.randint(0, vocab, (length,), generator=torch.Generator().manual_seed(seed)).tolist()


def fill_requests(engine, batch: int, prompt_len: int, total_new: int, tag: str):
    """`batch` requests through the engine's scheduler until each has its prompt in the cache and one token
    to decode; their pages are then grown for `total_new` more tokens.  Returns the decode plan."""
    from distie_b200.engine.scheduler import Sequence

    vocab = engine.model.vocab_size
    # Requests admitted first decode while the later ones are still being prefilled: room for those tokens too.
    for b in range(batch):
        engine.scheduler.submit(Sequence(f"{tag}-{b}", random_prompt(vocab, prompt_len, 100 + b), total_new + 8 + 2 * batch))
    while True:
        plan = engine.scheduler.schedule()
        if plan.kind == "decode" and len(plan.items) == batch and engine.scheduler.num_waiting == 0:
            break
        engine.scheduler.complete(plan, engine.runner.run_plan(plan))
    for item in plan.items:
        assert engine.cache.grow(item.seq.seat, item.past_len + 1 + total_new), "the bench pool is too small"
    return plan


def release(engine, batch: int, tag: str) -> None:
    for b in range(batch):
        engine.scheduler.abort(f"{tag}-{b}")
    engine.drain()
    engine.scheduler.schedule()
    assert engine.cache.free_pages() == engine.cache.total_pages()


def time_decode(engine, burst, batch: int, prompt_len: int, steps: int, warmup: int) -> dict:
    """K decode steps back to back on the device, after W warm-up steps; CUDA events around them."""
    import torch

    tag = f"bench{batch}"
    plan = fill_requests(engine, batch, prompt_len, warmup + steps + 1, tag)
    burst.run(plan.items, max(warmup, 1))
    # The burst advanced the positions on the device; the timed burst starts where it stopped.
    advanced = [type(item)(item.seq, item.token_ids, item.past_len + max(warmup, 1), True) for item in plan.items]
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()  # a profiler started with "profile from start off" sees the timed steps only
    begin.record()
    tokens = burst.run(advanced, steps)
    end.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    ms = begin.elapsed_time(end)
    engine.runner.finish_step()
    assert tokens.shape == (steps, batch)
    mean_context = sum(item.past_len for item in plan.items) / batch + 1 + max(warmup, 1) + steps / 2
    release(engine, batch, tag)
    return {
        "ms_per_step": ms / steps,
        "tokens_per_s": batch * steps / (ms / 1e3),
        "mean_context": mean_context,
        "launches": burst.kernels_per_step(batch) * steps,
    }


def time_e2e(engine, batch: int, prompt_len: int, steps: int, warmup: int) -> dict:
    """The same decode steps through ``Engine.step``: host planning, pinned staging, replay, ids back."""
    import torch

    from distie_b200.engine.scheduler import Sequence

    vocab = engine.model.vocab_size
    for b in range(batch):
        engine.scheduler.submit(Sequence(f"e2e-{b}", random_prompt(vocab, prompt_len, 500 + b), warmup + steps + 8))
    while any(s.num_pending > 1 for s in engine.scheduler.running()) or engine.scheduler.num_waiting:
        engine.step()
    for _ in range(max(warmup, 1)):
        engine.step()
    torch.cuda.synchronize()
    produced = 0
    started = time.perf_counter()
    for _ in range(steps):
        produced += len(engine.step())
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - started
    release(engine, batch, "e2e")
    size = engine.runner.bucket_for(batch)
    return {
        "value": produced / elapsed,
        "unit": "tokens/s",
        "h2d_bytes_per_step": 5 * size * 4 + 2 * size * 4,
        "d2h_bytes_per_step": batch * 4 + 4,
        "ms_per_step": elapsed / steps * 1e3,
    }


def time_prefill(engine, repeats: int = 5, past: int = 0) -> dict:
    """One 2,048-token portion through the step function, behind `past` tokens that are already in the cache."""
    import torch

    from distie_b200.engine.batch import BatchEntry

    vocab = engine.model.vocab_size
    prompt = random_prompt(vocab, past + PREFILL_TOKENS, 7)
    times = []
    for index in range(repeats + 2):
        seat = engine.cache.open_seat()
        assert engine.cache.grow(seat, past + PREFILL_TOKENS)
        for start in range(0, past, PREFILL_TOKENS):  # the earlier portions, untimed
            engine.runner.step([BatchEntry(seat, prompt[start : min(past, start + PREFILL_TOKENS)], start, ())])
            engine.runner.finish_step()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if index == repeats + 1:
            torch.cuda.profiler.start()  # a profiler started with "profile from start off" sees the last repeat only
        begin.record()
        engine.runner.step([BatchEntry(seat, prompt[past:], past, (PREFILL_TOKENS - 1,))])
        end.record()
        torch.cuda.synchronize()
        if index == repeats + 1:
            torch.cuda.profiler.stop()
        times.append(begin.elapsed_time(end))
        engine.runner.finish_step()
        engine.cache.close_seat(seat)
    ms = statistics.median(times[2:])
    return {"ms": ms, "tokens": PREFILL_TOKENS, "past": past, "value": PREFILL_TOKENS / (ms / 1e3)}


def percentile(values, q: float) -> float:
    ordered = sorted(values)
    if not ordered:
        return 0.0
    at = min(len(ordered) - 1, max(0, int(round(q * (len(ordered) - 1)))))
    return ordered[at]


def serving_run(engine, requests: int = 64, longest: int = 2048, shortest: int = 64, new_tokens: int = 256) -> dict:
    """Mixed continuous batching through ``Engine.generate``: every request handed over at once, prompts of
    seeded uniform length, `new_tokens` outputs each; admission, portions, decoding and preemption as the
    scheduler decides.  Times are wall clock from the hand-over, as the reference's load test measures them
    (benchmarks/load/stats.py:29-34: the time per output token leaves the first token out)."""
    import random

    import torch

    rng = random.Random(0)
    vocab = engine.model.vocab_size
    lengths = [rng.randint(shortest, longest) for _ in range(requests)]
    prompts = [random_prompt(vocab, n, 7000 + i) for i, n in enumerate(lengths)]
    engine.generate(prompts[:2], max_new_tokens=4, ignore_eos=True)  # kernels loaded, first graphs captured
    torch.cuda.synchronize()
    steps_before = engine.steps
    started = time.perf_counter()
    results = engine.generate(prompts, max_new_tokens=new_tokens, ignore_eos=True)
    torch.cuda.synchronize()
    wall = time.perf_counter() - started
    produced = sum(r.completion_tokens for r in results)
    ttft = [r.time_to_first_token_ms for r in results]
    tpot = [(r.total_latency_ms - r.time_to_first_token_ms) / max(1, r.completion_tokens - 1) for r in results]
    out = {
        "requests": requests, "seats": engine.config.max_seqs, "token_budget": engine.config.token_budget,
        "outputs_each": new_tokens, "prompt_tokens": sum(lengths), "output_tokens": produced, "wall_s": round(wall, 3),
        "tokens_per_s": produced / wall, "total_tokens_per_s": (produced + sum(lengths)) / wall,
        "steps": engine.steps - steps_before, "preemptions": sum(r.preemptions for r in results),
        "ttft_ms": {q: round(percentile(ttft, v), 2) for q, v in (("p50", 0.5), ("p90", 0.9), ("p99", 0.99))},
        "tpot_ms": {q: round(percentile(tpot, v), 3) for q, v in (("p50", 0.5), ("p90", 0.9), ("p99", 0.99))},
    }
    if engine.stats is not None:
        engine.stats.flush()
        out["step_stats"] = engine.stats.lines[-3:]
    return out


def prefill_flops(shape: dict, layers: int, tokens: int) -> float:
    h, inter = shape["hidden_size"], shape["intermediate_size"]
    nq, nkv, d = shape["num_attention_heads"], shape["num_key_value_heads"], shape["head_dim"]
    per_layer = 2 * tokens * h * (nq + 2 * nkv) * d + 2 * tokens * nq * d * h + 2 * tokens * h * 2 * inter + 2 * tokens * inter * h
    attention = 4 * (tokens * (tokens + 1) / 2) * nq * d
    head = 2 * 1 * h * shape["vocab_size"]
    return layers * (per_layer + attention) + head


def reference_arm(args) -> int:
    """The unmodified reference on the same workload; none of this repository's engine is imported."""
    from baseline import reference_arm as arm

    shape = shape_from_baseline()
    layers = args.layers or shape["num_hidden_layers"]
    peaks, peaks_kind = measured_peaks()
    constants = {"prompt_len": PROMPT_LEN, "context": CONTEXT, "prefill_tokens": PREFILL_TOKENS}
    try:
        line = arm.run(args, shape, layers, peaks, peaks_kind, constants, ClockSampler, prefill_flops)
    except arm.Unavailable as exc:
        line = {"impl": "reference", "unavailable": str(exc)}
    except Exception as exc:  # noqa: BLE001  (the contract: a reference that cannot run prints why and exits 0)
        line = {"impl": "reference", "unavailable": f"the reference raised {type(exc).__name__}: {exc}"[:400]}
    print(json.dumps(line))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=GEN_LEN)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--shape", default="1.5b", choices=list(SHAPE_CONFIG),
                        help="layer sizes: the default run is 1.5b; 14b decodes at 2,048-token contexts; 7b is the mixed serving run")
    parser.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"], help="fp32: the true 32-bit engine")
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--only", default=None, choices=["decode", "prefill", "serving"],
                        help="run one part and print a short line (for profiling captures; not a bench value)")
    parser.add_argument("--pages", type=int, default=None,
                        help="cache pages instead of sizing from free memory (small captures under a profiler)")
    parser.add_argument("--past", type=int, default=0,
                        help="with --only prefill: tokens already in the cache ahead of the timed 2,048-token portion")
    parser.add_argument("--ref-attn", default=None, choices=["auto", "flash", "torch"],
                        help="with --impl reference: its attention backend (default: DISTIE_ATTN, else auto)")
    parser.add_argument("--ref-device", default=None, help=argparse.SUPPRESS)  # "cpu": a dry run of the reference arm
    args = parser.parse_args()
    if args.gpus != 1:
        print(json.dumps({"unsupported": f"--gpus {args.gpus}: this engine runs on one GPU; run with --gpus 1", "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return reference_arm(args)

    from distie_b200.engine.measure import DecodeBurst

    shape = shape_from_baseline(args.shape)
    layers_full = shape["num_hidden_layers"]
    layers = args.layers or layers_full
    peaks, peaks_kind = measured_peaks()
    dtype = "bfloat16" if args.dtype == "bf16" else "float32"
    name = SHAPE_NAME[args.shape]
    # The default run decodes behind 1,024-token prompts; the 14B configuration asks for 2,048-token contexts,
    # which its requests reach at the end of the timed steps.
    context = CONTEXT if args.shape == "1.5b" else 2048 + 256  # room for the tokens requests decode while others are still prefilled
    prompt_len = PROMPT_LEN if args.shape == "1.5b" else 2048 - (max(args.warmup, 1) + args.steps + 1)
    if prompt_len < 64:
        print(json.dumps({"unsupported": "--steps too large for a 2,048-token context"}))
        return 2
    config = {
        "model": f"{name} shape (Qwen2ForCausalLM)", "layers": layers, "layers_full": layers_full,
        "hidden": shape["hidden_size"], "q_heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
        "head_dim": shape["head_dim"], "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
        "tied": shape["tie_word_embeddings"], "global_batch": args.batch, "prompt_len": prompt_len,
        "seq_len": context, "page_size": PAGE, "parallelism": "none (1 GPU)", "decode": "CUDA graph per batch bucket",
        "l2": "inputs larger than L2 (the weights alone, read once per step)", "peaks": peaks_kind,
    }
    common = {
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": args.dtype,
        "data": "synthetic: random N(0,0.02) weights, uniform random token ids", "impl": "ours",
    }

    if args.only == "serving" or (args.shape == "7b" and args.only is None):
        # BASELINE.json configs[3]: mixed continuous batching through the Python entry point.
        engine = build_engine(shape, layers, 32, None, 2048 + 256 + 64, dtype, gpu_mem_fraction=0.85, step_stats=100000)
        with ClockSampler() as sampler:
            run = serving_run(engine)
        config.update({"global_batch": 32, "prompt_len": "uniform 64..2048", "seq_len": 2048 + 256,
                       "cache_pages": engine.config.num_blocks})
        line = {
            "metric": f"output tok/s, 64 requests through Engine.generate ({name} shape, {args.dtype}, mixed continuous batching)",
            "value": round(run["tokens_per_s"], 1), **common, "steps": run["steps"], "warmup": 1,
            "ms_per_step": round(run["wall_s"] * 1e3 / max(1, run["steps"]), 3), "config": config,
            "serving": {k: (round(v, 1) if isinstance(v, float) else v) for k, v in run.items()},
            "clocks": sampler.summary(),
        }
        print(json.dumps(line))
        return 0

    new_tokens = args.warmup + args.steps + 8
    if args.only == "prefill" and args.past > 0:
        pages = 2 * -(-(args.past + PREFILL_TOKENS) // PAGE)
        engine = build_engine(shape, layers, 8, pages, max(CONTEXT, args.past + PREFILL_TOKENS), dtype)
    elif args.shape == "1.5b" and args.pages is None:
        pages = 64 * -(-(prompt_len + new_tokens + 2 * 64 + 1) // PAGE) + 2 * (PREFILL_TOKENS // PAGE)
        engine = build_engine(shape, layers, 64, pages, context, dtype)
    else:
        engine = build_engine(shape, layers, 64, args.pages, context, dtype, gpu_mem_fraction=0.85)
        config["cache_pages"] = engine.config.num_blocks
    burst = DecodeBurst(engine.runner)
    weight_bytes = engine.model.weight_bytes()
    kv_bytes_per_token = engine.cache.bytes_per_token()

    if args.only == "decode":
        print(json.dumps({"only": "decode", "batch": args.batch, "layers": layers, "dtype": args.dtype,
                          **time_decode(engine, burst, args.batch, prompt_len, args.steps, args.warmup)}))
        return 0
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "layers": layers, "dtype": args.dtype,
                          **time_prefill(engine, repeats=max(1, args.steps), past=args.past)}))
        return 0

    with ClockSampler() as sampler:
        head = time_decode(engine, burst, args.batch, prompt_len, args.steps, args.warmup)
        e2e = time_e2e(engine, args.batch, prompt_len, args.steps, args.warmup)
        points, fractions = {}, {}
        for batch in (1, 64):
            point = time_decode(engine, burst, batch, prompt_len, args.steps, args.warmup)
            points[f"decode_b{batch}"] = round(point["tokens_per_s"], 1)
            moved = weight_bytes + batch * point["mean_context"] * kv_bytes_per_token
            fractions[f"decode_b{batch}"] = round(moved / (point["ms_per_step"] / 1e3) / 1e9 / peaks["hbm_gbs"], 4)
        prefill = time_prefill(engine)
        time.sleep(0.3)
    clocks = sampler.summary()

    step_bytes = weight_bytes + args.batch * head["mean_context"] * kv_bytes_per_token
    achieved = step_bytes / (head["ms_per_step"] / 1e3) / 1e9
    flops = prefill_flops(shape, layers, PREFILL_TOKENS)
    prefill.pop("past", None)
    peak_flops = peaks["bf16_tflops"] * 1e12 if args.dtype == "bf16" else None
    prefill["frac"] = round(flops / (prefill["ms"] / 1e3) / peak_flops, 4) if peak_flops else None
    prefill["value"] = round(prefill["value"], 1)
    prefill["ms"] = round(prefill["ms"], 3)
    line = {
        "metric": f"decode tok/s at batch {args.batch} ({name} shape, {args.dtype}, {prompt_len:,}-token prompts)",
        "value": round(head["tokens_per_s"], 1),
        **common,
        "ms_per_step": round(head["ms_per_step"], 4),
        "config": config,
        "e2e": {k: (round(v, 1) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": head["launches"],
        "points": points,
        "prefill": prefill,
        "roofline": {
            "bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": round(achieved / peaks["hbm_gbs"], 4), "points": fractions,
        },
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
