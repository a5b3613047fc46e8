"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

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


def shape_from_baseline() -> dict:
    """Layer sizes parsed from the prose of ``BASELINE.json`` ``configs[2]``."""
    try:
        with open(os.path.join(ROOT, "BASELINE.json"), "r", encoding="utf-8") as handle:
            text = json.load(handle)["configs"][2]
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
        return dict(FALLBACK_SHAPE)


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


def build_engine(shape: dict, layers: int, max_seqs: int, num_blocks: int, max_model_len: int = CONTEXT):
    import torch

    from distie_b200.config import EngineConfig, get_architecture
    from distie_b200.engine.engine import Engine
    from distie_b200.kernels import make_kernels
    from distie_b200.models import model_tensor_specs
    from distie_b200.weights import RandomSource

    raw = {"architectures": ["Qwen2ForCausalLM"], **shape, "num_hidden_layers": layers, "max_position_embeddings": 32768}
    arch = get_architecture("Qwen2ForCausalLM")
    typed = arch.config_cls.from_dict(raw)
    kernels = make_kernels(torch.bfloat16, "cuda:0")
    source = RandomSource(model_tensor_specs(arch.recipe(typed)), seed=0, std=0.02, dtype=torch.bfloat16, device="cuda:0")
    config = EngineConfig(
        num_blocks=num_blocks, page_size=PAGE, max_seqs=max_seqs, token_budget=2048, max_model_len=max_model_len,
        dtype="bfloat16", decode_graphs=True, device="cuda:0",
    )
    return Engine.assemble(arch, typed, source, kernels, config)


def random_prompt(vocab: int, length: int, seed: int) -> list[int]:
    import torch

    return torch.randint(0, vocab, (length,), generator=torch.Generator().manual_seed(seed)).tolist()


def fill_requests(engine, batch: int, total_new: int):
    """`batch` requests with their 1,024-token prompts in the cache and pages for `total_new` more tokens."""
    from distie_b200.engine.batch import BatchEntry
    from distie_b200.engine.scheduler import ScheduledSeq, Sequence

    vocab = engine.model.vocab_size
    seqs = []
    for b in range(batch):
        seq = Sequence(f"bench-{b}", random_prompt(vocab, PROMPT_LEN, 100 + b), total_new)
        seq.seat = engine.cache.open_seat()
        assert engine.cache.grow(seq.seat, PROMPT_LEN + total_new + 1), "the bench pool is too small"
        seqs.append(seq)
    for start in range(0, batch, 2):  # two prompts (2,048 tokens) per prefill step
        group = seqs[start : start + 2]
        engine.runner.step([BatchEntry(s.seat, s.prompt_ids[:-1], 0, ()) for s in group])
    engine.runner.finish_step()
    return [ScheduledSeq(s, [s.prompt_ids[-1]], PROMPT_LEN - 1, True) for s in seqs], seqs


def release(engine, seqs) -> None:
    for seq in seqs:
        engine.cache.close_seat(seq.seat)


def time_decode(engine, batch: int, steps: int, warmup: int) -> dict:
    """K decode steps back to back on the device, after W warm-up steps; CUDA events around them."""
    import torch

    items, seqs = fill_requests(engine, batch, warmup + steps)
    engine.runner.decode_burst(items, max(warmup, 1))
    # The burst advanced the positions on the device; mirror that in the items of the timed burst.
    advanced = [type(item)(item.seq, item.token_ids, item.past_len + max(warmup, 1), True) for item in items]
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    bucket = engine.runner._buckets[engine.runner.bucket_for(batch)]
    begin.record()
    tokens = engine.runner.decode_burst(advanced, steps)
    end.record()
    torch.cuda.synchronize()
    ms = begin.elapsed_time(end)
    engine.runner.finish_step()
    assert tokens.shape == (steps, batch)
    mean_context = PROMPT_LEN + max(warmup, 1) + steps / 2
    release(engine, seqs)
    return {
        "ms_per_step": ms / steps,
        "tokens_per_s": batch * steps / (ms / 1e3),
        "mean_context": mean_context,
        "launches": bucket.kernels_per_replay * steps,
    }


def time_e2e(engine, batch: int, steps: int, warmup: int) -> dict:
    """The same decode steps through ``Engine.step``: host planning, pinned staging, replay, ids back."""
    import torch

    from distie_b200.engine.scheduler import Sequence

    vocab = engine.model.vocab_size
    for b in range(batch):
        engine.scheduler.submit(Sequence(f"e2e-{b}", random_prompt(vocab, PROMPT_LEN, 500 + b), warmup + steps + 8))
    while any(s.num_pending > 1 for s in engine.scheduler._running) or engine.scheduler.num_waiting:
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
    for b in range(batch):
        engine.scheduler.abort(f"e2e-{b}")
    engine.drain()
    engine.scheduler.schedule()
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
    for _ in range(repeats + 2):
        seat = engine.cache.open_seat()
        assert engine.cache.grow(seat, past + PREFILL_TOKENS)
        for start in range(0, past, PREFILL_TOKENS):  # the earlier portions, untimed
            engine.runner.step([BatchEntry(seat, prompt[start : min(past, start + PREFILL_TOKENS)], start, ())])
            engine.runner.finish_step()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        engine.runner.step([BatchEntry(seat, prompt[past:], past, (PREFILL_TOKENS - 1,))])
        end.record()
        torch.cuda.synchronize()
        times.append(begin.elapsed_time(end))
        engine.runner.finish_step()
        engine.cache.close_seat(seat)
    ms = statistics.median(times[2:])
    return {"ms": ms, "tokens": PREFILL_TOKENS, "past": past, "value": PREFILL_TOKENS / (ms / 1e3)}


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
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--only", default=None, choices=["decode", "prefill"],
                        help="run one part and print a short line (for profiling captures; not a bench value)")
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

    shape = shape_from_baseline()
    layers_full = shape["num_hidden_layers"]
    layers = args.layers or layers_full
    peaks, peaks_kind = measured_peaks()
    new_tokens = args.warmup + args.steps + 8
    pages = 64 * -(-(PROMPT_LEN + new_tokens + 1) // PAGE) + 2 * (PREFILL_TOKENS // PAGE)
    if args.only == "prefill" and args.past > 0:
        pages = 2 * -(-(args.past + PREFILL_TOKENS) // PAGE)
        engine = build_engine(shape, layers, 8, pages, max(CONTEXT, args.past + PREFILL_TOKENS))
    else:
        engine = build_engine(shape, layers, 64, pages)
    weight_bytes = engine.model.weight_bytes()
    kv_bytes_per_token = engine.cache.bytes_per_token()

    if args.only == "decode":
        print(json.dumps({"only": "decode", "batch": args.batch, "layers": layers, **time_decode(engine, args.batch, args.steps, args.warmup)}))
        return 0
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "layers": layers, **time_prefill(engine, repeats=max(1, args.steps), past=args.past)}))
        return 0

    with ClockSampler() as sampler:
        head = time_decode(engine, args.batch, args.steps, args.warmup)
        e2e = time_e2e(engine, args.batch, args.steps, args.warmup)
        points = {}
        for batch in (1, 64):
            points[f"decode_b{batch}"] = round(time_decode(engine, batch, args.steps, args.warmup)["tokens_per_s"], 1)
        prefill = time_prefill(engine)
        time.sleep(0.3)
    clocks = sampler.summary()

    step_bytes = weight_bytes + args.batch * head["mean_context"] * kv_bytes_per_token
    achieved = step_bytes / (head["ms_per_step"] / 1e3) / 1e9
    flops = prefill_flops(shape, layers, PREFILL_TOKENS)
    prefill.pop("past", None)
    prefill["frac"] = round(flops / (prefill["ms"] / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)
    prefill["value"] = round(prefill["value"], 1)
    prefill["ms"] = round(prefill["ms"], 3)
    line = {
        "metric": "decode tok/s at batch 8 (Qwen2.5-1.5B shape, bf16, 1,024-token prompts)",
        "value": round(head["tokens_per_s"], 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(head["ms_per_step"], 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: random N(0,0.02) weights, uniform random token ids",
        "impl": "ours",
        "config": {
            "model": "Qwen2.5-1.5B shape (Qwen2ForCausalLM)", "layers": layers, "layers_full": layers_full,
            "hidden": shape["hidden_size"], "q_heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
            "head_dim": shape["head_dim"], "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
            "tied": shape["tie_word_embeddings"], "global_batch": args.batch, "prompt_len": PROMPT_LEN,
            "seq_len": CONTEXT, "page_size": PAGE, "parallelism": "none (1 GPU)", "decode": "CUDA graph per batch bucket",
            "l2": "inputs larger than L2 (3 GB of weights per step)", "peaks": peaks_kind,
        },
        "e2e": {k: (round(v, 1) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": head["launches"],
        "points": points,
        "prefill": prefill,
        "roofline": {
            "bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": round(achieved / peaks["hbm_gbs"], 4),
        },
        "clocks": clocks,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
