"""Command line of the engine: ``python -m distie_b200 <command>``.

Option names and meanings follow the reference where it has them: its tools take
``--model --device --dtype --max-new-tokens --num-blocks --prompts --out``
(benchmarks/correctness/hf_parity.py:168-182) and ``--warmup --repeats --prompt``
(benchmarks/correctness/decode_latency.py:29-52); its worker reads ``WORKER_MODEL``,
``WORKER_DEVICE``, ``WORKER_NUM_BLOCKS``, ``WORKER_MAX_SEQS``, ``WORKER_TOKEN_BUDGET``,
``WORKER_DECODE_GRAPHS`` and ``WORKER_STEP_STATS`` from the environment
(README.md:105-119), which give the defaults here too.  Prompts are token ids:
the reference tokenises with a model library, which is not part of the engine.

Commands
  generate     generate for prompts given as ids (``--prompt`` / ``--prompts`` file), batched together
  trace        one request step by step: arg-max and logits of every step, free-running or teacher-forced
  latency      time-to-first-token and time-per-output-token of one request (warm-up, repeats)
  init-random  write a model folder (config.json, model.safetensors) from a configuration and a seed
  replay       the trace replay program (same as bin/trace_run)

Sampling is greedy (``--temperature 0``) or by temperature; like the reference,
the engine has no top-k, top-p or repetition penalty.
"""

from __future__ import annotations

import argparse
import json
import logging
import os
import sys
import time


def _ids(text: str) -> list[int]:
    return [int(part) for part in text.replace(",", " ").split()]


def _read_prompts(args) -> list[list[int]]:
    prompts: list[list[int]] = []
    if args.prompt:
        prompts += [_ids(p) for p in args.prompt]
    if args.prompts:
        with open(args.prompts, "r", encoding="utf-8") as handle:
            loaded = json.load(handle)
        for item in loaded:
            prompts.append([int(t) for t in (item["prompt_ids"] if isinstance(item, dict) else item)])
    if not prompts:
        raise SystemExit("give --prompt '1 2 3' (repeatable) or --prompts FILE.json (a list of id lists)")
    return prompts


def _engine_options(parser: argparse.ArgumentParser) -> None:
    parser.add_argument("--model", default=os.getenv("WORKER_MODEL"), help="model folder (config.json + safetensors)")
    parser.add_argument("--device", default=os.getenv("WORKER_DEVICE", "cuda"), choices=["cuda"], help="the engine runs on CUDA only")
    parser.add_argument("--dtype", default="bf16", choices=["auto", "bf16", "fp32", "bfloat16", "float32"])
    parser.add_argument("--num-blocks", type=int, default=None, help="KV pages (default WORKER_NUM_BLOCKS or 1024)")
    parser.add_argument("--gpu-mem-fraction", type=float, default=None,
                        help="size the cache from this fraction of the free device memory instead of --num-blocks")
    parser.add_argument("--page-size", type=int, default=None, help="tokens per page (default 16)")
    parser.add_argument("--max-seqs", type=int, default=None, help="requests running at once (default WORKER_MAX_SEQS or 32)")
    parser.add_argument("--token-budget", type=int, default=None, help="tokens per scheduler step (default WORKER_TOKEN_BUDGET or 2048)")
    parser.add_argument("--prefill-chunk", type=int, default=None, help="largest portion of a prompt in one step")
    parser.add_argument("--max-model-len", type=int, default=None, help="longest request the block tables hold")
    parser.add_argument("--no-decode-graphs", action="store_true", help="keep pure-decode steps eager (WORKER_DECODE_GRAPHS=0)")
    parser.add_argument("--step-stats", type=int, default=None, help="log where step time goes every N steps (WORKER_STEP_STATS)")


def _load(args):
    from .engine.engine import Engine

    if not args.model:
        raise SystemExit("--model (or WORKER_MODEL) must name a model folder")
    knobs = dict(
        num_blocks=args.num_blocks, page_size=args.page_size, max_seqs=args.max_seqs, token_budget=args.token_budget,
        prefill_chunk=args.prefill_chunk, max_model_len=args.max_model_len, step_stats=args.step_stats,
        gpu_mem_fraction=args.gpu_mem_fraction,
    )
    if args.no_decode_graphs:
        knobs["decode_graphs"] = False
    return Engine.load(args.model, device=args.device, dtype=args.dtype, **knobs)


def cmd_generate(args) -> int:
    engine = _load(args)
    prompts = _read_prompts(args)
    results = engine.generate(
        prompts, max_new_tokens=args.max_new_tokens, temperature=args.temperature, seed=args.seed,
        eos_id=None if args.ignore_eos else "config", ignore_eos=args.ignore_eos,
    )
    report = [
        {
            "prompt_tokens": r.prompt_tokens, "completion_tokens": r.completion_tokens, "token_ids": r.token_ids,
            "finish_reason": r.finish_reason, "time_to_first_token_ms": round(r.time_to_first_token_ms, 3),
            "total_latency_ms": round(r.total_latency_ms, 3), "preemptions": r.preemptions,
        }
        for r in results
    ]
    text = json.dumps(report, indent=2)
    if args.out:
        with open(args.out, "w", encoding="utf-8") as handle:
            handle.write(text)
    print(text)
    return 0


def cmd_trace(args) -> int:
    engine = _load(args)
    prompt = _read_prompts(args)[0]
    forced = _ids(args.forced_ids) if args.forced_ids else None
    trace = engine.trace(prompt, args.max_new_tokens, forced)
    report = {"token_ids": trace.token_ids, "steps": len(trace.token_ids), "vocab": int(trace.logits.shape[1])}
    if args.out:
        import torch

        torch.save({"token_ids": trace.token_ids, "logits": trace.logits}, args.out)
        report["logits_file"] = args.out
    print(json.dumps(report))
    return 0


def cmd_latency(args) -> int:
    if args.max_new_tokens < 2:
        raise SystemExit("--max-new-tokens must be >= 2 so TPOT has a gap")
    if args.repeats < 1 or args.warmup < 1:
        raise SystemExit("--repeats and --warmup must be >= 1")
    engine = _load(args)
    prompt = _read_prompts(args)[0]
    runs = []
    for index in range(args.warmup + args.repeats):
        stamps = [time.perf_counter()]
        engine.generate(prompt, max_new_tokens=args.max_new_tokens, ignore_eos=True,
                        on_token=lambda *_: stamps.append(time.perf_counter()))
        gaps = [b - a for a, b in zip(stamps, stamps[1:])]
        if index >= args.warmup:
            runs.append({"ttft_ms": gaps[0] * 1e3, "tpot_ms": sum(gaps[1:]) / len(gaps[1:]) * 1e3})
    report = {
        "prompt_tokens": len(prompt), "max_new_tokens": args.max_new_tokens, "repeats": args.repeats,
        "ttft_ms": sum(r["ttft_ms"] for r in runs) / len(runs), "tpot_ms": sum(r["tpot_ms"] for r in runs) / len(runs),
    }
    text = json.dumps(report, indent=2)
    if args.out:
        with open(args.out, "w", encoding="utf-8") as handle:
            handle.write(text)
    print(text)
    return 0


def cmd_init_random(args) -> int:
    from .weights import write_random_model

    with open(args.config, "r", encoding="utf-8") as handle:
        config = json.load(handle)
    folder = write_random_model(args.out, config, seed=args.seed, std=args.std, norm_noise=args.norm_noise, dtype=args.dtype)
    print(folder)
    return 0


def cmd_replay(args) -> int:
    from .engine.trace_replay import main as replay_main

    return replay_main(args.rest)


def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(name)s %(message)s", stream=sys.stderr)
    parser = argparse.ArgumentParser(prog="distie_b200", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    commands = parser.add_subparsers(dest="command", required=True)

    gen = commands.add_parser("generate", help="generate for prompts given as token ids")
    _engine_options(gen)
    gen.add_argument("--prompt", action="append", help="token ids, e.g. '5 17 3' (repeatable)")
    gen.add_argument("--prompts", help="JSON file: a list of id lists (or of {'prompt_ids': [...]})")
    gen.add_argument("--max-new-tokens", type=int, default=16)
    gen.add_argument("--temperature", type=float, default=0.0, help="<= 0: greedy")
    gen.add_argument("--seed", type=int, default=0, help="sampling seed; request i uses seed + i")
    gen.add_argument("--ignore-eos", action="store_true")
    gen.add_argument("--out", help="write the JSON report here")
    gen.set_defaults(run=cmd_generate)

    trace = commands.add_parser("trace", help="one request step by step, logits of every step")
    _engine_options(trace)
    trace.add_argument("--prompt", action="append")
    trace.add_argument("--prompts")
    trace.add_argument("--max-new-tokens", type=int, default=32)
    trace.add_argument("--forced-ids", help="teacher-forced token ids, one per step")
    trace.add_argument("--out", help="write token ids and logits here (torch.save)")
    trace.set_defaults(run=cmd_trace)

    latency = commands.add_parser("latency", help="TTFT and TPOT of one request")
    _engine_options(latency)
    latency.add_argument("--prompt", action="append")
    latency.add_argument("--prompts")
    latency.add_argument("--max-new-tokens", type=int, default=64)
    latency.add_argument("--warmup", type=int, default=2)
    latency.add_argument("--repeats", type=int, default=5)
    latency.add_argument("--out")
    latency.set_defaults(run=cmd_latency)

    init = commands.add_parser("init-random", help="write a model folder with random weights")
    init.add_argument("--config", required=True, help="JSON file with the architecture's config.json keys")
    init.add_argument("--out", required=True, help="folder to write")
    init.add_argument("--seed", type=int, default=0)
    init.add_argument("--std", type=float, default=None, help="default: initializer_range of the config, else 0.02")
    init.add_argument("--norm-noise", type=float, default=0.0)
    init.add_argument("--dtype", default=None, choices=["bfloat16", "float32"])
    init.set_defaults(run=cmd_init_random)

    replay = commands.add_parser("replay", help="trace replay (arguments as bin/trace_run)")
    replay.add_argument("rest", nargs=argparse.REMAINDER)
    replay.set_defaults(run=cmd_replay)

    args = parser.parse_args(argv)
    return args.run(args)


if __name__ == "__main__":
    sys.exit(main())
