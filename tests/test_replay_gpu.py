"""Trace replay on the GPU against the plain implementation: every way of cutting, float32 and bfloat16."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MODES = {
    "whole": helpers.schedule_whole,
    "tail": helpers.schedule_tail,
    "portions": helpers.schedule_portions,
    # two requests are ended early and fed again from position 0, as a preemption does
    "mixed": lambda requests: helpers.schedule_mixed(requests, refeed=2),
}
LENGTHS = [40, 67, 33, 300, 50, 36, 129, 64]
# What a bfloat16 engine with head sizes 64 or 128 must have launched in each mode: prompts of 128 tokens
# and more take the tensor-core product (q/k/v with the rotation and the cache write in its epilogue), shorter
# steps the weight-streaming one; portions take the tensor-core prefill attention, steps of single tokens the
# tensor-core decode attention.
SERVING_KERNELS = {
    "whole": {"attention_prefill_tcgen05", "gemm_tcgen05", "gemm_tcgen05_qkv", "gemm_tcgen05_skinny"},
    "tail": {"attention_prefill_tcgen05", "attention_decode_mma", "gemm_tcgen05", "gemm_tcgen05_qkv", "gemm_tcgen05_skinny"},
    "portions": {"attention_prefill_tcgen05", "gemm_tcgen05_skinny"},
    "mixed": {"attention_prefill_tcgen05", "attention_decode_mma", "gemm_tcgen05_skinny"},
}


@pytest.fixture(scope="module", params=["A", "B", "C", "D", "E"])
def model(request, tmp_path_factory):
    """A model folder of the tiny configuration, written by the random-weights mode, and its plain logits."""
    from distie_b200.weights import ModelTensors, write_random_model

    cfg, page, _ = helpers.tiny(request.param)
    noise = helpers.TINY[request.param][3]
    folder = str(tmp_path_factory.mktemp(f"tiny{request.param}"))
    write_random_model(folder, cfg, seed=helpers.TINY[request.param][2], std=helpers.STD[request.param], norm_noise=noise, dtype="bfloat16")
    stored = ModelTensors(folder)
    weights = {name: stored.tensor(name).float() for name in stored.keys()}
    requests = {f"r{i}": helpers.random_ids(cfg["vocab_size"], n, 10 + i) for i, n in enumerate(LENGTHS)}
    expected = {rid: plain.forward_logits(ids, weights, cfg) for rid, ids in requests.items()}
    budget = helpers.Bf16Budget(requests, weights, cfg, expected)
    return {"folder": folder, "cfg": cfg, "page": page, "requests": requests, "expected": expected, "budget": budget,
            "name": request.param}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", list(MODES))
def test_replay_matches_plain(model, mode, dtype):
    from distie_b200.engine.trace_replay import TraceSession

    steps = MODES[mode](model["requests"])
    session = TraceSession.open(model["folder"], dtype, helpers.peak_tokens(steps), page_size=model["page"])
    got = helpers.collect(steps, helpers.run_schedule(session, steps))
    expected = helpers.expected_for(got, model["expected"])
    if mode == "mixed":
        assert any("#" in key for key in got), "the schedule was meant to give a request up and feed it again"
    if dtype == "float32":
        error, rid, at = helpers.worst_error(got, expected)
        if error > helpers.FP32_TOL:
            first = helpers.first_bad_position(got[rid], expected[rid], helpers.FP32_TOL)
            pytest.fail(
                f"{mode}: request {rid} (length {len(model['requests'][rid.split('#')[0]])}) first wrong at position {first}, "
                f"worst {error:.2e} of the logit scale at {at}"
            )
    else:
        model["budget"].check(got, expected, mode)
    runner = session.engine.runner
    if mode == "tail":  # the last 32 tokens one by one are steps of single tokens: the captured decode step ran them
        assert runner.graph_replays > 0, "steps of single tokens were meant to replay the captured decode step"
    if dtype == "bfloat16" and model["name"] in "CD":
        # The kernels serving runs on are the ones that were held to the oracle here.
        ran = {name for name, count in runner.kernels.kernel_counts.items() if count}
        assert SERVING_KERNELS[mode] <= ran, f"{mode}: expected {sorted(SERVING_KERNELS[mode] - ran)} to have run; ran {sorted(ran)}"
    cache = session.engine.cache
    assert cache.free_pages() == cache.total_pages() and cache.free_seats == cache.max_seats


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tail_without_graphs_matches_too(model, dtype):
    """The same steps of single tokens run eagerly: both forms of the decode step are held to the oracle."""
    from distie_b200.engine.trace_replay import TraceSession

    if model["name"] in "AB":
        pytest.skip("covered at the head sizes the serving kernels take")
    steps = helpers.schedule_tail(model["requests"])
    session = TraceSession.open(model["folder"], dtype, helpers.peak_tokens(steps), page_size=model["page"], decode_graphs=False)
    got = helpers.collect(steps, helpers.run_schedule(session, steps))
    assert session.engine.runner.graph_replays == 0
    if dtype == "float32":
        error, rid, at = helpers.worst_error(got, model["expected"])
        assert error <= helpers.FP32_TOL, f"request {rid} position {at} off by {error:.2e} of the logit scale"
    else:
        model["budget"].check(got, model["expected"], "tail, eager")


def test_trace_run_program(model, tmp_path):
    """The program itself: JSON lines in, done lines and .f32 files out, exit code 0."""
    steps = helpers.schedule_mixed(model["requests"], seed=3)
    out_dir = tmp_path / "out"
    text = "".join(json.dumps(step) + "\n" for step in steps)
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model["folder"], "--dtype", "float32",
         "--out", str(out_dir), "--max-tokens", str(helpers.peak_tokens(steps)), "--page-size", str(model["page"])],
        input=text, capture_output=True, text=True, timeout=600,
    )
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[: len(steps)] == [f"done {s['step']}" for s in steps]
    vocab = model["cfg"]["vocab_size"]
    outputs = {s["step"]: np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab) for s in steps}
    got = helpers.collect(steps, outputs)
    error, rid, at = helpers.worst_error(got, helpers.expected_for(got, model["expected"]))
    assert error <= helpers.FP32_TOL, f"request {rid} position {at} off by {error:.2e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "tail", "mixed"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_run_order_is_data_on_the_gpu(mode, dtype, name):
    """The toy arrangement (a layer twice, a layer reading another's keys and values, windows on some
    layers): built from the same parts by a different list, replayed with the CUDA kernels; with
    configuration D in bfloat16 these are the tensor-core kernels, the merged ones included (a layer that
    writes no keys and values of its own, a window)."""
    from distie_b200.config import EngineConfig
    from distie_b200.engine.engine import Engine, build_cache
    from distie_b200.engine.trace_replay import TraceSession
    from distie_b200.kernels import make_kernels
    from distie_b200.models.decoder import DecoderModel, model_tensor_specs
    from distie_b200.weights import open_weights

    cfg, page, weights = helpers.tiny(name)
    weights = helpers.bf16_rounded(weights)
    spec = helpers.toy_arrangement_spec(cfg)
    requests = {f"r{i}": helpers.random_ids(cfg["vocab_size"], n, 60 + i) for i, n in enumerate([40, 67, 33, 200, 50, 36])}
    steps = MODES[mode](requests)
    kernels = make_kernels(torch.float32 if dtype == "float32" else torch.bfloat16, "cuda:0")
    config = EngineConfig(num_blocks=helpers.peak_tokens(steps) // page, page_size=page, max_seqs=8, dtype=dtype,
                          device="cuda:0", token_budget=4096)
    store = open_weights(weights, model_tensor_specs(spec), spec.tolerated, kernels.dtype, kernels.device)
    cache = build_cache(spec, config, kernels.dtype, kernels.device)
    engine = Engine(DecoderModel(spec, kernels, store), cache, config)
    got = helpers.collect(steps, helpers.run_schedule(TraceSession(engine), steps))
    expected = {rid: plain.forward_logits(ids, weights, cfg, order=helpers.TOY_ORDER) for rid, ids in requests.items()}
    if dtype == "float32":
        error, rid, at = helpers.worst_error(got, expected)
        assert error <= helpers.FP32_TOL, f"{mode}: request {rid} position {at} off by {error:.2e} of the logit scale"
    else:
        helpers.Bf16Budget(requests, weights, cfg, expected, order=helpers.TOY_ORDER).check(got, expected, mode)
        if name == "D" and mode == "tail":
            ran = {kernel for kernel, count in kernels.kernel_counts.items() if count}
            assert {"attention_decode_mma_qkv", "gemm_tcgen05_qkv", "attention_prefill_tcgen05"} <= ran, sorted(ran)
    assert cache.free_pages() == cache.total_pages() and cache.free_seats == cache.max_seats

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [1, 2, 3, 4])
@pytest.mark.parametrize("name", ["C", "D"])
def test_random_schedules_with_long_portions(name, seed, dtype, tmp_path_factory):
    """Seeded random schedules whose portions reach 130 and 260 tokens, so that steps hold prompt portions on the
    tensor-core product and attention kernels beside single tokens of other requests, with requests ended early
    and fed again and so few pages that they are used again."""
    from distie_b200.engine.trace_replay import TraceSession
    from distie_b200.weights import ModelTensors, write_random_model

    cfg, page, _ = helpers.tiny(name)
    folder = str(tmp_path_factory.mktemp(f"fuzz{name}"))
    write_random_model(folder, cfg, seed=helpers.TINY[name][2], std=helpers.STD[name], norm_noise=helpers.TINY[name][3], dtype="bfloat16")
    stored = ModelTensors(folder)
    weights = {n: stored.tensor(n).float() for n in stored.keys()}
    lengths = [300, 70, 410, 33, 150, 260, 64]
    requests = {f"r{i}": helpers.random_ids(cfg["vocab_size"], n, 500 + 10 * seed + i) for i, n in enumerate(lengths)}
    steps = helpers.schedule_mixed(requests, seed=seed, refeed=2, sizes=(2, 5, 17, 40, 130, 260))
    session = TraceSession.open(folder, dtype, helpers.peak_tokens(steps), page_size=page)
    got = helpers.collect(steps, helpers.run_schedule(session, steps))
    expected = helpers.expected_for(got, {rid: plain.forward_logits(ids, weights, cfg) for rid, ids in requests.items()})
    if dtype == "float32":
        error, rid, at = helpers.worst_error(got, expected)
        assert error <= helpers.FP32_TOL, f"seed {seed}: request {rid} position {at} off by {error:.2e} of the logit scale"
    else:
        full = {rid: plain.forward_logits(ids, weights, cfg) for rid, ids in requests.items()}
        helpers.Bf16Budget(requests, weights, cfg, full).check(got, expected, f"seed {seed}")
        ran = {kernel for kernel, count in session.engine.runner.kernels.kernel_counts.items() if count}
        assert {"attention_prefill_tcgen05", "gemm_tcgen05", "attention_decode_mma"} <= ran, sorted(ran)
    cache = session.engine.cache
    assert cache.free_pages() == cache.total_pages() and cache.free_seats == cache.max_seats
