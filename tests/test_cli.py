"""The command line, run as a user runs it: ``python -m distie_b200 <command>`` in a child process.

``init-random`` writes a model folder from a configuration file and a seed; ``generate`` and ``trace``
load it and must produce what the plain implementation produces.  The reference's tools of the same
kind are benchmarks/correctness/hf_parity.py:168-182 and decode_latency.py:29-52 (option names
``--model --dtype --max-new-tokens --num-blocks --prompts --out --warmup --repeats``).
"""

from __future__ import annotations

import json
import os
import subprocess
import sys

import pytest
import torch

import helpers
import plain_qwen2 as plain

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def cli(*args, check=True):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.run([sys.executable, "-m", "distie_b200", *map(str, args)], capture_output=True, text=True,
                          timeout=600, env=env, cwd=ROOT)
    if check:
        assert proc.returncode == 0, proc.stderr[-3000:]
    return proc


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    """A model folder written by ``init-random`` from the first tiny configuration."""
    base = tmp_path_factory.mktemp("cli")
    config = base / "tiny.json"
    config.write_text(json.dumps(helpers.TINY_A))
    out = base / "model"
    proc = cli("init-random", "--config", config, "--out", out, "--seed", 4, "--std", 0.2, "--dtype", "bfloat16")
    assert proc.stdout.strip() == str(out)
    return str(out)


def test_init_random_writes_a_loadable_folder(folder):
    from distie_b200.config import read_config
    from distie_b200.weights import ModelTensors

    arch, typed = read_config(folder)
    assert arch.name == "Qwen2ForCausalLM" and typed.hidden_size == helpers.TINY_A["hidden_size"]
    stored = ModelTensors(folder)
    assert stored.dtype("model.embed_tokens.weight") == torch.bfloat16
    assert "lm_head.weight" not in stored, "tied: the head is the embedding table"
    again = os.path.join(os.path.dirname(folder), "again")
    cli("init-random", "--config", os.path.join(os.path.dirname(folder), "tiny.json"), "--out", again, "--seed", 4,
        "--std", 0.2, "--dtype", "bfloat16")
    other = ModelTensors(again)
    assert all(torch.equal(stored.tensor(n), other.tensor(n)) for n in stored.keys()), "same seed, same weights"


def test_help_names_the_commands_and_says_what_sampling_there_is():
    text = cli("--help").stdout
    for word in ("generate", "trace", "latency", "init-random", "replay", "top-k"):
        assert word in text
    assert "--max-new-tokens" in cli("generate", "--help").stdout


@pytest.mark.gpu
def test_generate_and_trace_match_the_plain_implementation(folder, tmp_path):
    from distie_b200.weights import ModelTensors

    stored = ModelTensors(folder)
    weights = {name: stored.tensor(name).float() for name in stored.keys()}
    cfg = dict(helpers.TINY_A)
    prompts = [helpers.random_ids(cfg["vocab_size"], n, 600 + n) for n in (7, 13, 29)]
    prompt_file = tmp_path / "prompts.json"
    prompt_file.write_text(json.dumps(prompts))
    out_file = tmp_path / "out.json"
    proc = cli("generate", "--model", folder, "--dtype", "fp32", "--prompts", prompt_file, "--max-new-tokens", 16,
               "--num-blocks", 32, "--page-size", 16, "--max-seqs", 4, "--ignore-eos", "--out", out_file)
    report = json.loads(proc.stdout)
    assert report == json.loads(out_file.read_text())
    assert [r["token_ids"] for r in report] == [plain.greedy_generate(p, weights, cfg, 16) for p in prompts]
    assert all(r["finish_reason"] == "length" and r["completion_tokens"] == 16 for r in report)

    # One prompt on the command line, sampled: reproducible from the seed.
    argv = ["generate", "--model", folder, "--dtype", "fp32", "--prompt", " ".join(map(str, prompts[0])),
            "--max-new-tokens", 8, "--temperature", 0.8, "--seed", 3, "--num-blocks", 16, "--ignore-eos"]
    first, second = (json.loads(cli(*argv).stdout)[0]["token_ids"] for _ in range(2))
    assert first == second and len(first) == 8
    helpers.check_sampled_tokens(prompts[0], first, weights, cfg, 0.8, 3)

    forced = [3, 1, 4, 1, 5]
    logits_file = tmp_path / "trace.pt"
    proc = cli("trace", "--model", folder, "--dtype", "fp32", "--prompt", " ".join(map(str, prompts[1])),
               "--max-new-tokens", 5, "--forced-ids", " ".join(map(str, forced)), "--num-blocks", 16, "--out", logits_file)
    report = json.loads(proc.stdout)
    assert report["steps"] == 5 and report["vocab"] == cfg["vocab_size"]
    saved = torch.load(logits_file)
    want = plain.forward_logits(prompts[1] + forced[:-1], weights, cfg)[len(prompts[1]) - 1 :]
    assert float((saved["logits"] - want).abs().max()) <= helpers.FP32_TOL * plain.logit_scale(want)
    assert saved["token_ids"] == want.argmax(-1).tolist()


@pytest.mark.gpu
def test_latency_reports_first_token_and_per_token_times(folder):
    proc = cli("latency", "--model", folder, "--dtype", "bf16", "--prompt", "5 17 3 9", "--max-new-tokens", 8,
               "--warmup", 1, "--repeats", 2, "--num-blocks", 16)
    report = json.loads(proc.stdout)
    assert report["prompt_tokens"] == 4 and report["ttft_ms"] > 0 and report["tpot_ms"] > 0


def test_missing_model_is_refused_with_a_reason():
    proc = cli("generate", "--prompt", "1 2 3", check=False)
    assert proc.returncode != 0 and "--model" in (proc.stderr + proc.stdout)
