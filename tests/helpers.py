"""Shared pieces of the tests: the two tiny configurations, weights, replay schedules, comparisons."""

from __future__ import annotations

import random

import torch

import plain_qwen2 as plain

# Two tiny configurations of the architecture that differ in every size and option.
TINY_A = {
    "architectures": ["Qwen2ForCausalLM"],
    "vocab_size": 256,
    "hidden_size": 64,
    "intermediate_size": 160,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "rms_norm_eps": 1e-6,
    "rope_theta": 10000.0,
    "tie_word_embeddings": True,
    "max_position_embeddings": 512,
}
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"],
    "vocab_size": 384,
    "hidden_size": 96,
    "intermediate_size": 224,
    "num_hidden_layers": 3,
    "num_attention_heads": 3,
    "num_key_value_heads": 1,
    "rms_norm_eps": 1e-5,
    "rope_theta": 1000000.0,
    "tie_word_embeddings": False,
    "max_position_embeddings": 1024,
}
# Two more with the head sizes of real models (64 and 128): in bfloat16 these run on the tensor-core
# attention kernels and, from 128 rows on, the tensor-core products, which the first two never reach.
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"],
    "vocab_size": 1000,
    "hidden_size": 256,
    "intermediate_size": 416,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 64,
    "rms_norm_eps": 1e-6,
    "rope_theta": 10000.0,
    "tie_word_embeddings": True,
    "max_position_embeddings": 2048,
}
TINY_D = {
    "architectures": ["Qwen2ForCausalLM"],
    "vocab_size": 2003,
    "hidden_size": 512,
    "intermediate_size": 1384,
    "num_hidden_layers": 3,
    "num_attention_heads": 4,
    "num_key_value_heads": 1,
    "head_dim": 128,
    "rms_norm_eps": 1e-5,
    "rope_theta": 1000000.0,
    "tie_word_embeddings": False,
    "max_position_embeddings": 4096,
}
# Sizes chosen to be awkward: a head size that is no power of two, as many kv heads as heads, an intermediate
# size that is no multiple of 8, an odd vocabulary, pages of 4 tokens.
TINY_E = {
    "architectures": ["Qwen2ForCausalLM"],
    "vocab_size": 1001,
    "hidden_size": 240,
    "intermediate_size": 250,
    "num_hidden_layers": 2,
    "num_attention_heads": 5,
    "num_key_value_heads": 5,
    "head_dim": 48,
    "rms_norm_eps": 1e-6,
    "rope_theta": 50000.0,
    "tie_word_embeddings": False,
    "max_position_embeddings": 1024,
}
# config, page size, seed, norm noise
TINY = {"A": (TINY_A, 16, 0, 0.0), "B": (TINY_B, 8, 1, 0.02), "C": (TINY_C, 16, 2, 0.0), "D": (TINY_D, 32, 3, 0.02),
        "E": (TINY_E, 4, 4, 0.02)}
# Standard deviation of the test weights per configuration: wide layers need smaller weights for logits
# of a scale at which a wrong key shows without saturating the softmax.
STD = {"A": 0.2, "B": 0.2, "C": 0.1, "D": 0.07, "E": 0.1}

# Weights far larger than N(0, 0.02): logits then have a scale at which a wrong key shows.
TEST_STD = 0.2

FP32_TOL = 1e-4   # max |diff| / logit scale, float32 engine against the plain implementation
# bfloat16 has no fixed tolerance: what the dtype itself costs is measured by running the plain
# implementation with bfloat16 tensors (the reference's formulas, rounding after every operation),
# and the engine, which keeps more in 32-bit, must stay within that: see `Bf16Budget`.
BF16_RMS_MARGIN = 1.0    # pooled rms error: at most what the formulas in bfloat16 cost
BF16_MAX_MARGIN = 2.0    # largest single error: at most twice the largest of the formulas in bfloat16
BF16_TOP1_MARGIN = 0.02  # pooled top-1 agreement may fall this far below theirs


def tiny(name: str):
    cfg, page, seed, noise = TINY[name]
    return dict(cfg), page, plain.random_weights(cfg, seed, std=STD[name], norm_noise=noise)


def bf16_rounded(weights: dict) -> dict:
    return {k: v.to(torch.bfloat16).float() for k, v in weights.items()}


def random_ids(vocab: int, length: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


# -- replay schedules -----------------------------------------------------------
def schedule_whole(requests: dict) -> list[dict]:
    return [
        {"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]}
        for i, (rid, ids) in enumerate(requests.items())
    ]


def schedule_tail(requests: dict, tail: int = 32) -> list[dict]:
    """Most of each request in one step, the last `tail` tokens one by one."""
    steps, n = [], 0
    for rid, ids in requests.items():
        head = max(1, len(ids) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": ids[:head], "want": list(range(head))}], "end": []})
        n += 1
        for at in range(head, len(ids)):
            steps.append(
                {"step": n, "entries": [{"id": rid, "tokens": [ids[at]], "want": [0]}], "end": [rid] if at == len(ids) - 1 else []}
            )
            n += 1
        if head == len(ids):
            steps[-1]["end"] = [rid]
    return steps


PORTIONS = (7, 2, 13, 2, 5, 3, 11, 2, 17, 4, 2, 29, 2, 9)


def schedule_portions(requests: dict) -> list[dict]:
    steps, n = [], 0
    for rid, ids in requests.items():
        at, turn = 0, 0
        while at < len(ids):
            size = min(PORTIONS[turn % len(PORTIONS)], len(ids) - at)
            if len(ids) - at - size == 1:  # never leave a single token over: portions go down to two
                size += 1
            turn += 1
            steps.append(
                {
                    "step": n,
                    "entries": [{"id": rid, "tokens": ids[at : at + size], "want": list(range(size))}],
                    "end": [rid] if at + size == len(ids) else [],
                }
            )
            at += size
            n += 1
    return steps


def schedule_mixed(requests: dict, seed: int = 0, live_max: int = 4, refeed: int = 0,
                   sizes: tuple = (2, 3, 5, 8, 13, 21, 40)) -> list[dict]:
    """Up to four live requests; portions of some beside single tokens of others; some sit a step out.

    With ``refeed`` that many requests are ended early, once each, somewhere past their middle (what a
    preemption does: their pages go back) and fed again from position 0 later, under the same id.
    """
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: dict[str, int] = {}
    sent_back: set[str] = set()
    steps, n = [], 0
    while waiting or live:
        while waiting and len(live) < live_max and (not live or rng.random() < 0.7):
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, end = [], []
        for rid in list(live):
            ids, at = requests[rid], live[rid]
            if len(live) > 1 and rng.random() < 0.2:
                continue  # left out of this step, goes on later
            if len(sent_back) < refeed and rid not in sent_back and at >= len(ids) // 2 and steps:
                sent_back.add(rid)  # given up after the step before; comes back from position 0
                steps[-1]["end"].append(rid)
                del live[rid]
                waiting.insert(min(1, len(waiting)), (rid, ids))
                continue
            left = len(ids) - at
            if at > 0 and rng.random() < 0.5:
                size = 1
            else:
                size = min(left, rng.choice(sizes))
            if left - size == 1 and size > 1:
                size += 1
            entries.append({"id": rid, "tokens": ids[at : at + size], "want": list(range(size))})
            live[rid] = at + size
            if live[rid] == len(ids):
                end.append(rid)
                del live[rid]
        if not entries:
            continue
        steps.append({"step": n, "entries": entries, "end": end})
        n += 1
    return steps


def peak_tokens(steps: list[dict], granule: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to `granule`."""
    held: dict[str, int] = {}
    peak = 0
    for step in steps:
        for entry in step["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        peak = max(peak, sum(-(-v // granule) * granule for v in held.values()))
        for rid in step["end"]:
            held.pop(rid, None)
    return peak


def collect(steps: list[dict], outputs: dict) -> dict:
    """Per request, the logits of every position, gathered from per-step outputs {step: array [wanted, vocab]}.

    A request that was ended early and fed again appears twice: the pass that was given up under
    ``"<id>#<n>"`` (its first positions only), the complete one under its id; see `expected_for`.
    """
    rows: dict[str, dict[int, torch.Tensor]] = {}
    cursor: dict[str, int] = {}
    passes: dict[str, int] = {}
    done: dict[str, torch.Tensor] = {}
    for step in steps:
        out = outputs.get(step["step"])
        at = 0
        for entry in step["entries"]:
            base = cursor.get(entry["id"], 0)
            for place in entry["want"]:
                rows.setdefault(entry["id"], {})[base + place] = torch.as_tensor(out[at])
                at += 1
            cursor[entry["id"]] = base + len(entry["tokens"])
        for rid in step["end"]:
            held = rows.pop(rid, None)
            cursor.pop(rid, None)
            if held is None:
                continue
            if rid in done:  # an earlier pass was given up: keep it under a name of its own
                passes[rid] = passes.get(rid, 0) + 1
                done[f"{rid}#{passes[rid]}"] = done[rid]
            done[rid] = torch.stack([held[i] for i in sorted(held)])
    for rid, held in rows.items():  # schedules that never end their requests
        done[rid] = torch.stack([held[i] for i in sorted(held)])
    return done


def expected_for(got: dict, expected: dict) -> dict:
    """`expected` with an entry for every pass `collect` found: a pass that was given up is compared
    with the first positions of its request."""
    out = dict(expected)
    for key, value in got.items():
        if "#" in key:
            out[key] = expected[key.split("#")[0]][: value.shape[0]]
    return out


def run_schedule(session, steps: list[dict]) -> dict:
    outputs = {}
    for step in steps:
        result = session.run_step(step["entries"], step["end"])
        if result is not None:
            outputs[step["step"]] = result
    return outputs


def worst_error(got: dict, expected: dict) -> tuple[float, str, int]:
    """(max |diff| / scale, request, position) over all requests."""
    worst = (0.0, "", -1)
    for rid, want in expected.items():
        have = got[rid]
        assert have.shape == want.shape, (rid, have.shape, want.shape)
        scale = plain.logit_scale(want)
        diff = (have.float() - want).abs().max(dim=-1).values / scale
        at = int(diff.argmax())
        if float(diff[at]) > worst[0]:
            worst = (float(diff[at]), rid, at)
    return worst


def first_bad_position(have: torch.Tensor, want: torch.Tensor, tol: float) -> int | None:
    scale = plain.logit_scale(want)
    bad = ((have.float() - want).abs().max(dim=-1).values / scale) > tol
    return int(bad.nonzero()[0]) if bool(bad.any()) else None


class Bf16Budget:
    """Errors of the plain implementation run in bfloat16 against its float32 run, pooled over requests.

    Per-request maxima are too noisy to compare (one near-tie in a softmax moves them by a factor
    of two), so the budget pools: the rms over every logit of every request, the largest single
    error, and the share of positions with the same arg-max.  One position that is wrong by a third
    of the logit scale among thousands already doubles the pooled rms.
    """

    def __init__(self, requests: dict, weights: dict, cfg: dict, expected: dict, skip: int = 0, order=None) -> None:
        low = {k: v.to(torch.bfloat16) for k, v in weights.items()}
        rough = {rid: plain.forward_logits(ids, low, cfg, order=order)[skip:] for rid, ids in requests.items()}
        self.max_error, self.rms_error, self.top1 = pooled_stats(rough, {r: expected[r][-rough[r].shape[0]:] for r in rough})

    def check(self, got: dict, expected: dict, what: str = "") -> None:
        worst, rms, top1 = pooled_stats(got, expected)
        assert rms <= BF16_RMS_MARGIN * self.rms_error, (
            f"{what}: pooled rms error {rms:.3e} of the logit scale; the formulas in bfloat16 cost {self.rms_error:.3e}"
        )
        assert worst <= BF16_MAX_MARGIN * self.max_error, (
            f"{what}: largest error {worst:.3e} of the logit scale; the formulas in bfloat16 reach {self.max_error:.3e}"
        )
        assert top1 >= self.top1 - BF16_TOP1_MARGIN, f"{what}: top-1 agreement {top1:.3f}, theirs {self.top1:.3f}"


def pooled_stats(have: dict, want: dict) -> tuple[float, float, float]:
    """(largest, rms) of |diff| / logit scale over all requests, and the pooled top-1 agreement."""
    diffs, same = [], []
    for rid, target in want.items():
        assert have[rid].shape == target.shape, (rid, have[rid].shape, target.shape)
        diffs.append(((have[rid].float() - target).abs() / plain.logit_scale(target)).flatten())
        same.append((have[rid].argmax(-1) == target.argmax(-1)).float())
    diff, same = torch.cat(diffs), torch.cat(same)
    return float(diff.max()), float(diff.pow(2).mean().sqrt()), float(same.mean())


def error_stats(have: torch.Tensor, want: torch.Tensor) -> tuple[float, float, float]:
    """(max, rms) of |diff| / logit scale and the share of positions with the same arg-max."""
    diff = (have.float() - want).abs() / plain.logit_scale(want)
    top1 = float((have.argmax(-1) == want.argmax(-1)).float().mean())
    return float(diff.max()), float(diff.pow(2).mean().sqrt()), top1


# -- a toy arrangement of the architecture's own parts: the run order as data -----------------------
TOY_WINDOW = 9
# (layer, window of its attention, call whose keys and values it reads instead of writing its own)
TOY_ORDER = [(0, None, None), (1, TOY_WINDOW, None), (0, None, None), (2, TOY_WINDOW, 1)]


def toy_arrangement_spec(cfg: dict):
    """Configuration B's parts arranged differently: layer 1 and 2 attend through a window, layer 0 runs
    twice (each call with a cache slot of its own), and layer 2 reads the keys and values that layer 1
    wrote instead of writing any.  The plain counterpart is ``plain.forward_logits(order=TOY_ORDER)``."""
    from dataclasses import replace

    from distie_b200.config import LayerCall, PartSpec, get_architecture

    arch = get_architecture(cfg["architectures"][0])
    spec = arch.recipe(arch.config_cls.from_dict(cfg))
    layers = list(spec.layers)
    for index in (1, 2):
        mixer = layers[index].mixer
        layers[index] = replace(layers[index], mixer=PartSpec(mixer.kind, {**mixer.params, "window": TOY_WINDOW}, mixer.prefix))
    order = (LayerCall(0, 0, True), LayerCall(1, 1, True), LayerCall(0, 2, True), LayerCall(2, 1, False))
    return replace(spec, layers=tuple(layers), order=order)


# -- temperature sampling against an oracle -------------------------------------------------------------
def check_sampled_tokens(prompt, outputs, weights, cfg, temperature: float, seed: int, slack: float = 2e-4) -> None:
    """Every sampled token must be the inverse-CDF pick of the plain implementation's distribution.

    Output ``i`` of a request is drawn at ``u = uniform(seed, i)`` from
    ``plain.temperature_probabilities(logits after prompt + outputs[:i])``: the first token whose cumulative
    probability exceeds ``u``.  The engine's logits differ from the plain ones by rounding, so a token
    next to the oracle's is accepted when ``u`` lies within ``slack`` of the boundary between the two.
    """
    from distie_b200.sampling.sampler import uniform

    ids = list(prompt) + list(outputs)
    logits = plain.forward_logits(ids[:-1], weights, cfg)[len(prompt) - 1 :]
    assert logits.shape[0] == len(outputs)
    for index, token in enumerate(outputs):
        cdf = torch.cumsum(plain.temperature_probabilities(logits[index], temperature).double(), dim=0)
        u = uniform(seed, index) * float(cdf[-1])
        low = float(cdf[token - 1]) if token > 0 else 0.0
        high = float(cdf[token])
        assert low - slack <= u < high + slack, (
            f"output {index}: token {token} covers [{low:.6f}, {high:.6f}) of the cumulative distribution, u = {u:.6f}"
        )


TINY_B_PROMPTS = (1, 5, 17, 40, 63)  # the workload of the second tiny configuration: prompts of these lengths,
TINY_B_CHUNK, TINY_B_STEPS, TINY_B_TEMPERATURE, TINY_B_SEED = 11, 24, 0.8, 1  # portions of 11, 24 tokens each at T = 0.8


def run_tiny_b_workload(engine, cfg):
    """Five requests, prompts cut into portions of 11 beside decoding ones, temperature 0.8 from seed 1, 24
    tokens each, and one preemption forced on the request that was admitted last once it has decoded a few
    tokens.  Returns (prompts, results)."""
    from distie_b200.engine.engine import GenerateRequest

    prompts = [random_ids(cfg["vocab_size"], n, 400 + n) for n in TINY_B_PROMPTS]
    requests = [GenerateRequest(f"w{i}", p, TINY_B_STEPS, TINY_B_TEMPERATURE, TINY_B_SEED + i) for i, p in enumerate(prompts)]
    forced, seen = [], []

    def on_token(request_id, token, finished):
        # Called between steps (a step ahead may already be in flight: its row for this request is dropped).
        if request_id == "w4":
            seen.append(token)
            if len(seen) == 5:
                forced.append(engine.scheduler.force_preempt("w4"))

    results = engine.run(requests, ignore_eos=True, on_token=on_token)
    assert forced == [True], "the forced preemption did not happen"
    return prompts, results
