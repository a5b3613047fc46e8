"""The float32 gate and the bfloat16 budget at the layer widths of real models.

Two layers each of the Qwen2.5-1.5B, 7B and 14B shapes (hidden, heads, kv heads, head size,
intermediate size, vocabulary and eps as those models have them; only the number of layers is
cut), random weights, every way of cutting: whole prompts, the last 32 tokens one by one
(replayed from the captured decode step), portions down to two tokens, and a mixed schedule (portions of up
to 130 tokens beside single tokens of other requests, one request given up and fed again).  The reference's own
harness for this is benchmarks/correctness/hf_parity.py:92-113 with the thresholds of
benchmarks/correctness/metrics.py:16-22 (float32: same arg-max and 1e-3 absolute; 16-bit:
top-1 agreement of 0.98); the gate here is the stricter one of the other tests: float32 within
1e-4 of the logit scale, bfloat16 within what the reference's formulas cost when they are
evaluated in bfloat16 themselves.

The plain implementation runs on the GPU here (float32 library products without TF32): at
these widths the CPU would take minutes.  It still shares no code with the engine.
"""

from __future__ import annotations

import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu

SHAPES = {
    "1.5b": dict(hidden_size=1536, num_attention_heads=12, num_key_value_heads=2, head_dim=128, intermediate_size=8960,
                 vocab_size=151936, rms_norm_eps=1e-6, tie_word_embeddings=True),
    "7b": dict(hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128, intermediate_size=18944,
               vocab_size=152064, rms_norm_eps=1e-6, tie_word_embeddings=False),
    "14b": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128, intermediate_size=13824,
                vocab_size=152064, rms_norm_eps=1e-5, tie_word_embeddings=False),
}
LENGTHS = [300, 150, 70]
PAGE = 16
MODES = {"whole": helpers.schedule_whole, "tail": helpers.schedule_tail, "portions": helpers.schedule_portions,
         "mixed": lambda requests: helpers.schedule_mixed(requests, seed=5, refeed=1, sizes=(2, 9, 40, 130))}


def wide_weights(cfg: dict, seed: int) -> dict:
    """Random weights on the GPU, already rounded to bfloat16 values so that both engines and the plain
    implementation see the same numbers.  Matrices N(0, 1.7 / sqrt(fan_in)): activations stay of order one
    through the layers and the logits reach a scale at which a wrong key shows."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    hidden, inter, vocab = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

    def mat(rows, cols, gain=1.7):
        return (torch.randn(rows, cols, generator=g, device="cuda") * (gain / cols**0.5)).to(torch.bfloat16).float()

    def vec(n, std):
        return (torch.randn(n, generator=g, device="cuda") * std).to(torch.bfloat16).float()

    w = {"model.embed_tokens.weight": (torch.randn(vocab, hidden, generator=g, device="cuda")).to(torch.bfloat16).float()}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        for name, rows in (("q", nq * d), ("k", nkv * d), ("v", nkv * d)):
            w[p + f"self_attn.{name}_proj.weight"] = mat(rows, hidden)
            w[p + f"self_attn.{name}_proj.bias"] = vec(rows, 0.3)
        w[p + "self_attn.o_proj.weight"] = mat(hidden, nq * d)
        w[p + "mlp.gate_proj.weight"] = mat(inter, hidden)
        w[p + "mlp.up_proj.weight"] = mat(inter, hidden)
        w[p + "mlp.down_proj.weight"] = mat(hidden, inter)
        w[p + "input_layernorm.weight"] = 1 + vec(hidden, 0.05)
        w[p + "post_attention_layernorm.weight"] = 1 + vec(hidden, 0.05)
    w["model.norm.weight"] = 1 + vec(hidden, 0.05)
    if not cfg["tie_word_embeddings"]:
        w["lm_head.weight"] = mat(vocab, hidden, gain=3.0)
    return w


@pytest.fixture(scope="module", params=list(SHAPES))
def wide(request):
    cfg = {"architectures": ["Qwen2ForCausalLM"], "num_hidden_layers": 2, "rope_theta": 1000000.0,
           "max_position_embeddings": 4096, **SHAPES[request.param]}
    weights = wide_weights(cfg, seed=len(request.param))
    requests = {f"r{i}": helpers.random_ids(cfg["vocab_size"], n, 900 + i) for i, n in enumerate(LENGTHS)}
    with torch.inference_mode():
        expected = {rid: plain.forward_logits(ids, weights, cfg).cpu() for rid, ids in requests.items()}
        budget = helpers.Bf16Budget(requests, weights, cfg, {r: e.cuda() for r, e in expected.items()})
    yield {"name": request.param, "cfg": cfg, "weights": weights, "requests": requests, "expected": expected, "budget": budget}
    del weights
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_cutting_at_real_widths(wide, dtype):
    from distie_b200.config import EngineConfig, get_architecture
    from distie_b200.engine.engine import Engine
    from distie_b200.engine.trace_replay import TraceSession
    from distie_b200.kernels import make_kernels

    cfg, requests, expected = wide["cfg"], wide["requests"], wide["expected"]
    arch = get_architecture("Qwen2ForCausalLM")
    tokens = sum(-(-n // 64) * 64 for n in LENGTHS)
    config = EngineConfig(num_blocks=tokens // PAGE, page_size=PAGE, max_seqs=4, token_budget=512, max_model_len=512,
                          dtype=dtype, device="cuda:0")
    kernels = make_kernels(torch.float32 if dtype == "float32" else torch.bfloat16, "cuda:0")
    engine = Engine.assemble(arch, arch.config_cls.from_dict(cfg), wide["weights"], kernels, config)
    assert max(plain.logit_scale(e) for e in expected.values()) > 5, "logits too flat to show a fault"
    for mode, schedule in MODES.items():
        steps = schedule(requests)
        got = helpers.collect(steps, helpers.run_schedule(TraceSession(engine), steps))
        expected_here = helpers.expected_for(got, expected)
        if dtype == "float32":
            error, rid, at = helpers.worst_error(got, expected_here)
            assert error <= helpers.FP32_TOL, f"{wide['name']} {mode}: request {rid} position {at} off by {error:.2e} of the logit scale"
        else:
            wide["budget"].check(got, expected_here, f"{wide['name']} {mode}")
        assert engine.cache.free_pages() == engine.cache.total_pages()
    assert engine.runner.graph_replays > 0
    if dtype == "bfloat16":
        ran = {name for name, count in kernels.kernel_counts.items() if count}
        assert {"attention_prefill_tcgen05", "attention_decode_mma", "gemm_tcgen05", "gemm_tcgen05_skinny"} <= ran, sorted(ran)
    del engine
    torch.cuda.empty_cache()
