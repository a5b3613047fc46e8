"""The plain implementation itself: anchored in the reference's own model code, and self-consistent."""

from __future__ import annotations

import os

import pytest
import torch

import helpers
import plain_qwen2 as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_logits.pt")


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_reference_model_logits(name):
    """``golden/make_golden.py`` ran the reference's Qwen2CausalLM on these ids with these weights."""
    golden = torch.load(GOLDEN)[name]
    cfg, _, weights = helpers.tiny(name)
    logits = plain.forward_logits(golden["ids"], weights, cfg)
    scale = plain.logit_scale(golden["dense"])
    assert float((logits - golden["dense"]).abs().max()) <= 2e-5 * scale
    assert float((logits[-1] - golden["paged_last"]).abs().max()) <= 2e-5 * scale
    assert torch.equal(logits.argmax(-1), golden["dense"].argmax(-1))


def test_prefix_property():
    """Causality: logits of a prefix do not change when tokens are appended."""
    cfg, _, weights = helpers.tiny("B")
    ids = helpers.random_ids(cfg["vocab_size"], 30, 4)
    full = plain.forward_logits(ids, weights, cfg)
    part = plain.forward_logits(ids[:17], weights, cfg)
    assert float((full[:17] - part).abs().max()) <= 1e-5 * plain.logit_scale(full)


def test_rotate_half_pairs():
    x = torch.arange(8.0).view(1, 1, 8)
    assert plain.rotate_half(x).flatten().tolist() == [-4, -5, -6, -7, 0, 1, 2, 3]
    cos, sin = plain.rope_tables(torch.tensor([0]), 8, 10000.0)
    assert torch.equal(plain.apply_rope(x.view(1, 1, 8), cos, sin), x)  # position 0 rotates nothing


def test_rms_norm_formula():
    x = torch.tensor([[3.0, 4.0]])
    out = plain.rms_norm(x, torch.tensor([2.0, 0.5]), 0.0)
    rms = (12.5) ** 0.5
    assert torch.allclose(out, torch.tensor([[2 * 3 / rms, 0.5 * 4 / rms]]))


def test_window_mask_and_grouping():
    mask = plain.visible_mask(5, window=2)
    assert mask.int().tolist() == [[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [0, 1, 1, 0, 0], [0, 0, 1, 1, 0], [0, 0, 0, 1, 1]]
    q = torch.randn(4, 4, 8)
    k = torch.randn(4, 2, 8)
    v = torch.randn(4, 2, 8)
    out = plain.attention_mix(q, k, v)
    alone = plain.attention_mix(q[:, 2:3], k[:, 1:2], v[:, 1:2])  # head 2 reads kv head 1
    assert torch.allclose(out[:, 2:3], alone, atol=1e-6)


def test_greedy_stops_at_eos():
    cfg, _, weights = helpers.tiny("A")
    prompt = helpers.random_ids(cfg["vocab_size"], 6, 2)
    free = plain.greedy_generate(prompt, weights, cfg, 6)
    stopped = plain.greedy_generate(prompt, weights, cfg, 6, eos_id=free[2])
    assert stopped == free[: free.index(free[2]) + 1]
