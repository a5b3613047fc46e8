"""The engine's bookkeeping (cache, batching, scheduling, replay) on the CPU.

The CUDA kernels are replaced by their plain tensor-op references
(``ref_kernels.RefKernels``), everything else is the product's code, and the
results are compared with the plain whole-sequence implementation.  What these
tests catch is a fault of the cache or of the batch, not of a kernel.
"""

from __future__ import annotations

import pytest
import torch

import helpers
import plain_qwen2 as plain
from ref_kernels import RefKernels

from distie_b200.config import EngineConfig, get_architecture
from distie_b200.engine.engine import Engine
from distie_b200.engine.trace_replay import TraceSession


def cpu_engine(name: str, num_blocks: int, max_seqs: int = 8, **knobs) -> tuple[Engine, dict, dict]:
    cfg, page, weights = helpers.tiny(name)
    arch = get_architecture(cfg["architectures"][0])
    config = EngineConfig(
        num_blocks=num_blocks, page_size=page, max_seqs=max_seqs, dtype="float32", decode_graphs=False, device="cpu",
        **{"token_budget": 4096, **knobs},
    )
    engine = Engine.assemble(arch, arch.config_cls.from_dict(cfg), weights, RefKernels(torch.float32), config)
    return engine, cfg, weights


def requests_for(cfg, lengths, seed=10):
    return {f"r{i}": helpers.random_ids(cfg["vocab_size"], n, seed + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_replay_modes_match_plain(name, mode):
    cfg, page, weights = helpers.tiny(name)
    requests = requests_for(cfg, [40, 67, 33, 90, 50, 36])
    steps = {
        "whole": helpers.schedule_whole,
        "tail": helpers.schedule_tail,
        "portions": helpers.schedule_portions,
        "mixed": helpers.schedule_mixed,
    }[mode](requests)
    peak = helpers.peak_tokens(steps)
    engine, _, _ = cpu_engine(name, num_blocks=peak // page)
    session = TraceSession(engine)
    got = helpers.collect(steps, helpers.run_schedule(session, steps))
    expected = {rid: plain.forward_logits(ids, weights, cfg) for rid, ids in requests.items()}
    error, rid, at = helpers.worst_error(got, expected)
    assert error <= helpers.FP32_TOL, f"{mode}: request {rid} position {at} off by {error:.2e} of the logit scale"
    assert engine.cache.free_pages() == engine.cache.total_pages(), "pages were lost"
    assert engine.cache.free_seats == engine.cache.max_seats


def test_mixed_schedule_reuses_pages():
    cfg, page, _ = helpers.tiny("A")
    requests = requests_for(cfg, [40, 67, 33, 90, 50, 36])
    steps = helpers.schedule_mixed(requests)
    peak = helpers.peak_tokens(steps)
    total = sum(-(-len(v) // 64) * 64 for v in requests.values())
    assert peak < total, "the schedule must need fewer pages than all requests together"
    assert max(len(s["entries"]) for s in steps) >= 3
    assert any(len(e["tokens"]) == 1 for s in steps for e in s["entries"])
    assert any(len(e["tokens"]) > 1 for s in steps for e in s["entries"] if len(s["entries"]) > 1)


def test_generate_matches_plain_and_sequential():
    engine, cfg, weights = cpu_engine("B", num_blocks=64, max_seqs=4)
    prompts = [helpers.random_ids(cfg["vocab_size"], n, 50 + n) for n in (1, 5, 17, 40)]
    together = [r.token_ids for r in engine.generate(prompts, max_new_tokens=6)]
    assert together == [plain.greedy_generate(p, weights, cfg, 6) for p in prompts]
    alone = [engine.generate(p, max_new_tokens=6)[0].token_ids for p in prompts]
    assert alone == together
    assert engine.cache.free_pages() == engine.cache.total_pages()


def test_chunked_prefill_and_preemption_keep_outputs():
    # A pool so small that decoding runs out of pages: the newest request is preempted and recomputed.
    engine, cfg, weights = cpu_engine("B", num_blocks=14, max_seqs=4, token_budget=24, prefill_chunk=11)
    prompts = [helpers.random_ids(cfg["vocab_size"], n, 70 + n) for n in (17, 40, 23)]
    results = engine.generate(prompts, max_new_tokens=12)
    assert [r.token_ids for r in results] == [plain.greedy_generate(p, weights, cfg, 12) for p in prompts]
    assert sum(r.preemptions for r in results) >= 1, "the pool was meant to be too small"
    assert engine.cache.free_pages() == engine.cache.total_pages()


def test_temperature_sampling_is_reproducible_and_batch_independent():
    engine, cfg, _ = cpu_engine("A", num_blocks=64, max_seqs=4)
    prompts = [helpers.random_ids(cfg["vocab_size"], n, 90 + n) for n in (9, 21, 14)]
    first = [r.token_ids for r in engine.generate(prompts, max_new_tokens=8, temperature=0.8, seed=1)]
    again = [r.token_ids for r in engine.generate(prompts, max_new_tokens=8, temperature=0.8, seed=1)]
    assert first == again
    alone = engine.generate(prompts[1], max_new_tokens=8, temperature=0.8, seed=2)[0].token_ids
    assert alone == first[1], "request 1 has seed 1 + 1 in the batch: alone with seed 2 it must repeat itself"
    other = [r.token_ids for r in engine.generate(prompts, max_new_tokens=8, temperature=0.8, seed=5)]
    assert other != first


def test_trace_free_running_and_forced():
    engine, cfg, weights = cpu_engine("A", num_blocks=32)
    prompt = helpers.random_ids(cfg["vocab_size"], 12, 5)
    free = engine.trace(prompt, 5)
    assert free.token_ids == plain.greedy_generate(prompt, weights, cfg, 5)
    forced_ids = [3, 1, 4, 1, 5]
    forced = engine.trace(prompt, 5, forced_ids)
    want = plain.forward_logits(prompt + forced_ids[:-1], weights, cfg)[len(prompt) - 1 :]
    assert float((forced.logits - want).abs().max()) <= helpers.FP32_TOL * plain.logit_scale(want)
    with pytest.raises(ValueError):
        engine.trace([], 3)
    with pytest.raises(ValueError):
        engine.trace(prompt, 3, [1])
    assert engine.cache.free_pages() == engine.cache.total_pages()


@pytest.mark.parametrize("layer,which", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_corrupted_cache_is_detected(layer, which):
    """The comparison can fail: ONE page of ONE layer's keys (or values) overwritten between steps changes
    the logits that follow, whichever layer and whichever of the two it is."""
    engine, cfg, weights = cpu_engine("A", num_blocks=16)
    ids = helpers.random_ids(cfg["vocab_size"], 40, 3)
    session = TraceSession(engine)
    session.run_step([{"id": "x", "tokens": ids[:30], "want": []}])
    page = engine.cache.pages_held(session.live["x"][0])[0][0]
    engine.cache.groups[0].slab[layer, which, page] += 1.0
    got = session.run_step([{"id": "x", "tokens": ids[30:], "want": list(range(10))}], ["x"])
    want = plain.forward_logits(ids, weights, cfg)[30:]
    assert float((torch.as_tensor(got) - want).abs().max()) > 100 * helpers.FP32_TOL * plain.logit_scale(want)


@pytest.mark.parametrize("mode", ["whole", "portions", "mixed"])
def test_run_order_is_data(mode):
    """A layer run twice, a layer that reads another layer's keys and values, windows on some layers only:
    the model is built from the same parts by a different list, and every way of cutting still matches."""
    from distie_b200.engine.engine import build_cache
    from distie_b200.engine.runner import ModelRunner
    from distie_b200.models.decoder import DecoderModel, model_tensor_specs
    from distie_b200.weights import open_weights

    cfg, page, weights = helpers.tiny("B")
    spec = helpers.toy_arrangement_spec(cfg)
    requests = requests_for(cfg, [40, 67, 33, 90, 50, 36], seed=40)
    steps = {"whole": helpers.schedule_whole, "portions": helpers.schedule_portions, "mixed": helpers.schedule_mixed}[mode](requests)
    kernels = RefKernels(torch.float32)
    config = EngineConfig(num_blocks=helpers.peak_tokens(steps) // page, page_size=page, max_seqs=8, dtype="float32",
                          decode_graphs=False, device="cpu", token_budget=4096)
    store = open_weights(weights, model_tensor_specs(spec), spec.tolerated, kernels.dtype, kernels.device)
    model = DecoderModel(spec, kernels, store)
    cache = build_cache(spec, config, kernels.dtype, kernels.device)
    assert len(cache.groups) == 2, "full and windowed layers keep pages of their own"
    engine = Engine(model, cache, config)
    got = helpers.collect(steps, helpers.run_schedule(TraceSession(engine), steps))
    expected = {rid: plain.forward_logits(ids, weights, cfg, order=helpers.TOY_ORDER) for rid, ids in requests.items()}
    error, rid, at = helpers.worst_error(got, expected)
    assert error <= helpers.FP32_TOL, f"{mode}: request {rid} position {at} off by {error:.2e} of the logit scale"
    assert cache.free_pages() == cache.total_pages() and cache.free_seats == cache.max_seats


def test_a_refused_request_leaves_nothing_behind():
    """A batch whose second request can never fit is refused as a whole: nothing waits in the scheduler
    for the next call to pick up, and no page or seat is held."""
    from distie_b200.cache import CacheExhausted
    from distie_b200.engine.engine import GenerateRequest

    engine, cfg, weights = cpu_engine("A", num_blocks=8, max_seqs=4)  # 128 tokens of cache
    fits = helpers.random_ids(cfg["vocab_size"], 9, 1)
    never = helpers.random_ids(cfg["vocab_size"], 200, 2)
    with pytest.raises(CacheExhausted, match="can never fit"):
        engine.run([GenerateRequest("a", fits, 4), GenerateRequest("b", never, 4), GenerateRequest("c", fits, 4)])
    assert not engine.scheduler.has_work() and not engine.has_work()
    assert engine.cache.free_pages() == engine.cache.total_pages() and engine.cache.free_seats == engine.cache.max_seats
    with pytest.raises(ValueError, match="duplicate"):
        engine.run([GenerateRequest("a", fits, 4), GenerateRequest("a", fits, 4)])
    assert not engine.scheduler.has_work()
    steps_before = engine.steps
    out = engine.run([GenerateRequest("a", fits, 4)])
    assert out[0].token_ids == plain.greedy_generate(fits, weights, cfg, 4)
    assert engine.steps - steps_before == 4, "only the one request ran: nothing was left over from the refused batch"


def kv_rows(engine, seat: int, tokens: int) -> dict:
    """The keys and values a request holds, gathered through its block table: {slot: (k, v) [tokens, heads, dim]}."""
    cache = engine.cache
    out = {}
    for group, ids in zip(cache.groups, cache.pages_held(seat).values()):
        pages = torch.tensor(ids, dtype=torch.long, device=group.slab.device)
        for index, slot in enumerate(group.slots):
            k, v = (group.slab[index, which].index_select(0, pages) for which in (0, 1))  # [pages, heads, page, dim]
            out[slot] = tuple(t.permute(0, 2, 1, 3).reshape(-1, t.shape[1], t.shape[3])[:tokens].float().cpu() for t in (k, v))
    return out


@pytest.mark.parametrize("name", ["A", "B"])
def test_two_slabs_hold_equal_keys_and_values(name):
    """The same requests cut two ways (whole, and in portions mixed with single tokens) leave the same keys
    and values in their pages, not only the same logits (the reference's two-slab comparison,
    worker/tests/test_qwen2_batch.py:71-109)."""
    cfg, page, _ = helpers.tiny(name)
    requests = requests_for(cfg, [40, 67, 33, 50])
    slabs = []
    for schedule in (helpers.schedule_whole, helpers.schedule_mixed):
        steps = [dict(step, end=[]) for step in schedule(requests)]  # nobody ends: the pages stay held
        engine, _, _ = cpu_engine(name, num_blocks=4 * 128 // page)
        session = TraceSession(engine)
        helpers.run_schedule(session, steps)
        slabs.append({rid: kv_rows(engine, session.live[rid][0], len(ids)) for rid, ids in requests.items()})
    for rid in requests:
        for slot, (k, v) in slabs[0][rid].items():
            k2, v2 = slabs[1][rid][slot]
            for a, b in ((k, k2), (v, v2)):  # 1e-5 of the largest entry: the sums run in another order, nothing more
                assert float(a.abs().max()) > 0
                assert float((a - b).abs().max()) <= 1e-5 * max(1.0, float(a.abs().max())), (rid, slot)


def test_second_tiny_workload_against_the_sampling_oracle():
    """Prompts of 1/5/17/40/63 tokens in portions of 11 beside decoding requests, temperature 0.8 from
    seed 1, 24 tokens each, one forced preemption: every token is the oracle's inverse-CDF pick."""
    engine, cfg, weights = cpu_engine("B", num_blocks=64, max_seqs=8, token_budget=24, prefill_chunk=helpers.TINY_B_CHUNK)
    prompts, results = helpers.run_tiny_b_workload(engine, cfg)
    assert results[4].preemptions == 1 and all(len(r.token_ids) == helpers.TINY_B_STEPS for r in results)
    for index, (prompt, result) in enumerate(zip(prompts, results)):
        helpers.check_sampled_tokens(prompt, result.token_ids, weights, cfg, helpers.TINY_B_TEMPERATURE, helpers.TINY_B_SEED + index)
    assert engine.cache.free_pages() == engine.cache.total_pages()


def test_step_statistics_split_and_line():
    from distie_b200.engine.step_stats import StepStats

    stats = StepStats(every=3)
    stats.record("prefill", 2, 40, 3.0, sched=0.5, gpu=4.0, emit=0.5)
    stats.record("decode", 4, 4, None, sched=0.25, gpu=1.0, emit=0.25)
    assert stats.lines == []
    stats.record("decode", 2, 2, 0.5, sched=0.25, gpu=1.5, emit=0.25)
    assert len(stats.lines) == 1 and stats.flush() is None, "the third step closed the window"
    line, numbers = stats.lines[0], stats.summaries[0]
    assert line.startswith("step stats steps=3 | decode n=2 rows=3.0 tok=3 ms/step[sched=0.25 gpu=1.25 emit=0.25 (kernel=0.50 host=1.00)]")
    assert "prefill n=1 rows=2.0 tok=40 ms/step[sched=0.50 gpu=4.00 emit=0.50 (kernel=3.00 host=1.00)] share=59%" in line
    assert line.endswith("wall sched=12% gpu=76% emit=12%")
    assert numbers["kinds"]["decode"]["n"] == 2 and abs(numbers["wall"]["gpu"] - 6.5 / 8.5) < 1e-9
    with pytest.raises(ValueError):
        StepStats(0)
    engine, cfg, _ = cpu_engine("A", num_blocks=32, max_seqs=4, step_stats=4)
    engine.generate([helpers.random_ids(cfg["vocab_size"], n, n) for n in (5, 9)], max_new_tokens=6)
    assert engine.stats.lines and "decode n=" in " ".join(engine.stats.lines)
    assert sum(s["steps"] for s in engine.stats.summaries) == engine.steps


def test_constants_around_the_stack_and_a_position_encoding_of_its_own():
    """What another architecture may need of the model builder, set from outside the package: a scale on
    the embedded tokens, a scale and a soft cap on the logits, a factor on the rotation's cos and sin, and
    a position encoding that is no table of frequencies at all (it offers ``apply`` and the mixer calls it)."""
    from dataclasses import replace

    from distie_b200.config import PartSpec
    from distie_b200.engine.engine import build_cache
    from distie_b200.models.decoder import DecoderModel, model_tensor_specs
    from distie_b200.parts import POSITION_ENCODINGS
    from distie_b200.weights import open_weights

    cfg, page, weights = helpers.tiny("A")
    hidden, heads, kv_heads, d = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    arch = get_architecture(cfg["architectures"][0])
    spec = arch.recipe(arch.config_cls.from_dict(cfg))

    def angles(positions):  # a rotation whose angle is no multiple of the position: not a table of frequencies
        inv = plain.rope_inverse_frequencies(d, 10000.0)
        return torch.sqrt(positions.float() + 1.0)[:, None] * inv[None, :]

    class RootRotation:
        applied = 0

        @classmethod
        def build(cls, part, ctx):
            return cls()

        def rotary_table(self):
            return None

        def apply(self, qkv, step, num_heads, num_kv_heads, head_dim):
            RootRotation.applied += 1
            a = angles(step.positions[: step.num_tokens])
            cos, sin = torch.cat((a, a), -1).cos(), torch.cat((a, a), -1).sin()
            rot = qkv[:, : (num_heads + num_kv_heads) * head_dim].reshape(step.num_tokens, num_heads + num_kv_heads, head_dim)
            rot.copy_(plain.apply_rope(rot.float(), cos, sin).to(qkv.dtype))

    def build(layers_position, **around):
        layers = tuple(
            replace(layer, mixer=PartSpec(layer.mixer.kind, {**layer.mixer.params, "position": layers_position}, layer.mixer.prefix))
            for layer in spec.layers
        )
        changed = replace(spec, layers=layers, **around)
        kernels = RefKernels(torch.float32)
        config = EngineConfig(num_blocks=8, page_size=page, max_seqs=2, dtype="float32", decode_graphs=False, device="cpu")
        store = open_weights(weights, model_tensor_specs(changed), changed.tolerated, kernels.dtype, kernels.device)
        return Engine(DecoderModel(changed, kernels, store), build_cache(changed, config, kernels.dtype, kernels.device), config)

    def plain_logits(ids, rope, embedding_scale=1.0, logit_scale=1.0, softcap=None):
        """The plain implementation's parts, put together with another rotation and the constants around the stack."""
        positions = torch.arange(len(ids))
        h = plain.embedding(torch.tensor(ids), weights["model.embed_tokens.weight"]) * embedding_scale
        for layer in range(cfg["num_hidden_layers"]):
            p = f"model.layers.{layer}."
            x = plain.rms_norm(h, weights[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
            q, k, v = (torch.nn.functional.linear(x, weights[p + f"self_attn.{n}_proj.weight"], weights[p + f"self_attn.{n}_proj.bias"])
                       for n in "qkv")
            cos, sin = rope(positions)
            q = plain.apply_rope(q.view(-1, heads, d), cos, sin)
            k = plain.apply_rope(k.view(-1, kv_heads, d), cos, sin)
            mixed = plain.attention_mix(q, k, v.view(-1, kv_heads, d))
            h = h + torch.nn.functional.linear(mixed.reshape(-1, heads * d), weights[p + "self_attn.o_proj.weight"])
            h = h + plain.swiglu_mlp(plain.rms_norm(h, weights[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"]), weights, p + "mlp.")
        logits = plain.output_head(h, weights, cfg).float() * logit_scale
        return softcap * torch.tanh(logits / softcap) if softcap else logits

    ids = helpers.random_ids(cfg["vocab_size"], 37, 8)

    def engine_logits(engine):
        session = TraceSession(engine)
        first = session.run_step([{"id": "x", "tokens": ids[:20], "want": list(range(20))}])
        rest = [session.run_step([{"id": "x", "tokens": [t], "want": [0]}]) for t in ids[20:]]
        return torch.cat([torch.as_tensor(first)] + [torch.as_tensor(r) for r in rest])

    # 1. constants around the stack and a factor on cos and sin
    factor = 1.3
    scaled = build(PartSpec("rotary", {"head_dim": d, "theta": cfg["rope_theta"], "factor": factor}),
                   embedding_scale=hidden**0.5, logit_scale=0.25, logit_softcap=30.0)

    def scaled_rope(positions):
        cos, sin = plain.rope_tables(positions, d, cfg["rope_theta"])
        return cos * factor, sin * factor

    want = plain_logits(ids, scaled_rope, hidden**0.5, 0.25, 30.0)
    assert float((engine_logits(scaled) - want).abs().max()) <= helpers.FP32_TOL * plain.logit_scale(want)
    assert float(want.abs().max()) <= 30.0

    # 2. a position encoding with an ``apply`` of its own
    POSITION_ENCODINGS.register("test_root_rotation", RootRotation)
    try:
        own = build(PartSpec("test_root_rotation", {}))

        def root_rope(positions):
            a = angles(positions)
            return torch.cat((a, a), -1).cos(), torch.cat((a, a), -1).sin()

        want = plain_logits(ids, root_rope)
        assert float((engine_logits(own) - want).abs().max()) <= helpers.FP32_TOL * plain.logit_scale(want)
        assert RootRotation.applied > 0
        differs = plain.forward_logits(ids, weights, cfg)
        assert float((differs - want).abs().max()) > 100 * helpers.FP32_TOL * plain.logit_scale(want), "the rotation must matter"
    finally:
        POSITION_ENCODINGS.unregister("test_root_rotation")
