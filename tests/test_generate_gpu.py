"""Generation through the Python entry point on the GPU, the parts alone, and a toy mixer."""

from __future__ import annotations

import pytest
import torch

import helpers
import plain_qwen2 as plain

pytestmark = pytest.mark.gpu


def folder_for(name, tmp_path_factory, dtype="bfloat16"):
    from distie_b200.weights import ModelTensors, write_random_model

    cfg, page, _ = helpers.tiny(name)
    folder = str(tmp_path_factory.mktemp(f"gen{name}"))
    write_random_model(folder, cfg, seed=helpers.TINY[name][2], std=helpers.STD[name], norm_noise=helpers.TINY[name][3], dtype=dtype)
    stored = ModelTensors(folder)
    return folder, cfg, page, {n: stored.tensor(n).float() for n in stored.keys()}


@pytest.fixture(scope="module", params=["A", "B", "D"])
def tiny_model(request, tmp_path_factory):
    return folder_for(request.param, tmp_path_factory)


@pytest.mark.parametrize("graphs", [True, False])
def test_greedy_generation_float32(tiny_model, graphs):
    from distie_b200.engine.engine import Engine

    folder, cfg, page, weights = tiny_model
    engine = Engine.load(folder, dtype="float32", num_blocks=64, page_size=page, max_seqs=4, decode_graphs=graphs)
    prompts = [helpers.random_ids(cfg["vocab_size"], n, 30 + n) for n in (7, 13, 29)]
    results = engine.generate(prompts, max_new_tokens=16)
    assert [r.token_ids for r in results] == [plain.greedy_generate(p, weights, cfg, 16) for p in prompts]
    assert all(r.finish_reason == "length" and r.completion_tokens == 16 for r in results)
    if graphs:
        assert engine.runner.graph_replays > 0, "pure-decode steps were meant to replay graphs"
    assert engine.cache.free_pages() == engine.cache.total_pages()


@pytest.mark.parametrize("temperature", [0.0, 0.9])
def test_decoding_a_step_ahead_changes_nothing(tiny_model, temperature):
    """Steps launched before the tokens of the step ahead are known: same tokens, same ends, an end by EOS
    in the middle included (the request's row in the step already launched is dropped)."""
    from distie_b200.engine.engine import Engine

    folder, cfg, page, _ = tiny_model
    prompts = [helpers.random_ids(cfg["vocab_size"], n, 70 + n) for n in (3, 9, 20, 6)]
    outcomes = {}
    for ahead in (False, True):
        engine = Engine.load(folder, dtype="float32", num_blocks=64, page_size=page, max_seqs=4, decode_ahead=ahead)
        free = engine.generate(prompts, max_new_tokens=24, temperature=temperature, seed=5, ignore_eos=True)
        # Make the token that request 1 produces as its 8th output the end-of-sequence id: it ends there, the
        # others wherever they meet that id or at their length.
        eos = free[1].token_ids[7]
        stopped = engine.generate(prompts, max_new_tokens=24, temperature=temperature, seed=5, eos_id=eos)
        outcomes[ahead] = [(r.token_ids, r.finish_reason) for r in free + stopped]
        assert stopped[1].finish_reason == "eos" and len(stopped[1].token_ids) <= 8
        assert engine.cache.free_pages() == engine.cache.total_pages()
        if ahead:
            assert engine.runner.graph_replays > 0
    assert outcomes[True] == outcomes[False]


def test_first_tokens_of_a_sequence(tiny_model):
    """Positions 0, 1, 2: a one-token prompt and the tokens right after it."""
    from distie_b200.engine.engine import Engine

    folder, cfg, page, weights = tiny_model
    starts = {f"s{i}": helpers.random_ids(cfg["vocab_size"], 5, 200 + i) for i in range(16)}
    want = {rid: plain.forward_logits(ids[:4], weights, cfg) for rid, ids in starts.items()}
    budget = helpers.Bf16Budget({rid: ids[:4] for rid, ids in starts.items()}, weights, cfg, want)
    for dtype in ("float32", "bfloat16"):
        engine = Engine.load(folder, dtype=dtype, num_blocks=16, page_size=page, max_seqs=2, decode_graphs=False)
        got = {rid: engine.trace(ids[:1], 4, ids[1:]).logits for rid, ids in starts.items()}
        if dtype == "float32":
            assert helpers.worst_error(got, want)[0] <= helpers.FP32_TOL
        else:
            budget.check(got, want, "first tokens")


def test_long_decoding_bfloat16_and_float32(tiny_model):
    """Several hundred decode steps after a short prompt, teacher-forced so that logits stay comparable."""
    from distie_b200.engine.engine import Engine

    folder, cfg, page, weights = tiny_model
    ids = helpers.random_ids(cfg["vocab_size"], 420, 77)
    full = plain.forward_logits(ids, weights, cfg)
    budget = helpers.Bf16Budget({"x": ids}, weights, cfg, {"x": full}, skip=7)
    want = {"x": full[7:]}
    for dtype in ("float32", "bfloat16"):
        engine = Engine.load(folder, dtype=dtype, num_blocks=64, page_size=page, max_seqs=2, decode_graphs=False)
        trace = engine.trace(ids[:8], len(ids) - 8 + 1, ids[8:] + [0])
        got = {"x": trace.logits[: want["x"].shape[0]]}
        if dtype == "float32":
            assert helpers.worst_error(got, want)[0] <= helpers.FP32_TOL
        else:
            budget.check(got, want, "long decoding")


@pytest.mark.parametrize("name", ["C", "D"])
def test_the_merged_decode_attention_changes_no_logit(name, tmp_path_factory, monkeypatch):
    """Steps of single tokens with the attention kernel that starts from the projection, against the same steps
    with the projection, the rotation kernel and the attention one after the other: the sums, the rotation and
    the rounding are the same operations in the same order, so the logits must agree bit for bit (and the
    kernels that ran must differ)."""
    from distie_b200.engine.engine import Engine
    from distie_b200.kernels.device import DeviceKernels
    from distie_b200.kernels.interface import KernelSet

    folder, cfg, page, _ = folder_for(name, tmp_path_factory)
    ids = helpers.random_ids(cfg["vocab_size"], 150, 41)
    logits, counts = {}, {}
    for merged in (True, False):
        if not merged:
            monkeypatch.setattr(DeviceKernels, "qkv_attention", KernelSet.qkv_attention)
        engine = Engine.load(folder, dtype="bfloat16", num_blocks=64, page_size=page, max_seqs=2)
        trace = engine.trace(ids[:70], len(ids) - 70 + 1, ids[70:] + [0])
        logits[merged] = trace.logits
        counts[merged] = dict(engine.model.kernels.kernel_counts)
        assert engine.runner.graph_replays > 0
    assert counts[True].get("attention_decode_mma_qkv", 0) > 0 and counts[False].get("attention_decode_mma_qkv", 0) == 0
    assert counts[False].get("rope_kv_write_split", 0) > counts[True].get("rope_kv_write_split", 0)
    assert torch.equal(logits[True], logits[False]), float((logits[True] - logits[False]).abs().max())


@pytest.mark.parametrize("name", ["C", "D"])
def test_the_merged_projection_epilogue_changes_no_logit(name, tmp_path_factory, monkeypatch):
    """A prompt of 300 tokens with bias, rotation and the cache write in the q/k/v product's epilogue, against the
    product's float32 result handed to the rotation kernel: the same operations on the same float32 sums."""
    from distie_b200.engine.engine import Engine
    from distie_b200.kernels.device import DeviceKernels
    from distie_b200.kernels.interface import KernelSet

    folder, cfg, page, _ = folder_for(name, tmp_path_factory)
    ids = helpers.random_ids(cfg["vocab_size"], 300, 43)
    logits, counts = {}, {}
    for merged in (True, False):
        if not merged:
            monkeypatch.setattr(DeviceKernels, "qkv_rope_write", KernelSet.qkv_rope_write)
        engine = Engine.load(folder, dtype="bfloat16", num_blocks=64, page_size=page, max_seqs=2)
        trace = engine.trace(ids, 4, [1, 2, 3, 4])
        logits[merged] = trace.logits
        counts[merged] = dict(engine.model.kernels.kernel_counts)
    assert counts[True].get("gemm_tcgen05_qkv", 0) > 0 and counts[False].get("gemm_tcgen05_qkv", 0) == 0
    assert torch.equal(logits[True], logits[False]), float((logits[True] - logits[False]).abs().max())


def test_preemption_and_chunked_prefill_on_gpu(tmp_path_factory):
    """tiny-B, prompts 1/5/17/40/63, portions of 11 beside decoding, a pool that forces preemption."""
    from distie_b200.engine.engine import Engine

    folder, cfg, page, weights = folder_for("B", tmp_path_factory)
    engine = Engine.load(
        folder, dtype="float32", num_blocks=24, page_size=page, max_seqs=5, token_budget=32, prefill_chunk=11, decode_graphs=True
    )
    prompts = [helpers.random_ids(cfg["vocab_size"], n, 90 + n) for n in (1, 5, 17, 40, 63)]
    results = engine.generate(prompts, max_new_tokens=24)
    assert [r.token_ids for r in results] == [plain.greedy_generate(p, weights, cfg, 24) for p in prompts]
    assert sum(r.preemptions for r in results) >= 1
    sampled = engine.generate(prompts, max_new_tokens=24, temperature=0.8, seed=1)
    again = engine.generate(prompts, max_new_tokens=24, temperature=0.8, seed=1)
    assert [r.token_ids for r in sampled] == [r.token_ids for r in again]
    assert engine.cache.free_pages() == engine.cache.total_pages()


def test_preemption_and_portions_in_bfloat16_at_the_tensor_core_configuration(tmp_path_factory):
    """Configuration D in bfloat16 through the scheduler: prompts of 3 to 300 tokens in portions of 150 beside
    decoding requests, so few pages that requests are sent back and recomputed.  Every produced token must be the
    plain arg-max of its position or a near tie of it (bfloat16 may turn a near tie), and a second run must give
    the same tokens."""
    from distie_b200.engine.engine import Engine

    folder, cfg, page, weights = folder_for("D", tmp_path_factory)
    engine = Engine.load(folder, dtype="bfloat16", num_blocks=16, page_size=page, max_seqs=5, token_budget=256,
                         prefill_chunk=150, decode_graphs=True)
    prompts = [helpers.random_ids(cfg["vocab_size"], n, 190 + n) for n in (3, 40, 300, 131, 64)]
    results = engine.generate(prompts, max_new_tokens=64, ignore_eos=True)
    assert sum(r.preemptions for r in results) >= 1, "the pool was meant to be too small"
    for prompt, result in zip(prompts, results):
        ids = prompt + result.token_ids[:-1]
        full = plain.forward_logits(ids, weights, cfg)
        budget = helpers.Bf16Budget({"x": ids}, weights, cfg, {"x": full})
        rows = full[len(prompt) - 1 :]
        slack = 3 * budget.max_error * plain.logit_scale(full)
        for step, token in enumerate(result.token_ids):
            short = float(rows[step].max() - rows[step][token])
            assert short <= slack, f"prompt of {len(prompt)}: output {step} is {short:.3f} below the plain maximum (slack {slack:.3f})"
    again = engine.generate(prompts, max_new_tokens=64, ignore_eos=True)
    assert [r.token_ids for r in again] == [r.token_ids for r in results]
    ran = {name for name, count in engine.model.kernels.kernel_counts.items() if count}
    assert {"attention_decode_mma_qkv", "gemm_tcgen05_qkv", "attention_prefill_tcgen05"} <= ran, sorted(ran)
    assert engine.cache.free_pages() == engine.cache.total_pages()


def test_second_tiny_workload_against_the_sampling_oracle(tmp_path_factory):
    """The workload of the second tiny configuration with an oracle: prompts of 1/5/17/40/63 tokens in
    portions of 11 beside decoding requests, temperature 0.8 from seed 1, 24 tokens each, one forced
    preemption; decode graphs and a step ahead on.  Every token must be the inverse-CDF pick of the plain
    implementation's distribution at the request's own uniform number."""
    from distie_b200.engine.engine import Engine

    folder, cfg, page, weights = folder_for("B", tmp_path_factory)
    engine = Engine.load(folder, dtype="float32", num_blocks=64, page_size=page, max_seqs=8, token_budget=24,
                         prefill_chunk=helpers.TINY_B_CHUNK)
    prompts, results = helpers.run_tiny_b_workload(engine, cfg)
    assert results[4].preemptions == 1 and all(len(r.token_ids) == helpers.TINY_B_STEPS for r in results)
    for index, (prompt, result) in enumerate(zip(prompts, results)):
        helpers.check_sampled_tokens(prompt, result.token_ids, weights, cfg, helpers.TINY_B_TEMPERATURE, helpers.TINY_B_SEED + index)
    assert engine.runner.graph_replays > 0
    assert engine.cache.free_pages() == engine.cache.total_pages()


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


@pytest.mark.parametrize("dtype,tol,deeper", [("float32", 1e-5, 1e-5), ("bfloat16", 2.0**-7, 1.6e-2)])
@pytest.mark.parametrize("name", ["B", "D"])
def test_two_slabs_hold_equal_keys_and_values(name, dtype, tol, deeper, tmp_path_factory):
    """The same requests cut three ways (whole; the tail token by token through the captured decode step;
    portions mixed with single tokens) leave the same keys and values in their pages, not only the same
    logits (the reference's two-slab comparison, worker/tests/test_qwen2_batch.py:71-109).  Differences
    are measured against the slab's largest entry.  bfloat16: in the first layer, whose input is the same
    embedding row however the request was cut, a key may differ by one rounding where the product that made
    it ran on another kernel; deeper layers read activations that already carry such roundings, so their
    keys are held to the four roundings the kernel tests allow a bfloat16 result."""
    from distie_b200.engine.trace_replay import TraceSession

    folder, cfg, page, _ = folder_for(name, tmp_path_factory)
    requests = {f"r{i}": helpers.random_ids(cfg["vocab_size"], n, 20 + i) for i, n in enumerate([40, 167, 33, 150])}
    slabs = []
    for schedule in (helpers.schedule_whole, helpers.schedule_tail, helpers.schedule_mixed):
        steps = [dict(step, end=[]) for step in schedule(requests)]  # nobody ends: the pages stay held
        session = TraceSession.open(folder, dtype, 4 * 192, page_size=page)
        helpers.run_schedule(session, steps)
        slabs.append({rid: kv_rows(session.engine, session.live[rid][0], len(ids)) for rid, ids in requests.items()})
    for other in slabs[1:]:
        for rid in requests:
            for slot, pair in slabs[0][rid].items():
                for a, b in zip(pair, other[rid][slot]):
                    assert float(a.abs().max()) > 0
                    worst = float((a - b).abs().max()) / float(a.abs().max())  # of the largest entry
                    assert worst <= (tol if slot == 0 else deeper), (rid, slot, worst)


def test_a_bad_request_does_not_switch_the_graphs_off(tmp_path_factory):
    """A device-side check that fails on one request's data (here: its block table names a page outside the
    pool) raises to the caller; it is not mistaken for a failure of the captured step, so later requests
    still replay graphs."""
    from distie_b200.engine.engine import Engine
    from distie_b200.kernels.library import KernelError

    folder, cfg, page, weights = folder_for("A", tmp_path_factory)
    engine = Engine.load(folder, dtype="float32", num_blocks=32, page_size=page, max_seqs=4, decode_ahead=False)
    prompt = helpers.random_ids(cfg["vocab_size"], 9, 3)
    want = plain.greedy_generate(prompt, weights, cfg, 6)
    assert engine.generate(prompt, max_new_tokens=6)[0].token_ids == want
    replays = engine.runner.graph_replays
    assert replays > 0 and engine.runner.use_graphs
    group = engine.cache.groups[0]
    spoiled = []

    def spoil(request_id, token, finished):
        if not spoiled:  # after the first token: the request's table now names a page the pool does not have
            seat = engine.scheduler.running()[0].seat
            group.device_table[seat, 0] = group.num_pages + 7
            spoiled.append(seat)

    with pytest.raises(KernelError, match="block table"):
        engine.generate(prompt, max_new_tokens=6, on_token=spoil)
    assert engine.runner.use_graphs, "a bad request must not cost every later request its graphs"
    assert engine.cache.free_pages() == engine.cache.total_pages() and not engine.has_work()
    group.device_table[spoiled[0]] = -1
    assert engine.generate(prompt, max_new_tokens=6)[0].token_ids == want
    assert engine.runner.graph_replays > replays


def test_float32_checkpoint_in_the_bfloat16_engine_runs_the_bfloat16_kernels(tmp_path_factory):
    """A checkpoint stored wholly in float32 is cast by the bfloat16 engine, as the reference casts on load
    (worker/src/inference/torch_engine.py:135-141): the tensor-core kernels run and the logits stay within
    the bfloat16 budget.  With ``float32_weights="keep"`` the matrices stay wide and none of them runs."""
    from distie_b200.engine.engine import Engine

    folder, cfg, page, weights = folder_for("D", tmp_path_factory, dtype="float32")
    ids = helpers.random_ids(cfg["vocab_size"], 200, 5)
    rounded = helpers.bf16_rounded(weights)
    want = {"x": plain.forward_logits(ids, rounded, cfg)}
    budget = helpers.Bf16Budget({"x": ids}, rounded, cfg, want)
    engine = Engine.load(folder, dtype="bfloat16", num_blocks=16, page_size=page, max_seqs=2)
    got = {"x": engine.trace(ids[:160], 41, ids[160:] + [0]).logits[:40]}
    budget_want = {"x": want["x"][159:199]}
    worst, rms, top1 = helpers.pooled_stats(got, budget_want)
    assert rms <= 2 * budget.rms_error and top1 >= budget.top1 - 0.05, (worst, rms, top1, budget.rms_error)
    ran = {name for name, count in engine.model.kernels.kernel_counts.items() if count}
    assert {"gemm_tcgen05", "gemm_tcgen05_skinny", "attention_prefill_tcgen05", "attention_decode_mma"} <= ran, sorted(ran)
    del engine
    wide = Engine.load(folder, dtype="bfloat16", num_blocks=16, page_size=page, max_seqs=2, float32_weights="keep")
    wide.trace(ids[:160], 2, ids[160:162])
    ran = {name for name, count in wide.model.kernels.kernel_counts.items() if count}
    assert not ({"gemm_tcgen05", "gemm_tcgen05_skinny"} & ran), sorted(ran)


def test_missing_extension_fails_loudly(monkeypatch):
    from distie_b200.csrc import build
    from distie_b200.kernels import library

    monkeypatch.setattr(library, "_libraries", {})
    monkeypatch.setattr(library, "_functions", {})
    monkeypatch.setattr(build, "build_cuda_unit", lambda name: "/nonexistent/libdistie.so")
    with pytest.raises(library.KernelError):
        library.function("distie_embed")


# -- each part alone ------------------------------------------------------------
def part_context(dtype, tensors, hidden):
    from distie_b200.kernels import make_kernels
    from distie_b200.parts.base import BuildContext
    from distie_b200.weights.loader import DictSource, WeightStore

    kernels = make_kernels(dtype, "cuda:0")
    return BuildContext(kernels, hidden, WeightStore(DictSource(tensors), [], dtype, "cuda:0"))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_feed_forward_part_alone(dtype, tol):
    from distie_b200.config import PartSpec
    from distie_b200.parts import FEED_FORWARDS, build_part

    hidden, inter = 72, 200
    w = {f"ff.{n}_proj.weight": torch.randn(s) * 0.2 for n, s in (("gate", (inter, hidden)), ("up", (inter, hidden)), ("down", (hidden, inter)))}
    w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    part = build_part(FEED_FORWARDS, PartSpec("swiglu", {"intermediate_size": inter}, "ff."), part_context(dtype, w, hidden))
    x = torch.randn(9, hidden).to(torch.bfloat16).float()
    got = part.forward(x.cuda().to(dtype), None).float()
    got = (got.sum(0) if got.dim() == 3 else got).cpu()  # slices of a split product add up to the result
    want = plain.swiglu_mlp(x, {k.replace("ff.", "p."): v for k, v in w.items()}, "p.")
    assert float((got - want).abs().max()) <= tol * float(want.abs().max())


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_norm_part_alone(dtype, tol):
    from distie_b200.config import PartSpec
    from distie_b200.parts import NORMS, build_part

    hidden = 88
    w = {"n.weight": (1 + 0.1 * torch.randn(hidden)).to(torch.bfloat16).float()}
    part = build_part(NORMS, PartSpec("rmsnorm", {"eps": 1e-5}, "n."), part_context(dtype, w, hidden))
    x = torch.randn(5, hidden) * 4
    out = torch.empty(5, hidden, dtype=dtype, device="cuda")
    part.apply(None, x.cuda(), out)
    want = plain.rms_norm(x, w["n.weight"], 1e-5)
    assert float((out.float().cpu() - want).abs().max()) <= tol * float(want.abs().max())


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_alone(dtype, tol, window):
    """The mixer over a real cache manager: a prompt in two portions, compared with the plain layer."""
    from distie_b200.cache import CacheManager
    from distie_b200.config import PartSpec
    from distie_b200.engine.batch import BatchEntry, StepStaging, lay_out
    from distie_b200.parts import MIXERS, LayerRun, build_part

    hidden, heads, kv_heads, head_dim, theta, tokens = 80, 5, 1, 16, 5000.0, 37
    names = {"q": (heads * head_dim, hidden), "k": (kv_heads * head_dim, hidden), "v": (kv_heads * head_dim, hidden)}
    w = {f"a.{n}_proj.weight": (torch.randn(s) * 0.3).to(torch.bfloat16).float() for n, s in names.items()}
    w.update({f"a.{n}_proj.bias": (torch.randn(s[0]) * 0.3).to(torch.bfloat16).float() for n, s in names.items()})
    w["a.o_proj.weight"] = (torch.randn(hidden, heads * head_dim) * 0.3).to(torch.bfloat16).float()
    spec = PartSpec(
        "gqa_attention",
        {"num_heads": heads, "num_kv_heads": kv_heads, "head_dim": head_dim, "qkv_bias": True, "out_bias": False,
         "window": window, "position": PartSpec("rotary", {"head_dim": head_dim, "theta": theta})},
        "a.",
    )
    ctx = part_context(dtype, w, hidden)
    part = build_part(MIXERS, spec, ctx)
    cache = CacheManager({0: MIXERS.get("gqa_attention").cache_need(spec)}, {}, num_pages=8, page_size=8, max_seats=2,
                         max_tokens_per_request=64, dtype=dtype, device="cuda:0")
    seat = cache.open_seat()
    x = torch.randn(tokens, hidden).to(torch.bfloat16).float()
    staging = StepStaging(256, torch.device("cuda:0"))
    outs, done = [], 0
    for count in (20, 17):
        assert cache.grow(seat, done + count)
        layout = lay_out([BatchEntry(seat, [0] * count, done)])
        cache.upload_tables([seat])
        step, _ = staging.upload(layout)
        run = LayerRun(step=step, seqs=layout.seqs, kv=cache.kv_slot(0), writes_cache=True)
        delta = part.forward(x[done : done + count].cuda().to(dtype), run).float()
        outs.append((delta.sum(0) if delta.dim() == 3 else delta).cpu())
        done += count
        cache.trim(seat, done)
    ctx.kernels.check_errors()
    want, _ = plain.attention_layer(x, w, "a.", torch.arange(tokens), heads, kv_heads, head_dim, theta, window)
    assert float((torch.cat(outs) - want).abs().max()) <= tol * float(want.abs().max())
    if window is not None:
        assert len(cache.pages_held(seat)[0]) < -(-tokens // 8), "pages behind the window were meant to be given back"


def test_position_encoding_part_alone():
    """The rotary part hands the fused kernel the reference's inverse frequencies (model.py:98)."""
    from distie_b200.config import PartSpec
    from distie_b200.parts import POSITION_ENCODINGS, build_part

    ctx = part_context(torch.float32, {}, 64)
    table = build_part(POSITION_ENCODINGS, PartSpec("rotary", {"head_dim": 48, "theta": 12345.0}), ctx).rotary_table()
    assert table.rotary_dim == 48 and not table.interleaved
    assert torch.equal(table.inv_freq.cpu(), plain.rope_inverse_frequencies(48, 12345.0))
    partial = build_part(POSITION_ENCODINGS, PartSpec("rotary", {"head_dim": 48, "theta": 10.0, "rotary_dim": 16}), ctx)
    assert partial.rotary_table().inv_freq.shape == (8,)
    assert build_part(POSITION_ENCODINGS, PartSpec("none", {}), ctx).rotary_table() is None


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 3e-2)])
def test_block_arrangement_alone(dtype, tol):
    """One pre-norm block over a real cache: norms, mixer, feed-forward and both residual sums."""
    from distie_b200.cache import CacheManager
    from distie_b200.config import LayerSpec, PartSpec
    from distie_b200.engine.batch import BatchEntry, StepStaging, lay_out
    from distie_b200.parts import BLOCKS, MIXERS, LayerRun, ResidualStream

    cfg = {"hidden_size": 64, "intermediate_size": 96, "num_attention_heads": 2, "num_key_value_heads": 1,
           "rms_norm_eps": 1e-5, "rope_theta": 3000.0, "num_hidden_layers": 1, "vocab_size": 8}
    w = {k: v.to(torch.bfloat16).float() for k, v in plain.random_weights(cfg, 11, std=0.25, norm_noise=0.05).items()}
    p = "model.layers.0."
    attn = PartSpec("gqa_attention", {"num_heads": 2, "num_kv_heads": 1, "head_dim": 32, "qkv_bias": True, "out_bias": False,
                                      "window": None, "position": PartSpec("rotary", {"head_dim": 32, "theta": 3000.0})}, p + "self_attn.")
    layer = LayerSpec("pre_norm", attn, PartSpec("swiglu", {"intermediate_size": 96}, p + "mlp."),
                      {"input": PartSpec("rmsnorm", {"eps": 1e-5}, p + "input_layernorm."),
                       "post_mixer": PartSpec("rmsnorm", {"eps": 1e-5}, p + "post_attention_layernorm.")})
    ctx = part_context(dtype, w, 64)
    block = BLOCKS.get("pre_norm").build(layer, ctx)
    cache = CacheManager({0: MIXERS.get("gqa_attention").cache_need(attn)}, {}, num_pages=4, page_size=16, max_seats=1,
                         max_tokens_per_request=64, dtype=dtype, device="cuda:0")
    seat, tokens = cache.open_seat(), 19
    cache.grow(seat, tokens)
    h = torch.randn(tokens, 64)
    layout = lay_out([BatchEntry(seat, [0] * tokens, 0)])
    cache.upload_tables([seat])
    step, _ = StepStaging(256, torch.device("cuda:0")).upload(layout)
    stream = ResidualStream(h.cuda().clone())
    block.forward(stream, LayerRun(step=step, seqs=layout.seqs, kv=cache.kv_slot(0)))
    got = stream.settle().cpu()
    ctx.kernels.check_errors()
    want, _ = plain.decoder_layer(h, w, 0, torch.arange(tokens), cfg)
    assert float((got - want).abs().max()) <= tol * float(want.abs().max())


# -- a toy mixer with state of its own, registered from outside the package --------
def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    """A running-mean mixer defined here: state per request, no change to the framework's files."""
    from distie_b200.config import LayerCall, LayerSpec, ModelSpec, PartSpec, register_architecture, unregister_architecture
    from distie_b200.engine.engine import Engine
    from distie_b200.engine.trace_replay import TraceSession
    from distie_b200.parts import MIXERS, StateNeed, TensorSpec
    from distie_b200.weights import write_random_model

    hidden, vocab = 48, 64

    class RunningMeanMixer:
        """delta[t] = W @ mean(x[0..t]) of the token's request; state = (sum [hidden], count [1])."""

        graph_safe = False

        def __init__(self, weight, kernels):
            self.weight, self.kernels = weight, kernels

        @classmethod
        def tensor_specs(cls, spec, hidden_size):
            return [TensorSpec(spec.prefix + "mix.weight", (hidden_size, hidden_size))]

        @classmethod
        def cache_need(cls, spec):
            return None

        @classmethod
        def state_need(cls, spec):
            return StateNeed((hidden + 1,), torch.float32)

        @classmethod
        def build(cls, spec, ctx):
            return cls(ctx.weights.matrix(spec.prefix + "mix.weight"), ctx.kernels)

        def forward(self, x, run):
            means = torch.empty_like(x, dtype=torch.float32)
            for seq in run.seqs:
                state = run.state[seq.seat]
                rows = x[seq.start : seq.start + seq.q_len].float()
                sums = state[:hidden] + torch.cumsum(rows, 0)
                counts = state[hidden] + torch.arange(1, seq.q_len + 1, device=x.device)
                means[seq.start : seq.start + seq.q_len] = sums / counts[:, None]
                state[:hidden] = sums[-1]
                state[hidden] = counts[-1]
            return self.kernels.linear(means.to(x.dtype), self.weight)

    class ToyConfig:
        def __init__(self, raw):
            self.raw = raw
            self.eos_token_id = None

        @classmethod
        def from_dict(cls, raw):
            return cls(dict(raw))

    def recipe(cfg):
        layers = tuple(
            LayerSpec(
                "pre_norm",
                PartSpec("test_running_mean", {}, f"l{i}."),
                PartSpec("swiglu", {"intermediate_size": 80}, f"l{i}.ff."),
                {"input": PartSpec("rmsnorm", {"eps": 1e-5}, f"l{i}.n1."), "post_mixer": PartSpec("rmsnorm", {"eps": 1e-5}, f"l{i}.n2.")},
            )
            for i in range(2)
        )
        return ModelSpec("ToyRunningMean", vocab, hidden, layers, (LayerCall(0, 0), LayerCall(1, 1)),
                         PartSpec("rmsnorm", {"eps": 1e-5}, "norm."), "embed.weight", None)

    MIXERS.register("test_running_mean", RunningMeanMixer)
    register_architecture("ToyRunningMean", ToyConfig, recipe)
    try:
        folder = write_random_model(str(tmp_path / "toy"), {"architectures": ["ToyRunningMean"]}, seed=4, std=0.3, dtype="float32")
        engine = Engine.load(folder, dtype="float32", num_blocks=4, page_size=16, max_seqs=3, decode_graphs=True)
        assert not engine.runner.use_graphs, "a part that reads host-side batch data keeps steps eager"
        assert engine.cache.states[0].shape == (4, hidden + 1) and not engine.cache.groups
        session = TraceSession(engine)
        ids_a, ids_b = helpers.random_ids(vocab, 21, 1), helpers.random_ids(vocab, 9, 2)
        whole = session.run_step([{"id": "w", "tokens": ids_a, "want": list(range(21))}], ["w"])
        parts = [
            session.run_step([{"id": "a", "tokens": ids_a[:8], "want": list(range(8))}, {"id": "b", "tokens": ids_b, "want": [8]}], ["b"]),
            session.run_step([{"id": "a", "tokens": ids_a[8:9], "want": [0]}]),
            session.run_step([{"id": "a", "tokens": ids_a[9:], "want": list(range(12))}], ["a"]),
        ]
        cut = torch.cat([torch.as_tensor(parts[0][:8]), torch.as_tensor(parts[1]), torch.as_tensor(parts[2])])
        assert float((cut - torch.as_tensor(whole)).abs().max()) <= 1e-4 * max(1.0, float(torch.as_tensor(whole).abs().max()))
        seat = engine.cache.open_seat()  # a reopened seat starts from zero state
        assert float(engine.cache.states[0][seat].abs().sum()) == 0.0
        engine.cache.close_seat(seat)
    finally:
        MIXERS.unregister("test_running_mean")
        unregister_architecture("ToyRunningMean")


def test_toy_mixer_with_state_on_the_device_keeps_the_graphs(tmp_path):
    """The same running mean written against the step's device tensors only (the token's seat through
    ``step.seq_seat[step.token_seq]``, its count through ``step.positions``): state of fixed size then costs
    no graphs, and a captured decode step reads and updates the slots of whatever seats it is replayed for."""
    from distie_b200.config import LayerCall, LayerSpec, ModelSpec, PartSpec, register_architecture, unregister_architecture
    from distie_b200.engine.engine import Engine
    from distie_b200.engine.trace_replay import TraceSession
    from distie_b200.parts import MIXERS, StateNeed, TensorSpec
    from distie_b200.weights import write_random_model

    hidden, vocab = 48, 64

    class DeviceRunningMeanMixer:
        """delta[t] = W @ mean(x[0..t]) of the token's request; state = the sum so far [hidden]."""

        graph_safe = True  # nothing below looks at run.seqs or any other host-side batch data

        def __init__(self, weight, kernels):
            self.weight, self.kernels = weight, kernels

        @classmethod
        def tensor_specs(cls, spec, hidden_size):
            return [TensorSpec(spec.prefix + "mix.weight", (hidden_size, hidden_size))]

        @classmethod
        def cache_need(cls, spec):
            return None

        @classmethod
        def state_need(cls, spec):
            return StateNeed((hidden,), torch.float32)

        @classmethod
        def build(cls, spec, ctx):
            return cls(ctx.weights.matrix(spec.prefix + "mix.weight"), ctx.kernels)

        def forward(self, x, run):
            step = run.step
            rows = x.float()
            token_seq = step.token_seq.long()
            seats = step.seq_seat.long()[token_seq]  # the slot of each token's request
            index = torch.arange(rows.shape[0], device=x.device)
            starts = torch.ones_like(token_seq, dtype=torch.bool)
            starts[1:] = token_seq[1:] != token_seq[:-1]
            first = torch.cummax(torch.where(starts, index, torch.zeros_like(index)), 0).values  # first token of the request's portion
            running = torch.cumsum(rows, 0)
            before = torch.cat([torch.zeros_like(running[:1]), running[:-1]])[first]
            sums = run.state[seats] + (running - before)
            means = sums / (step.positions.float() + 1.0)[:, None]
            run.state.index_add_(0, seats, rows)  # every request's slot moves on by its portion
            return self.kernels.linear(means.to(x.dtype), self.weight)

    class ToyConfig:
        def __init__(self, raw):
            self.raw = raw
            self.eos_token_id = None

        @classmethod
        def from_dict(cls, raw):
            return cls(dict(raw))

    def recipe(cfg):
        layers = tuple(
            LayerSpec(
                "pre_norm",
                PartSpec("test_device_running_mean", {}, f"l{i}."),
                PartSpec("swiglu", {"intermediate_size": 80}, f"l{i}.ff."),
                {"input": PartSpec("rmsnorm", {"eps": 1e-5}, f"l{i}.n1."), "post_mixer": PartSpec("rmsnorm", {"eps": 1e-5}, f"l{i}.n2.")},
            )
            for i in range(2)
        )
        return ModelSpec("ToyDeviceRunningMean", vocab, hidden, layers, (LayerCall(0, 0), LayerCall(1, 1)),
                         PartSpec("rmsnorm", {"eps": 1e-5}, "norm."), "embed.weight", None)

    MIXERS.register("test_device_running_mean", DeviceRunningMeanMixer)
    register_architecture("ToyDeviceRunningMean", ToyConfig, recipe)
    try:
        folder = write_random_model(str(tmp_path / "toy"), {"architectures": ["ToyDeviceRunningMean"]}, seed=4, std=0.3, dtype="float32")
        engine = Engine.load(folder, dtype="float32", num_blocks=4, page_size=16, max_seqs=4, decode_graphs=True)
        assert engine.runner.use_graphs, "state indexed on the device keeps the captured decode steps"
        session = TraceSession(engine)
        ids_a, ids_b, ids_c = (helpers.random_ids(vocab, n, seed) for n, seed in ((21, 1), (12, 2), (7, 3)))
        whole = {name: torch.as_tensor(session.run_step([{"id": name, "tokens": ids, "want": list(range(len(ids)))}], [name]))
                 for name, ids in (("a", ids_a), ("b", ids_b), ("c", ids_c))}
        assert engine.runner.graph_replays == 0
        # Portions, then single tokens of two and three requests at once (captured steps of bucket 2 and 4,
        # replayed for changing seats), compared with each request run whole.
        got = {"a": [], "b": [], "c": []}
        out = session.run_step([{"id": "a", "tokens": ids_a[:8], "want": list(range(8))}, {"id": "b", "tokens": ids_b[:5], "want": list(range(5))}])
        got["a"].append(torch.as_tensor(out[:8])), got["b"].append(torch.as_tensor(out[8:]))
        for at in range(5):
            entries = [{"id": "a", "tokens": [ids_a[8 + at]], "want": [0]}, {"id": "b", "tokens": [ids_b[5 + at]], "want": [0]}]
            if at >= 2:
                entries.append({"id": "c", "tokens": [ids_c[at - 2]], "want": [0]})
            out = torch.as_tensor(session.run_step(entries))
            for row, entry in enumerate(entries):
                got[entry["id"]].append(out[row : row + 1])
        assert engine.runner.graph_replays >= 3
        for name, ids in (("a", ids_a), ("b", ids_b), ("c", ids_c)):
            have = torch.cat(got[name])
            want = whole[name][: have.shape[0]]
            assert float((have - want).abs().max()) <= 1e-4 * max(1.0, float(want.abs().max())), name
        for name in "abc":
            session.run_step([], [name])
        seat = engine.cache.open_seat()  # a reopened seat starts from zero state
        assert float(engine.cache.states[0][seat].abs().sum()) == 0.0
        engine.cache.close_seat(seat)
    finally:
        MIXERS.unregister("test_device_running_mean")
        unregister_architecture("ToyDeviceRunningMean")


# -- a toy feed-forward with routing and a toy position encoding, registered from outside the package ------
def test_toy_routed_feed_forward_and_position_encoding(tmp_path):
    """Two experts chosen per token by a router, and a rotation with frequencies of its own: both defined
    here, registered, built from a model folder and stepped, with no change to the framework's files."""
    from distie_b200.config import LayerCall, LayerSpec, ModelSpec, PartSpec, register_architecture, unregister_architecture
    from distie_b200.engine.engine import Engine
    from distie_b200.engine.trace_replay import TraceSession
    from distie_b200.kernels.interface import RotaryTable
    from distie_b200.parts import FEED_FORWARDS, POSITION_ENCODINGS, TensorSpec
    from distie_b200.weights import ModelTensors, write_random_model

    hidden, vocab, inter, heads, kv_heads, head_dim, experts = 64, 96, 48, 4, 2, 16, 3

    class RoutedFeedForward:
        """out[t] = expert_{argmax_e(router[e] . x[t])}(x[t]), each expert a SwiGLU; router logits in float32."""

        graph_safe = False  # the routing below reads nothing on the host, but gathers rows with index ops

        def __init__(self, router, gate_up, down, kernels):
            self.router, self.gate_up, self.down, self.kernels = router, gate_up, down, kernels

        @classmethod
        def tensor_specs(cls, spec, hidden_size):
            p = spec.prefix
            specs = [TensorSpec(p + "router.weight", (experts, hidden_size))]
            for e in range(experts):
                specs += [TensorSpec(p + f"e{e}.gate_proj.weight", (inter, hidden_size)),
                          TensorSpec(p + f"e{e}.up_proj.weight", (inter, hidden_size)),
                          TensorSpec(p + f"e{e}.down_proj.weight", (hidden_size, inter))]
            return specs

        @classmethod
        def build(cls, spec, ctx):
            p, w = spec.prefix, ctx.weights
            gate_up = [torch.cat([w.matrix(p + f"e{e}.gate_proj.weight"), w.matrix(p + f"e{e}.up_proj.weight")]) for e in range(experts)]
            down = [w.matrix(p + f"e{e}.down_proj.weight") for e in range(experts)]
            return cls(w.matrix(p + "router.weight"), gate_up, down, ctx.kernels)

        def forward(self, x, run):
            k = self.kernels
            choice = k.linear(x, self.router, out_dtype=torch.float32).argmax(-1)
            out = torch.zeros((x.shape[0], hidden), dtype=torch.float32, device=x.device)
            for e in range(experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    mid = k.linear_swiglu(x.index_select(0, rows).contiguous(), self.gate_up[e])
                    out.index_copy_(0, rows, k.linear(mid, self.down[e], out_dtype=torch.float32))
            return out

    class SlowRotation:
        """Rotate-half with frequencies of its own: inv_freq[j] = 0.5 / (j + 1)."""

        def __init__(self, table):
            self._table = table

        @classmethod
        def build(cls, spec, ctx):
            d = int(spec.params["head_dim"])
            return cls(RotaryTable((0.5 / torch.arange(1, d // 2 + 1, dtype=torch.float32)).to(ctx.device), d, False))

        def rotary_table(self):
            return self._table

    class ToyConfig:
        def __init__(self, raw):
            self.raw, self.eos_token_id = raw, None

        @classmethod
        def from_dict(cls, raw):
            return cls(dict(raw))

    def recipe(cfg):
        layers = tuple(
            LayerSpec(
                "pre_norm",
                PartSpec("gqa_attention", {"num_heads": heads, "num_kv_heads": kv_heads, "head_dim": head_dim, "qkv_bias": True,
                                           "out_bias": False, "window": None,
                                           "position": PartSpec("test_slow_rotation", {"head_dim": head_dim})}, f"l{i}.attn."),
                PartSpec("test_routed", {}, f"l{i}.ff."),
                {"input": PartSpec("rmsnorm", {"eps": 1e-5}, f"l{i}.n1."), "post_mixer": PartSpec("rmsnorm", {"eps": 1e-5}, f"l{i}.n2.")},
            )
            for i in range(2)
        )
        return ModelSpec("ToyRouted", vocab, hidden, layers, (LayerCall(0, 0), LayerCall(1, 1)),
                         PartSpec("rmsnorm", {"eps": 1e-5}, "norm."), "embed.weight", None)

    def plain_logits(ids, w):
        """The same model written out with the plain functions (rotation with the toy's own frequencies)."""
        ids = torch.as_tensor(ids)
        pos = torch.arange(len(ids))
        angles = pos[:, None].float() * (0.5 / torch.arange(1, head_dim // 2 + 1, dtype=torch.float32))[None, :]
        cos, sin = torch.cat([angles.cos()] * 2, -1), torch.cat([angles.sin()] * 2, -1)
        h = plain.embedding(ids, w["embed.weight"])
        for i in range(2):
            x = plain.rms_norm(h, w[f"l{i}.n1.weight"], 1e-5)
            p = f"l{i}.attn."
            q = torch.nn.functional.linear(x, w[p + "q_proj.weight"], w[p + "q_proj.bias"]).view(-1, heads, head_dim)
            k = torch.nn.functional.linear(x, w[p + "k_proj.weight"], w[p + "k_proj.bias"]).view(-1, kv_heads, head_dim)
            v = torch.nn.functional.linear(x, w[p + "v_proj.weight"], w[p + "v_proj.bias"]).view(-1, kv_heads, head_dim)
            mixed = plain.attention_mix(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v, None)
            h = h + torch.nn.functional.linear(mixed.reshape(len(ids), -1), w[p + "o_proj.weight"])
            x = plain.rms_norm(h, w[f"l{i}.n2.weight"], 1e-5)
            choice = torch.nn.functional.linear(x, w[f"l{i}.ff.router.weight"]).argmax(-1)
            rows = [plain.swiglu_mlp(x[t : t + 1], w, f"l{i}.ff.e{int(choice[t])}.") for t in range(len(ids))]
            h = h + torch.cat(rows)
        return torch.nn.functional.linear(plain.rms_norm(h, w["norm.weight"], 1e-5), w["embed.weight"])

    FEED_FORWARDS.register("test_routed", RoutedFeedForward)
    POSITION_ENCODINGS.register("test_slow_rotation", SlowRotation)
    register_architecture("ToyRouted", ToyConfig, recipe)
    try:
        folder = write_random_model(str(tmp_path / "routed"), {"architectures": ["ToyRouted"]}, seed=6, std=0.3, dtype="float32")
        stored = ModelTensors(folder)
        weights = {n: stored.tensor(n).float() for n in stored.keys()}
        engine = Engine.load(folder, dtype="float32", num_blocks=16, page_size=8, max_seqs=3)
        session = TraceSession(engine)
        ids_a, ids_b = helpers.random_ids(vocab, 30, 3), helpers.random_ids(vocab, 11, 4)
        first = session.run_step([{"id": "a", "tokens": ids_a[:13], "want": list(range(13))},
                                  {"id": "b", "tokens": ids_b, "want": list(range(11))}], ["b"])
        rest = [session.run_step([{"id": "a", "tokens": [t], "want": [0]}]) for t in ids_a[13:]]
        session.run_step([], ["a"])
        got_a = torch.cat([torch.as_tensor(first[:13])] + [torch.as_tensor(r) for r in rest])
        got_b = torch.as_tensor(first[13:])
        for got, ids in ((got_a, ids_a), (got_b, ids_b)):
            want = plain_logits(ids, weights)
            assert float((got - want).abs().max()) <= 1e-4 * float(want.abs().max())
        used = {int(c) for i in range(2) for c in torch.nn.functional.linear(
            plain.rms_norm(plain.embedding(torch.as_tensor(ids_a), weights["embed.weight"]), weights[f"l{i}.n2.weight"], 1e-5),
            weights[f"l{i}.ff.router.weight"]).argmax(-1)}
        assert len(used) > 1, "the test is meant to send tokens to more than one expert"
        assert engine.cache.free_pages() == engine.cache.total_pages()
    finally:
        FEED_FORWARDS.unregister("test_routed")
        POSITION_ENCODINGS.unregister("test_slow_rotation")
        unregister_architecture("ToyRouted")
