"""Anchors in the reference project's own code, run live when a copy of it is on disk.

The reference (stanzixinwan/distie) needs no installation: its worker runs from
``worker/src`` on ``sys.path``, and its model, cache, batch builder and scheduler
import with torch alone.  A copy is looked for under ``DISTIE_REF``,
``baseline/_ref`` and ``/root/reference``; without one these tests are skipped and
``tests/golden/reference_logits.pt`` (made once by ``tests/golden/make_golden.py``)
remains the anchor.

* The plain implementation of ``tests/plain_qwen2.py`` against the reference's
  ``Qwen2CausalLM``: its dense ``forward`` and its paged, batched ``forward_batch`` fed in
  portions beside another request (worker/src/inference/qwen2/model.py:305-314, 369-380).
* This engine's scheduler against the reference's ``Scheduler`` on scripted workloads
  (worker/src/inference/scheduler.py:141-236): with a token budget that never binds and no
  ``prefill_chunk`` both must take the same decisions, step by step.
"""

from __future__ import annotations

import os
import random
import sys

import pytest
import torch

import helpers
import plain_qwen2 as plain

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_src() -> str | None:
    for root in (os.environ.get("DISTIE_REF"), os.path.join(ROOT, "baseline", "_ref"), "/root/reference"):
        if root and os.path.isfile(os.path.join(root, "worker", "src", "inference", "scheduler.py")):
            return os.path.join(root, "worker", "src")
    return None


SRC = _reference_src()
pytestmark = pytest.mark.skipif(SRC is None, reason="no copy of the reference project on disk")


@pytest.fixture(scope="module")
def reference():
    sys.path.insert(0, SRC)
    try:
        import inference.kv_cache as kv_cache
        import inference.qwen2.model as model
        import inference.qwen2.paged_attn as paged_attn
        import inference.scheduler as scheduler

        yield {"kv_cache": kv_cache, "model": model, "paged_attn": paged_attn, "scheduler": scheduler}
    finally:
        sys.path.remove(SRC)


def _reference_model(ref, cfg, weights):
    dims = ref["model"].Qwen2Dims(
        vocab_size=cfg["vocab_size"], hidden_size=cfg["hidden_size"], intermediate_size=cfg["intermediate_size"],
        num_hidden_layers=cfg["num_hidden_layers"], num_attention_heads=cfg["num_attention_heads"],
        num_key_value_heads=cfg["num_key_value_heads"], head_dim=plain.head_dim_of(cfg),
        rms_norm_eps=cfg["rms_norm_eps"], rope_theta=cfg["rope_theta"], tie_word_embeddings=cfg["tie_word_embeddings"],
    )
    model = ref["model"].Qwen2CausalLM(dims).eval()
    state = {(k[len("model."):] if k.startswith("model.") else k): v for k, v in weights.items()}
    if cfg["tie_word_embeddings"]:
        state["lm_head.weight"] = state["embed_tokens.weight"]
    model.load_state_dict(state)
    return model, dims


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_plain_matches_the_reference_model_live(reference, name):
    cfg, page, weights = helpers.tiny(name)
    model, dims = _reference_model(reference, cfg, weights)
    ids = helpers.random_ids(cfg["vocab_size"], 61, 321)
    other = helpers.random_ids(cfg["vocab_size"], 9, 7)
    want = plain.forward_logits(ids, weights, cfg)
    want_other = plain.forward_logits(other, weights, cfg)
    scale = plain.logit_scale(want)
    kv, pa = reference["kv_cache"], reference["paged_attn"]
    with torch.inference_mode():
        dense = model(torch.tensor([ids]))[0].float()
        assert float((dense - want).abs().max()) <= 2e-5 * scale
        assert torch.equal(dense.argmax(-1), want.argmax(-1))
        # Its paged, batched path: 29 tokens, 16 more beside a second request, then the rest token by token
        # beside that request's decoded tokens.  forward_batch returns each request's last row.
        pages = -(-len(ids) // page)
        cache = kv.PagedKvCache(kv.KvShape(dims.num_hidden_layers, dims.num_key_value_heads, dims.head_dim),
                                pages + 4, "cpu", torch.float32, page)
        mine, theirs = tuple(range(pages)), tuple(range(pages, pages + 4))
        last = model.forward_batch(torch.tensor(ids[:29]), cache, pa.build_batch([pa.BatchSeq(mine, 0, 29)], cache, "cpu"))
        assert float((last[0].float() - want[28]).abs().max()) <= 2e-5 * scale
        meta = pa.build_batch([pa.BatchSeq(mine, 29, 16), pa.BatchSeq(theirs, 0, 5)], cache, "cpu")
        last = model.forward_batch(torch.tensor(ids[29:45] + other[:5]), cache, meta)
        assert float((last[0].float() - want[44]).abs().max()) <= 2e-5 * scale
        assert float((last[1].float() - want_other[4]).abs().max()) <= 2e-5 * plain.logit_scale(want_other)
        for at in range(45, len(ids)):
            seqs = [pa.BatchSeq(mine, at, 1)]
            tokens = [ids[at]]
            step = at - 45
            if 5 + step < len(other):
                seqs.append(pa.BatchSeq(theirs, 5 + step, 1))
                tokens.append(other[5 + step])
            last = model.forward_batch(torch.tensor(tokens), cache, pa.build_batch(seqs, cache, "cpu"))
            assert float((last[0].float() - want[at]).abs().max()) <= 2e-5 * scale, at
            if len(seqs) == 2:
                assert float((last[1].float() - want_other[5 + step]).abs().max()) <= 2e-5 * plain.logit_scale(want_other)


class CountingPool:
    """Page ids with the native pool's surface (allocate, free, num_blocks, num_free): lowest ids first
    at the start, last freed first afterwards."""

    def __init__(self, num_blocks: int) -> None:
        self.num_blocks = num_blocks
        self._free = list(range(num_blocks - 1, -1, -1))

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self, count: int):
        if count > len(self._free):
            raise RuntimeError("out of blocks")
        return [self._free.pop() for _ in range(count)]

    def free(self, ids) -> None:
        self._free.extend(ids)


def _token(request_id: str, index: int) -> int:
    """A stand-in for the model: the token a request produces at output position `index`."""
    return (sum(map(ord, request_id)) * 31 + index * 7) % 50 + 1


def _script(seed: int, count: int, pages: int, page: int):
    """Requests (name, prompt length, new tokens, step at which they arrive) and aborts (step, name)."""
    rng = random.Random(seed)
    arrivals, aborts, step = [], [], 0
    for index in range(count):
        step += rng.choice((0, 0, 1, 2, 5))
        longest = pages * page
        prompt = rng.randint(1, max(1, longest // 3))
        new = rng.randint(1, max(1, min(24, longest - prompt)))
        arrivals.append((f"q{index}", prompt, new, step))
        if rng.random() < 0.15:
            aborts.append((step + rng.randint(1, 12), f"q{index}"))
    return arrivals, aborts


@pytest.mark.parametrize("seed,pages,page,seats", [(0, 12, 4, 4), (1, 9, 4, 3), (2, 40, 8, 6), (3, 6, 16, 2), (4, 14, 4, 8)])
def test_scheduler_takes_the_reference_schedulers_decisions(reference, seed, pages, page, seats):
    """The same arrivals, aborts and sampled tokens through both schedulers: every step the same requests
    run with the same number of tokens behind the same number of cached tokens, the same tokens are
    emitted, and the same requests are sent back when pages run out."""
    from distie_b200.cache import CacheManager
    from distie_b200.engine.scheduler import Scheduler, Sequence
    from distie_b200.parts import CacheNeed

    ref = reference["scheduler"]
    budget = 10 * pages * page  # never binds: the reference has no portions, so a budget that cuts a prompt differs by design
    eos = 17
    theirs = ref.Scheduler(CountingPool(pages), page_size=page, max_seqs=seats, token_budget=budget)
    cache = CacheManager({0: CacheNeed(1, 16, None)}, {}, num_pages=pages, page_size=page, max_seats=seats,
                         max_tokens_per_request=pages * page)
    ours = Scheduler(cache, seats, budget, None)
    arrivals, aborts = _script(seed, 24, pages, page)
    mine: dict[str, Sequence] = {}
    its: dict[str, object] = {}
    step = preempted = 0
    while arrivals or aborts or ours.has_work() or theirs.has_work():
        assert step < 2000
        while arrivals and arrivals[0][3] <= step:
            name, prompt, new, _ = arrivals.pop(0)
            ids = list(range(1, prompt + 1))
            mine[name] = Sequence(name, ids, new, eos_id=eos)
            its[name] = ref.Sequence(request_id=name, prompt_ids=list(ids), max_new_tokens=new, eos_id=eos)
            ours.submit(mine[name])
            theirs.submit(its[name])
        for at, name in [a for a in aborts if a[0] <= step]:
            ours.abort(name)
            theirs.abort(name)
        aborts = [a for a in aborts if a[0] > step]
        plan_a, plan_b = ours.schedule(), theirs.schedule()
        key = lambda item: item.seq.request_id  # noqa: E731  (the reference lists requests in admission order, this engine decoding ones first)
        items_a, items_b = sorted(plan_a.items, key=key), sorted(plan_b.items, key=key)
        assert [(i.seq.request_id, i.past_len, list(i.token_ids)) for i in items_a] == \
               [(i.seq.request_id, i.past_len, list(i.token_ids)) for i in items_b], f"step {step}"
        assert all(item.samples for item in plan_a.items), "without portions every scheduled request samples"
        assert (ours.num_waiting, ours.num_running) == (theirs.num_waiting, theirs.num_running), f"step {step}"
        assert [s.request_id for s in ours.running()] == [s.request_id for s in theirs._running]
        assert [s.request_id for s in ours.waiting()] == [s.request_id for s in theirs._waiting]
        token_of = lambda item: _token(item.seq.request_id, item.past_len + len(item.token_ids) - len(item.seq.prompt_ids))  # noqa: E731
        out_a = ours.complete(plan_a, [token_of(i) for i in plan_a.items])
        out_b = theirs.complete(plan_b, [token_of(i) for i in plan_b.items])
        assert sorted((e.seq.request_id, e.token_id, e.finished) for e in out_a) == \
               sorted((e.seq.request_id, e.token_id, e.finished) for e in out_b), f"step {step}"
        step += 1
    for name, seq in mine.items():
        assert seq.output_ids == its[name].output_ids and seq.preemptions == its[name].preemptions, name
        preempted += seq.preemptions
    assert cache.free_pages() == pages and cache.free_seats == seats
    if seed in (0, 1, 3):
        assert preempted > 0, "these pools were meant to be too small"
