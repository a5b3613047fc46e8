"""The reference arm of ``bench.py``: the unmodified reference engine on the same workload.

The reference (stanzixinwan/distie) is not a package: it has no ``setup.py`` and no
``pyproject.toml``, its worker runs with ``PYTHONPATH=worker/src`` (README.md:88).  A copy of
its ``worker/`` and ``core/`` trees under ``baseline/_ref`` (or the tree ``DISTIE_REF`` names)
is therefore put on ``sys.path`` as it is.  Nothing of ``distie_b200`` is imported here.

What runs is the reference's stock serving path, built the way its own engine builds it
(worker/src/inference/torch_engine.py:210-240, 416-446):

* ``Qwen2CausalLM(Qwen2Dims(...))`` with random ``N(0, 0.02)`` weights in bfloat16;
* its C++ ``BlockPool`` (``core/``, compiled with ``g++`` as ``scripts/build_core.sh`` does
  with CMake) through ``inference.native.load_block_pool``;
* ``PagedKvCache`` with one spare page, ``Scheduler``, ``ModelRunner`` and, when its flash
  path is on, ``BatchDecodeGraphs``.

Attention backend: the reference's serving configuration is ``DISTIE_ATTN=flash`` (README.md:88,
every published result); its default ``torch`` is the exact path for float32 checks and keeps
every step eager.  ``auto`` takes ``flash`` when the installed ``flash_attn`` runs on this GPU
and falls back to ``torch`` with a note otherwise.

* ``value``: K decode steps of ``ModelRunner.step`` on plans of its ``Scheduler`` between two
  CUDA events (each of its steps ends with a host read of the sampled ids).
* ``e2e``: the same through its public API, ``TorchEngine.generate`` (asyncio, one coroutine
  per request, the ``BatchLoop`` inside), with a tokenizer that maps ``"5 17 3"`` to ids.
"""

from __future__ import annotations

import asyncio
import os
import statistics
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))


class Unavailable(RuntimeError):
    pass


def find_reference() -> tuple[str, str | None]:
    """``(worker/src, core/build or None)`` of the first reference tree found."""
    roots = [os.environ.get("DISTIE_REF"), os.path.join(HERE, "_ref"), "/root/reference"]
    for root in roots:
        if root and os.path.isfile(os.path.join(root, "worker", "src", "inference", "scheduler.py")):
            build = os.path.join(root, "core", "build")
            return os.path.join(root, "worker", "src"), build if os.path.isdir(build) else None
    raise Unavailable("no copy of the reference under baseline/_ref, DISTIE_REF or /root/reference")


_PROBE = """
import torch
from flash_attn import flash_attn_with_kvcache
q = torch.randn(2, 1, 4, 128, device='cuda', dtype=torch.bfloat16)
kc = torch.zeros(3, 256, 2, 128, device='cuda', dtype=torch.bfloat16)
vc = torch.zeros_like(kc)
k = torch.randn(2, 1, 2, 128, device='cuda', dtype=torch.bfloat16)
table = torch.tensor([[0], [1]], dtype=torch.int32, device='cuda')
lens = torch.tensor([5, 9], dtype=torch.int32, device='cuda')
out = flash_attn_with_kvcache(q, kc, vc, k=k, v=k.clone(), cache_seqlens=lens, block_table=table, causal=True)
torch.cuda.synchronize()
assert torch.isfinite(out.float()).all()
print('flash ok')
"""


def flash_usable() -> tuple[bool, str]:
    """Whether the installed flash_attn runs its paged decode call on this GPU (tried in a child process)."""
    try:
        proc = subprocess.run([sys.executable, "-c", _PROBE], capture_output=True, text=True, timeout=300)
    except Exception as exc:  # noqa: BLE001
        return False, f"probe did not run: {exc}"
    if proc.returncode == 0 and "flash ok" in proc.stdout:
        return True, ""
    tail = (proc.stderr or proc.stdout).strip().splitlines()
    return False, tail[-1][:200] if tail else f"exit code {proc.returncode}"


class IdTokenizer:
    """Prompts are token ids written as text; the reference tokenises with a model library."""

    eos_token_id = None
    chat_template = None

    def encode(self, prompt, add_special_tokens=True):
        return [int(part) for part in prompt.split()]

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(str(int(i)) for i in ids)


class ReferenceEngine:
    """The reference's model, pool, cache, scheduler and runner, put together as its engine does."""

    def __init__(self, shape: dict, layers: int, max_seqs: int, num_pages: int, backend: str, device: str = "cuda") -> None:
        import torch

        self.device = device

        os.environ["DISTIE_ATTN"] = backend
        os.environ["WORKER_MAX_SEQS"] = str(max_seqs)
        os.environ["WORKER_TOKEN_BUDGET"] = "2048"
        from inference.native import load_block_pool
        from inference.qwen2.model import Qwen2CausalLM, Qwen2Dims
        from inference.torch_engine import TorchEngine, _maybe_paged_cache

        dims = Qwen2Dims(
            vocab_size=shape["vocab_size"], hidden_size=shape["hidden_size"],
            intermediate_size=shape["intermediate_size"], num_hidden_layers=layers,
            num_attention_heads=shape["num_attention_heads"], num_key_value_heads=shape["num_key_value_heads"],
            head_dim=shape["head_dim"], rms_norm_eps=shape["rms_norm_eps"], rope_theta=shape["rope_theta"],
            tie_word_embeddings=shape["tie_word_embeddings"],
        )
        torch.manual_seed(0)
        with torch.device(device):
            model = Qwen2CausalLM(dims)
        model = model.to(torch.bfloat16 if device == "cuda" else torch.float32)
        with torch.no_grad():
            for name, param in model.named_parameters():
                if name.endswith("layernorm.weight") or name == "norm.weight":
                    param.fill_(1.0)
                else:
                    param.normal_(0.0, 0.02)
        model.eval()
        self.model = model
        self.dims = dims
        self.pool = load_block_pool(num_pages)
        self.kv = _maybe_paged_cache(model, self.pool, device)  # one spare page, page size by backend
        self.engine = TorchEngine(model, IdTokenizer(), device, self.pool, self.kv)
        self.max_seqs = max_seqs

    def scheduler_and_runner(self):
        """A scheduler and a runner of their own (the engine's loop keeps its pair to itself)."""
        from inference.model_runner import ModelRunner
        from inference.scheduler import Scheduler

        scheduler = Scheduler(self.pool, page_size=self.kv.page_size, max_seqs=self.max_seqs, token_budget=2048)
        runner = ModelRunner(self.model, self.kv, self.device, self.engine._decode_graphs(self.max_seqs))
        return scheduler, runner

    def weight_bytes(self) -> int:
        seen = {}
        for name, param in self.model.named_parameters():
            if name.startswith("embed_tokens") and not self.dims.tie_word_embeddings:
                continue
            seen[param.data_ptr()] = param.numel() * param.element_size()
        return sum(seen.values())

    def kv_bytes_per_token(self) -> int:
        d = self.dims
        return 2 * d.num_hidden_layers * d.num_key_value_heads * d.head_dim * 2


class _DeviceTimer:
    """CUDA events on the current stream with a synchronise on both sides (wall clock on a CPU, for dry runs)."""

    def __init__(self, device: str) -> None:
        self.cuda = device == "cuda"

    def __enter__(self):
        import torch

        if self.cuda:
            torch.cuda.synchronize()
            self.begin, self.end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.begin.record()
        else:
            self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        import torch

        if self.cuda:
            self.end.record()
            torch.cuda.synchronize()
            self.ms = self.begin.elapsed_time(self.end)
        else:
            self.ms = (time.perf_counter() - self.t0) * 1e3


def _random_prompt(vocab: int, length: int, seed: int) -> list[int]:
    import torch

    return torch.randint(0, vocab, (length,), generator=torch.Generator().manual_seed(seed)).tolist()


def time_decode(ref: ReferenceEngine, batch: int, prompt_len: int, steps: int, warmup: int) -> dict:
    import torch
    from inference.scheduler import Sequence

    scheduler, runner = ref.scheduler_and_runner()
    vocab = ref.dims.vocab_size
    for b in range(batch):
        scheduler.submit(Sequence(f"bench-{b}", _random_prompt(vocab, prompt_len, 100 + b), warmup + steps + 8))

    def one_step():
        plan = scheduler.schedule()
        scheduler.complete(plan, runner.step(plan))
        return plan

    while True:  # prefill, as its scheduler deals the prompts out
        plan = one_step()
        if scheduler.num_waiting == 0 and all(len(item.token_ids) == 1 for item in plan.items) and len(plan.items) == batch:
            break
    for _ in range(max(warmup, 1) - 1):
        one_step()
    with _DeviceTimer(ref.device) as timer:
        for _ in range(steps):
            one_step()
    ms = timer.ms
    for b in range(batch):
        scheduler.abort(f"bench-{b}")
    scheduler.schedule()
    return {
        "ms_per_step": ms / steps,
        "tokens_per_s": batch * steps / (ms / 1e3),
        "mean_context": prompt_len + max(warmup, 1) + steps / 2,
        "graphs": runner.graphs_active,
    }


def time_prefill(ref: ReferenceEngine, tokens: int, repeats: int = 5) -> dict:
    import torch
    from inference.scheduler import Sequence

    scheduler, runner = ref.scheduler_and_runner()
    times = []
    for index in range(repeats + 2):
        seq = Sequence(f"prefill-{index}", _random_prompt(ref.dims.vocab_size, tokens, 7), 1)
        scheduler.submit(seq)
        plan = scheduler.schedule()
        assert len(plan.items) == 1 and len(plan.items[0].token_ids) == tokens
        with _DeviceTimer(ref.device) as timer:
            picks = runner.step(plan)
        times.append(timer.ms)
        scheduler.complete(plan, picks)  # one new token: finished, pages returned
    ms = statistics.median(times[2:])
    return {"ms": ms, "tokens": tokens, "value": tokens / (ms / 1e3)}


def time_e2e(ref: ReferenceEngine, batch: int, prompt_len: int, steps: int, warmup: int) -> dict:
    """Through ``TorchEngine.generate``: tokens per second while every request decodes."""
    from inference.engine import HARD_MAX_TOKENS, GenerateRequest

    total = min(HARD_MAX_TOKENS, warmup + steps + batch + 8)  # its engine caps a request at 256 new tokens
    vocab = ref.dims.vocab_size
    stamps: list[list[float]] = [[] for _ in range(batch)]

    async def one(index: int) -> None:
        prompt = " ".join(str(t) for t in _random_prompt(vocab, prompt_len, 500 + index))
        req = GenerateRequest(request_id=f"e2e-{index}", model_name="bench", prompt=prompt, max_tokens=total)
        async for _event in ref.engine.generate(req):
            stamps[index].append(time.perf_counter())

    async def everything() -> None:
        await asyncio.gather(*(one(i) for i in range(batch)))
        await ref.engine.close()

    asyncio.run(everything())
    # Steady state: after every request has its first `warmup` tokens, until the first request ends.
    begin = max(s[min(warmup, len(s) - 1)] for s in stamps)
    end = min(s[-1] for s in stamps)
    produced = sum(1 for s in stamps for t in s if begin < t <= end)
    timed_steps = max(1, produced // batch)
    elapsed = max(end - begin, 1e-9)
    size = batch
    width = ref.kv.num_blocks
    graphs = bool(os.environ.get("DISTIE_ATTN") == "flash")
    # What a step copies: with graphs, token and position (int64), length (int32) and the whole table row;
    # eagerly, ids, positions, slots, last rows (int64), two cumulative lengths and the padded tables (int32).
    pages = -(-(prompt_len + total) // ref.kv.page_size)
    h2d = size * (8 + 8 + 4 + 4 * width) if graphs else size * (8 * 4 + 4 * 2 + 4 * pages) + 8
    return {
        "value": produced / elapsed,
        "unit": "tokens/s",
        "h2d_bytes_per_step": int(h2d),
        "d2h_bytes_per_step": batch * 8,
        "ms_per_step": elapsed / timed_steps * 1e3,
        "steps_timed": timed_steps,
    }


def run(args, shape: dict, layers: int, peaks: dict, peaks_kind: str, constants: dict, sampler_cls, prefill_flops) -> dict:
    """The reference's JSON line (same keys as this repository's own arm)."""
    src, core_build = find_reference()
    if core_build is None:
        raise Unavailable("the reference's C++ pool is not built (baseline/_ref/core/build has no distie_core)")
    sys.path.insert(0, src)
    os.environ["DISTIE_CORE_DIR"] = core_build
    prompt_len, context, prefill_tokens = constants["prompt_len"], constants["context"], constants["prefill_tokens"]

    backend = (getattr(args, "ref_attn", None) or os.environ.get("DISTIE_ATTN") or "auto").strip().lower()
    note = ""
    if backend == "auto":
        ok, why = flash_usable() if (getattr(args, "ref_device", None) or "cuda") == "cuda" else (False, "not a CUDA run")
        backend = "flash" if ok else "torch"
        if not ok:
            note = f"flash_attn not usable here ({why}); the reference's default torch path ran"
    page = 256 if backend == "flash" else 16
    new_tokens = args.warmup + args.steps + 16
    per_request = -(-(prompt_len + max(new_tokens, 256 + 8) + 1) // page)
    pages = 64 * per_request + 2 * -(-prefill_tokens // page)
    device = getattr(args, "ref_device", None) or "cuda"
    ref = ReferenceEngine(shape, layers, 64, pages, backend, device)

    failures = {}

    def attempt(name, call):
        try:
            return call()
        except Exception as exc:  # noqa: BLE001  (one point that cannot run must not hide the others)
            failures[name] = f"{type(exc).__name__}: {exc}"[:300]
            return None

    with sampler_cls() as sampler:
        head = time_decode(ref, args.batch, prompt_len, args.steps, args.warmup)
        e2e = attempt("e2e", lambda: time_e2e(ref, args.batch, prompt_len, args.steps, args.warmup))
        points = {}
        for batch in (1, 64):
            got = attempt(f"decode_b{batch}", lambda: time_decode(ref, batch, prompt_len, args.steps, args.warmup))
            points[f"decode_b{batch}"] = round(got["tokens_per_s"], 1) if got else None
        prefill = attempt("prefill", lambda: time_prefill(ref, prefill_tokens))
        time.sleep(0.3)
    clocks = sampler.summary()

    step_bytes = ref.weight_bytes() + args.batch * head["mean_context"] * ref.kv_bytes_per_token()
    achieved = step_bytes / (head["ms_per_step"] / 1e3) / 1e9
    if prefill:
        flops = prefill_flops(shape, layers, prefill_tokens)
        prefill["frac"] = round(flops / (prefill["ms"] / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)
        prefill["value"], prefill["ms"] = round(prefill["value"], 1), round(prefill["ms"], 3)
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
        "impl": "reference",
        "reference_backend": f"DISTIE_ATTN={backend}, page {ref.kv.page_size}, decode graphs {'on' if head['graphs'] else 'off'}",
        "config": {
            "model": "Qwen2.5-1.5B shape (Qwen2ForCausalLM)", "layers": layers, "layers_full": shape["num_hidden_layers"],
            "hidden": shape["hidden_size"], "q_heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
            "head_dim": shape["head_dim"], "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
            "tied": shape["tie_word_embeddings"], "global_batch": args.batch, "prompt_len": prompt_len,
            "seq_len": context, "page_size": ref.kv.page_size, "parallelism": "none (1 GPU)",
            "decode": "CUDA graph per batch bucket" if head["graphs"] else "eager",
            "l2": "inputs larger than L2 (the weights alone, read once per step)", "peaks": peaks_kind,
        },
        "e2e": {k: (round(v, 1) if isinstance(v, float) else v) for k, v in e2e.items()} if e2e else None,
        "points": points,
        "prefill": prefill,
        "roofline": {
            "bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": round(achieved / peaks["hbm_gbs"], 4),
        },
        "clocks": clocks,
    }
    if note:
        line["note"] = note
    if failures:
        line["unavailable_points"] = failures
    return line
