"""The decoder every recipe builds: embedding, the run order over blocks, final norm, head.

Nothing here names an architecture.  ``forward`` runs only the tokens of the step
it is given, against the cache slots the step's :class:`CacheView` hands out, and
returns float32 logits at the wanted rows (embedding -> layers -> row select ->
final norm -> head, the order of worker/src/inference/qwen2/model.py:369-380).
A spec may put constants around the stack (a scale on the embedded tokens, a scale
and a soft cap on the logits); the architecture built here sets none of them.
"""

from __future__ import annotations

from typing import Protocol

import torch

from ..config.model_spec import ModelSpec
from ..kernels.interface import KernelSet, KvSlot, StepTensors
from ..parts.base import BLOCKS, MIXERS, NORMS, BuildContext, CacheNeed, LayerRun, ResidualStream, StateNeed, TensorSpec, build_part
from ..parts.linear import Linear


def model_tensor_specs(spec: ModelSpec) -> list[TensorSpec]:
    """Every tensor the model reads, in a fixed order (also the order random weights are drawn in)."""
    specs = [TensorSpec(spec.embedding_name, (spec.vocab_size, spec.hidden_size), "table")]
    for layer in spec.layers:
        specs += BLOCKS.get(layer.block).tensor_specs(layer, spec.hidden_size)
    specs += NORMS.get(spec.final_norm.kind).tensor_specs(spec.final_norm, spec.hidden_size)
    if spec.head_name is not None:
        specs.append(TensorSpec(spec.head_name, (spec.vocab_size, spec.hidden_size), "table"))
    return specs


def slot_needs(spec: ModelSpec) -> tuple[dict[int, CacheNeed], dict[int, StateNeed]]:
    """What each cache slot's owning mixer asks of the cache manager."""
    caches: dict[int, CacheNeed] = {}
    states: dict[int, StateNeed] = {}
    for call in spec.order:
        if not call.writes_cache:
            continue
        mixer = spec.layers[call.layer].mixer
        cls = MIXERS.get(mixer.kind)
        need = cls.cache_need(mixer)
        if need is not None:
            caches[call.cache_slot] = need
        state = cls.state_need(mixer)
        if state is not None:
            states[call.cache_slot] = state
    return caches, states


class CacheView(Protocol):
    def kv_slot(self, slot: int) -> KvSlot | None: ...

    def state_slot(self, slot: int) -> torch.Tensor | None: ...


class DecoderModel:
    def __init__(self, spec: ModelSpec, kernels: KernelSet, weights) -> None:
        self.spec = spec
        self.kernels = kernels
        ctx = BuildContext(kernels, spec.hidden_size, weights)
        self.embedding = weights.table(spec.embedding_name)
        self.blocks = [BLOCKS.get(layer.block).build(layer, ctx) for layer in spec.layers]
        self.final_norm = build_part(NORMS, spec.final_norm, ctx)
        head = self.embedding if spec.head_name is None else weights.table(spec.head_name)
        self.head = Linear(head, None, kernels)
        weights.release()

    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    def weight_bytes(self) -> int:
        """Bytes of every distinct weight tensor a decode step reads (the embedding only as the tied head)."""
        seen: dict[int, int] = {}

        def visit(obj) -> None:
            if isinstance(obj, torch.Tensor):
                seen[obj.data_ptr()] = obj.numel() * obj.element_size()
            elif isinstance(obj, (list, tuple)):
                for item in obj:
                    visit(item)
            elif hasattr(obj, "__dict__") and not isinstance(obj, (KernelSet, type)):
                for value in vars(obj).values():
                    if not isinstance(value, KernelSet):
                        visit(value)

        visit(self.blocks)
        visit(self.final_norm)
        visit(self.head)
        return sum(seen.values())

    def forward(self, step: StepTensors, seqs, cache: CacheView, logit_rows: torch.Tensor | None) -> torch.Tensor | None:
        k = self.kernels
        residual = torch.empty((step.num_tokens, self.spec.hidden_size), dtype=torch.float32, device=k.device)
        k.embed(step, self.embedding, residual)
        if self.spec.embedding_scale is not None:
            residual.mul_(float(self.spec.embedding_scale))
        stream = ResidualStream(residual)
        for call in self.spec.order:
            run = LayerRun(
                step=step,
                seqs=seqs,
                kv=cache.kv_slot(call.cache_slot),
                state=cache.state_slot(call.cache_slot),
                writes_cache=call.writes_cache,
            )
            self.blocks[call.layer].forward(stream, run)
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        x = torch.empty((logit_rows.numel(), self.spec.hidden_size), dtype=k.dtype, device=k.device)
        self.final_norm.apply(stream.pending, residual, x, logit_rows)
        logits = self.head(x, out_dtype=torch.float32)
        if self.spec.logit_scale is not None:
            logits.mul_(float(self.spec.logit_scale))
        if self.spec.logit_softcap is not None:
            cap = float(self.spec.logit_softcap)
            logits = torch.tanh(logits / cap).mul_(cap)
        return logits
