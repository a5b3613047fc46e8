"""Architecture-neutral description of a decoder: which parts, in which order.

An architecture's recipe (for instance ``distie_b200.models.qwen2``) turns its typed
configuration into a :class:`ModelSpec`.  Everything below the recipe -- the weight
loader, the random initialiser, the cache manager and the model builder -- reads
only the spec, never the architecture's name.

* :class:`PartSpec` names one part (a mixer, a feed-forward, a norm, a position
  encoding) by its registry ``kind``, gives the constants it needs and the prefix
  its tensors carry in the checkpoint.
* :class:`LayerSpec` is one block: its arrangement (``block``) and its parts.
* :class:`LayerCall` is one entry of the run order.  The order is data: it may
  name a layer twice, and a call may read the cache that an earlier call wrote.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""

    def with_prefix(self, prefix: str) -> "PartSpec":
        return PartSpec(self.kind, self.params, prefix)


@dataclass(frozen=True)
class LayerSpec:
    """One block.  ``block`` picks the arrangement of the parts (registry kind)."""

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Mapping[str, PartSpec]


@dataclass(frozen=True)
class LayerCall:
    """One step of the run order.

    ``layer`` indexes :attr:`ModelSpec.layers`.  ``cache_slot`` is the slot of
    the cache (or of the per-request state) the call's mixer works on; calls
    with ``writes_cache=False`` read what the call owning that slot stored and
    store nothing themselves.
    """

    layer: int
    cache_slot: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: tuple[LayerSpec, ...]
    order: tuple[LayerCall, ...]
    final_norm: PartSpec
    embedding_name: str
    head_name: str | None  # None: the head is the embedding table (tied)
    tolerated: tuple[str, ...] = ()  # tensors a checkpoint may carry although the model does not read them
    max_positions: int | None = None
    eos_token_id: int | None = None
    init: Mapping[str, float] = field(default_factory=dict)  # hints for random weights
    # Constants some architectures put around the stack of layers; all off (None) for the plain decoder.
    embedding_scale: float | None = None  # the embedded tokens are multiplied by it
    logit_scale: float | None = None      # the logits are multiplied by it
    logit_softcap: float | None = None    # then logits = cap * tanh(logits / cap)

    def __post_init__(self) -> None:
        if not self.layers or not self.order:
            raise ValueError("a model needs at least one layer and one call")
        owners: dict[int, int] = {}
        for index, call in enumerate(self.order):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"order[{index}] names layer {call.layer}, model has {len(self.layers)}")
            if call.writes_cache:
                if call.cache_slot in owners:
                    raise ValueError(f"cache slot {call.cache_slot} is written by two calls")
                owners[call.cache_slot] = index
            elif call.cache_slot not in owners:
                raise ValueError(f"order[{index}] reads cache slot {call.cache_slot} before any call wrote it")
        if sorted(owners) != list(range(len(owners))):
            raise ValueError("cache slots must be numbered 0..n-1 without gaps")

    @property
    def num_cache_slots(self) -> int:
        return sum(1 for call in self.order if call.writes_cache)

    def slot_owner(self, slot: int) -> LayerCall:
        for call in self.order:
            if call.writes_cache and call.cache_slot == slot:
                return call
        raise KeyError(slot)
