"""Interfaces and registries of the parts a block is put together from.

A part is built from a :class:`~distie_b200.config.model_spec.PartSpec` (its
constants and the prefix of its tensors) and a :class:`BuildContext` (the kernel
set, the hidden width, the loaded weights).  No part knows which model it is in.

============== ==============================================================
kind of part   what it must offer
============== ==============================================================
norm           ``tensor_specs``, ``build``, ``apply(delta, residual, out, rows=None)``
position       ``build``; ``rotary_table()`` for the fused kernel, or ``None``
               and an ``apply(qkv, step, ...)`` of its own
mixer          ``tensor_specs``, ``build``, ``cache_need``, ``state_need``,
               ``forward(x, run) -> delta``
feed-forward   ``tensor_specs``, ``build``, ``forward(x, run) -> delta``
block          ``tensor_specs``, ``build``, ``forward(stream, run)``
============== ==============================================================

``forward`` of a mixer or feed-forward takes the normalised activations ``[T,
hidden]`` of the step's tokens and returns what is to be added to the residual
stream: ``[T, hidden]``, or float32 slices ``[S, T, hidden]`` whose sum it is (what
``KernelSet.linear_split`` returns; the norm that follows adds them up).  The :class:`LayerRun` tells a mixer everything about the step: the
tokens' positions and requests, its cache slot and its per-request state.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Sequence

import torch

from ..config.model_spec import PartSpec
from ..kernels.interface import KernelSet, KvSlot, StepTensors


# -- what parts declare --------------------------------------------------------
@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part reads from the checkpoint.  ``role`` decides conversion and random init:

    ``matrix``  2-D weight of a product (engine dtype; a float32-stored one stays float32)
    ``table``   embedding table (like ``matrix``)
    ``bias``    vector added to a product (kept in float32 on the device)
    ``norm``    scale of a norm (float32 on the device; random mode writes ones)
    """

    name: str
    shape: tuple[int, ...]
    role: str = "matrix"


@dataclass(frozen=True)
class CacheNeed:
    """Keys and values in pages.  Layers with equal needs share a group (pool, tables)."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None  # None: every key is kept; n: only the last n positions are read


@dataclass(frozen=True)
class StateNeed:
    """State of fixed size per request (one slot per seat), zeroed when a request starts."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


# -- what parts are given ------------------------------------------------------
@dataclass
class BuildContext:
    kernels: KernelSet
    hidden_size: int
    weights: Any  # distie_b200.weights.loader.WeightStore

    @property
    def dtype(self) -> torch.dtype:
        return self.kernels.dtype

    @property
    def device(self) -> torch.device:
        return self.kernels.device


@dataclass(frozen=True)
class SeqSlice:
    """One request's share of a step, on the host: tokens [start, start + q_len) of the batch."""

    seat: int
    start: int
    q_len: int
    past_len: int


@dataclass
class LayerRun:
    """Everything one call of the run order may look at."""

    step: StepTensors
    seqs: Sequence[SeqSlice]
    kv: KvSlot | None = None
    state: torch.Tensor | None = None  # [seats, *StateNeed.shape] of this call's slot
    writes_cache: bool = True
    extras: dict = field(default_factory=dict)


class ResidualStream:
    """The float32 residual ``[T, hidden]`` and a delta that is still to be added.

    Keeping the delta pending lets the next norm do the sum and the normalisation
    in one kernel; ``settle`` performs the sum for a consumer that wants the plain
    residual.
    """

    def __init__(self, residual: torch.Tensor, pending: torch.Tensor | None = None) -> None:
        self.residual = residual
        self.pending = pending

    def settle(self) -> torch.Tensor:
        if self.pending is not None:
            delta = self.pending.sum(0) if self.pending.dim() == 3 else self.pending  # slices of a split product
            self.residual.add_(delta.to(torch.float32))
            self.pending = None
        return self.residual


# -- registries ---------------------------------------------------------------
class Registry:
    def __init__(self, what: str) -> None:
        self.what = what
        self._kinds: dict[str, Any] = {}

    def register(self, kind: str, cls: Any = None) -> Callable | Any:
        if cls is None:
            def wrap(inner):
                self._kinds[kind] = inner
                return inner
            return wrap
        self._kinds[kind] = cls
        return cls

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def get(self, kind: str) -> Any:
        try:
            return self._kinds[kind]
        except KeyError:
            raise KeyError(f"unknown {self.what} {kind!r}; registered: {', '.join(sorted(self._kinds))}") from None

    def kinds(self) -> tuple[str, ...]:
        return tuple(sorted(self._kinds))


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block arrangement")


def build_part(registry: Registry, spec: PartSpec, ctx: BuildContext):
    return registry.get(spec.kind).build(spec, ctx)
