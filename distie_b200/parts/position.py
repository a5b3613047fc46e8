"""Position encodings.  A mixer is given one as a parameter.

``rotary``: the reference's default RoPE (worker/src/inference/qwen2/model.py:93-117):
``inv_freq[j] = 1 / theta**(2j / d)`` computed in float32 exactly as there, angles
``pos * inv_freq`` and their cos/sin evaluated in float32 inside the fused kernel,
pairs ``(j, j + d/2)`` (rotate-half).  ``rotary_dim < head_dim``, interleaved pairs and
a factor on cos and sin are parameters for other layer kinds.  ``none`` rotates nothing.

An encoding that is no table of frequencies (learned or additive positions, a rotation
that depends on more than the position) returns ``None`` from ``rotary_table()`` and
offers ``apply(qkv, step, num_heads, num_kv_heads, head_dim)`` instead: the mixer finishes
its projection, hands ``qkv [T, (heads + 2 kv_heads) * head_dim]`` over to be changed in
place, and the fused kernel then only stores the keys and values.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..kernels.interface import RotaryTable
from .base import POSITION_ENCODINGS, BuildContext


# Layers with the same parameters share one table (and one tensor of frequencies): what a kernel set derives
# from a table and a step's positions is then made once per step, not once per layer.
_TABLES: dict[tuple, RotaryTable] = {}


@POSITION_ENCODINGS.register("rotary")
class RotaryEncoding:
    """params: ``head_dim``, ``theta``, optional ``rotary_dim``, ``interleaved``, ``factor``."""

    def __init__(self, table: RotaryTable) -> None:
        self._table = table

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "RotaryEncoding":
        head_dim = int(spec.params["head_dim"])
        rotary_dim = int(spec.params.get("rotary_dim") or head_dim)
        theta = float(spec.params["theta"])
        if rotary_dim % 2 or rotary_dim > head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        key = (theta, rotary_dim, bool(spec.params.get("interleaved", False)), float(spec.params.get("factor", 1.0)),
               str(ctx.device))
        table = _TABLES.get(key)
        if table is None:
            inv_freq = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))
            table = _TABLES[key] = RotaryTable(inv_freq.to(ctx.device), *key[1:4])
        return cls(table)

    def rotary_table(self) -> RotaryTable | None:
        return self._table


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding:
    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "NoPositionEncoding":
        return cls()

    def rotary_table(self) -> RotaryTable | None:
        return None
