"""SwiGLU feed-forward, dense: ``down(silu(gate(x)) * up(x))``, no biases.

Formula of the reference (worker/src/inference/qwen2/model.py:228-236).  Gate and
up are one product against the row-stacked weight ``[2 * inter, hidden]``.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import FEED_FORWARDS, BuildContext, LayerRun, TensorSpec
from .linear import Linear, fuse_rows


@FEED_FORWARDS.register("swiglu")
class SwiGluFeedForward:
    """params: ``intermediate_size``.  tensors: ``gate_proj``/``up_proj``/``down_proj`` ``.weight``."""

    def __init__(self, gate_up: Linear, down: Linear, inter: int, kernels) -> None:
        self.gate_up = gate_up
        self.down = down
        self.inter = inter
        self.kernels = kernels

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        p, inter = spec.prefix, int(spec.params["intermediate_size"])
        return [
            TensorSpec(p + "gate_proj.weight", (inter, hidden_size)),
            TensorSpec(p + "up_proj.weight", (inter, hidden_size)),
            TensorSpec(p + "down_proj.weight", (hidden_size, inter)),
        ]

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "SwiGluFeedForward":
        p, w = spec.prefix, ctx.weights
        gate_up = fuse_rows([w.matrix(p + "gate_proj.weight"), w.matrix(p + "up_proj.weight")])
        return cls(
            Linear(gate_up, None, ctx.kernels),
            Linear(w.matrix(p + "down_proj.weight"), None, ctx.kernels),
            int(spec.params["intermediate_size"]),
            ctx.kernels,
        )

    def forward(self, x: torch.Tensor, run: LayerRun) -> torch.Tensor:
        # The down product's float32 slices are summed by the norm that follows (or by the stream).
        return self.kernels.linear_split(self.kernels.linear_swiglu(x, self.gate_up.weight), self.down.weight)
