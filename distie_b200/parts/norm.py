"""RMSNorm: float32 statistics, the weight applied after the cast back.

Formula of the reference (worker/src/inference/qwen2/model.py:85-90).  The part
also does the residual sum that precedes it, in the same kernel.
"""

from __future__ import annotations

from ..config.model_spec import PartSpec
from .base import NORMS, BuildContext, TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm:
    """params: ``eps``.  tensors: ``<prefix>weight [hidden]``."""

    def __init__(self, weight, eps: float, kernels) -> None:
        self.weight = weight
        self.eps = float(eps)
        self.kernels = kernels

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        return [TensorSpec(spec.prefix + "weight", (hidden_size,), "norm")]

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "RMSNorm":
        return cls(ctx.weights.vector(spec.prefix + "weight"), spec.params["eps"], ctx.kernels)

    def apply(self, delta, residual, out, rows=None) -> None:
        """``residual += delta`` (if any), ``out = norm(residual)``; with ``rows`` only those rows, residual kept."""
        self.kernels.add_rmsnorm(delta, residual, self.weight, self.eps, out, rows)
