"""A product ``x @ W.T (+ b)`` with its weight ``[out, in]``, as checkpoints store it."""

from __future__ import annotations

import torch


class Linear:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None, kernels) -> None:
        self.weight = weight
        self.bias = bias
        self.kernels = kernels

    def __call__(self, x: torch.Tensor, out_dtype=None) -> torch.Tensor:
        return self.kernels.linear(x, self.weight, self.bias, out_dtype)


def fuse_rows(pieces: list[torch.Tensor]) -> torch.Tensor:
    """Stack matrices (or biases) that share an input along the output axis.

    Pieces of different stored precision are promoted to the widest, so that a
    float32-stored piece is not rounded.
    """
    dtype = torch.float32 if any(p.dtype == torch.float32 for p in pieces) else pieces[0].dtype
    return torch.cat([p.to(dtype) for p in pieces], dim=0).contiguous()
