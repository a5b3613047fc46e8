"""Arrangements of parts in a block.

``pre_norm``: the reference's decoder layer (worker/src/inference/qwen2/model.py:
247-249): ``h += mixer(norm_in(h))``; ``h += ff(norm_post(h))``.  The sums are
float32 and are done by the norm kernel that follows them, so a block leaves its
feed-forward output pending on the stream.
"""

from __future__ import annotations

import torch

from ..config.model_spec import LayerSpec
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, BuildContext, LayerRun, ResidualStream, TensorSpec, build_part


@BLOCKS.register("pre_norm")
class PreNormBlock:
    """norms: ``input`` (before the mixer) and ``post_mixer`` (before the feed-forward)."""

    def __init__(self, norm_in, mixer, norm_post, feed_forward, dtype) -> None:
        self.norm_in = norm_in
        self.mixer = mixer
        self.norm_post = norm_post
        self.feed_forward = feed_forward
        self.dtype = dtype

    @property
    def graph_safe(self) -> bool:
        """False when a part reads host-side batch data, which a captured step cannot replay."""
        return all(getattr(part, "graph_safe", True) for part in (self.mixer, self.feed_forward))

    @classmethod
    def tensor_specs(cls, layer: LayerSpec, hidden_size: int) -> list[TensorSpec]:
        return (
            NORMS.get(layer.norms["input"].kind).tensor_specs(layer.norms["input"], hidden_size)
            + MIXERS.get(layer.mixer.kind).tensor_specs(layer.mixer, hidden_size)
            + NORMS.get(layer.norms["post_mixer"].kind).tensor_specs(layer.norms["post_mixer"], hidden_size)
            + FEED_FORWARDS.get(layer.feed_forward.kind).tensor_specs(layer.feed_forward, hidden_size)
        )

    @classmethod
    def build(cls, layer: LayerSpec, ctx: BuildContext) -> "PreNormBlock":
        return cls(
            build_part(NORMS, layer.norms["input"], ctx),
            build_part(MIXERS, layer.mixer, ctx),
            build_part(NORMS, layer.norms["post_mixer"], ctx),
            build_part(FEED_FORWARDS, layer.feed_forward, ctx),
            ctx.dtype,
        )

    def forward(self, stream: ResidualStream, run: LayerRun) -> None:
        residual = stream.residual
        x = torch.empty(residual.shape, dtype=self.dtype, device=residual.device)
        self.norm_in.apply(stream.pending, residual, x)
        mixed = self.mixer.forward(x, run)
        self.norm_post.apply(mixed, residual, x)
        stream.pending = self.feed_forward.forward(x, run)
