"""Grouped-query attention over the paged cache.

Formulas of the reference (worker/src/inference/qwen2/model.py:138-225):
``q, k, v = x Wq^T + bq, ...``; rotation of q and k; the new k and v are stored
in their pages before anything is read (worker/src/inference/qwen2/paged_attn.py:
388-389); query head ``h`` reads kv head ``h // (heads / kv_heads)``; scores scaled
by ``head_dim**-0.5``; a token at position ``p`` sees keys ``<= p`` (and, with a
window ``w``, ``> p - w``); softmax in float32; output projection.

The three projections are one product against the row-stacked weight; rotation
and cache write are one kernel; attention reads q from the same buffer.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import MIXERS, POSITION_ENCODINGS, BuildContext, CacheNeed, LayerRun, TensorSpec, build_part
from .linear import Linear, fuse_rows


@MIXERS.register("gqa_attention")
class GqaAttention:
    """params: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``qkv_bias``, ``out_bias``,
    ``window`` (None: full), ``scale`` (None: ``head_dim**-0.5``), ``position`` (a PartSpec).

    tensors: ``q_proj``/``k_proj``/``v_proj``/``o_proj`` ``.weight`` (and ``.bias``).
    """

    def __init__(self, qkv: Linear, out: Linear, position, params: dict, kernels) -> None:
        self.qkv = qkv
        self.out = out
        self.position = position
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.window = params.get("window")
        self.scale = float(params.get("scale") or self.head_dim**-0.5)
        self.kernels = kernels

    # -- declarations -------------------------------------------------------
    @staticmethod
    def _check(params) -> None:
        heads, kv_heads, dim = int(params["num_heads"]), int(params["num_kv_heads"]), int(params["head_dim"])
        if heads < 1 or kv_heads < 1 or heads % kv_heads:
            raise ValueError(f"num_heads ({heads}) must be a positive multiple of num_kv_heads ({kv_heads})")
        if dim < 16 or dim % 16 or dim > 256:
            raise ValueError(f"head_dim {dim}: the attention kernels take multiples of 16 from 16 to 256")
        window = params.get("window")
        if window is not None and int(window) < 1:
            raise ValueError(f"window must be >= 1, got {window}")

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        cls._check(spec.params)
        p, prm = spec.prefix, spec.params
        q_out = prm["num_heads"] * prm["head_dim"]
        kv_out = prm["num_kv_heads"] * prm["head_dim"]
        specs = [
            TensorSpec(p + "q_proj.weight", (q_out, hidden_size)),
            TensorSpec(p + "k_proj.weight", (kv_out, hidden_size)),
            TensorSpec(p + "v_proj.weight", (kv_out, hidden_size)),
            TensorSpec(p + "o_proj.weight", (hidden_size, q_out)),
        ]
        if prm.get("qkv_bias", False):
            specs += [
                TensorSpec(p + "q_proj.bias", (q_out,), "bias"),
                TensorSpec(p + "k_proj.bias", (kv_out,), "bias"),
                TensorSpec(p + "v_proj.bias", (kv_out,), "bias"),
            ]
        if prm.get("out_bias", False):
            specs.append(TensorSpec(p + "o_proj.bias", (hidden_size,), "bias"))
        return specs

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        prm = spec.params
        return CacheNeed(int(prm["num_kv_heads"]), int(prm["head_dim"]), prm.get("window"))

    @classmethod
    def state_need(cls, spec: PartSpec):
        return None

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "GqaAttention":
        cls._check(spec.params)
        p, prm, w = spec.prefix, spec.params, ctx.weights
        weight = fuse_rows([w.matrix(p + f"{n}_proj.weight") for n in "qkv"])
        bias = fuse_rows([w.vector(p + f"{n}_proj.bias") for n in "qkv"]) if prm.get("qkv_bias", False) else None
        out_bias = w.vector(p + "o_proj.bias") if prm.get("out_bias", False) else None
        position = build_part(POSITION_ENCODINGS, prm["position"], ctx)
        return cls(
            Linear(weight, bias, ctx.kernels),
            Linear(w.matrix(p + "o_proj.weight"), out_bias, ctx.kernels),
            position,
            dict(prm),
            ctx.kernels,
        )

    # -- the step -----------------------------------------------------------
    def forward(self, x: torch.Tensor, run: LayerRun) -> torch.Tensor:
        if run.kv is None:
            raise RuntimeError("attention needs a cache slot")
        k = self.kernels
        mixed = torch.empty((x.shape[0], self.num_heads * self.head_dim), dtype=x.dtype, device=x.device)
        table = self.position.rotary_table()
        if table is None and hasattr(self.position, "apply"):
            # An encoding of its own: the projection is finished here, the encoding changes q and k in
            # place, and the fused kernel only stores k and v and copies q out.
            q = torch.empty_like(mixed)
            qkv = k.linear(x, self.qkv.weight, self.qkv.bias)
            self.position.apply(qkv, run.step, self.num_heads, self.num_kv_heads, self.head_dim)
            k.rope_kv_write(qkv, run.step, run.kv if run.writes_cache else None, None, self.num_heads,
                            self.num_kv_heads, self.head_dim, q_out=q)
            k.attention(q, mixed, run.step, run.kv, self.num_heads, self.num_kv_heads, self.head_dim, self.window, self.scale)
        else:
            # The projection, the bias, the rotation of q and k, the store of k and v in their pages and the
            # attention over the pages as one op of the kernel set, which may merge kernels for some steps.
            k.qkv_attention(x, self.qkv.weight, self.qkv.bias, run.step, run.kv, run.writes_cache, table,
                            self.num_heads, self.num_kv_heads, self.head_dim, self.window, self.scale, mixed)
        if self.out.bias is not None:
            return self.out(mixed)
        return k.linear_split(mixed, self.out.weight)  # summed by the norm that follows
