"""The set of operations the parts are written against.

Parts never call a kernel by name; they are handed a :class:`KernelSet` when they
are built.  The engine has two of them, both in :mod:`distie_b200.kernels.device`:
the bfloat16 set that serving uses and the float32 set in which every product,
sum and exponential is a true 32-bit operation.  Tests pass a third, written with
plain tensor operations, to check each kernel against and to run the engine's
bookkeeping on a machine without a GPU; the product never falls back to it.

Shapes (``T`` tokens of this step, ``B`` requests of this step):

``StepTensors``   the step's metadata on the device, all int32
    token_ids [T], positions [T], token_seq [T] (batch row of each token),
    seq_seat [B] (seat = row of the block tables and of the state slots).
``KvSlot``        one cache slot of one group
    k, v  [pages, kv_heads, page_size, head_dim]; block_table [seats, width] int32
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass, field

import torch


Q_TILE = 128  # tokens per tile of StepTensors.q_tiles


@dataclass
class StepTensors:
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_seq: torch.Tensor
    seq_seat: torch.Tensor
    num_tokens: int
    num_seqs: int
    num_decode_tokens: int  # the first this-many tokens are single-token rows
    max_kv_len: int = 0  # bound on the keys any token sees; a captured step uses a fixed bound
    q_tiles: torch.Tensor | None = None  # [n, 2] int32: (first token, rows <= Q_TILE) of each tile of the
    num_q_tiles: int = 0                 # multi-token entries; a tile holds consecutive tokens of one request
    derived: dict = field(default_factory=dict)  # what a kernel set made of this step once and its layers share


@dataclass
class KvSlot:
    k: torch.Tensor
    v: torch.Tensor
    block_table: torch.Tensor
    page_size: int
    num_pages: int


@dataclass(frozen=True)
class RotaryTable:
    """What the fused rotation kernel needs of a rotary position encoding."""

    inv_freq: torch.Tensor  # [rotary_dim / 2] float32
    rotary_dim: int
    interleaved: bool = False
    factor: float = 1.0  # cos and sin are multiplied by it (the attention factor of scaled rotary encodings)


class KernelSet(ABC):
    dtype: torch.dtype
    device: torch.device

    @abstractmethod
    def embed(self, step: StepTensors, table: torch.Tensor, residual: torch.Tensor) -> None:
        """residual[t] = table[token_ids[t]] as float32."""

    @abstractmethod
    def add_rmsnorm(self, delta, residual, weight, eps: float, out, rows_index=None) -> None:
        """residual += delta (float32, kept), out = weight * cast(residual * rsqrt(mean sq + eps)).

        ``delta`` is ``[T, hidden]`` in the set's dtype, or ``[S, T, hidden]`` float32 slices as
        :meth:`linear_split` returns them, which are added up in the same kernel.
        """

    @abstractmethod
    def linear(self, x, weight, bias=None, out_dtype=None):
        """x @ weight.T (+ bias); weight is [out, in]."""

    def linear_split(self, x, weight):
        """``x @ weight.T`` as float32 slices ``[S, T, out]`` whose sum over ``S`` is the product.

        A set that splits the reduction of a skinny product over several thread blocks returns
        the slices as they are and leaves the sum to the consumer (``add_rmsnorm``,
        ``rope_kv_write``), which saves the product a round of synchronisation.  The default is
        one slice.
        """
        return self.linear(x, weight, None, torch.float32).unsqueeze(0)

    @abstractmethod
    def swiglu(self, gate_up, out) -> None:
        """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""

    def linear_swiglu(self, x, weight):
        """silu(x Wg^T) * (x Wu^T) for weight = [Wg; Wu] stacked along the rows; sets may fuse it."""
        gate_up = self.linear(x, weight)
        out = torch.empty((x.shape[0], weight.shape[0] // 2), dtype=gate_up.dtype, device=x.device)
        self.swiglu(gate_up, out)
        return out

    @abstractmethod
    def rope_kv_write(self, qkv, step: StepTensors, kv: KvSlot | None, rotary: RotaryTable | None,
                      num_heads: int, num_kv_heads: int, head_dim: int, bias=None, q_out=None) -> None:
        """Rotate q and k, store k and v of the new tokens in their pages (if kv).

        ``qkv`` is ``[T, (heads + 2 kv_heads) * head_dim]`` in the set's dtype with q rotated in
        place, or float32 slices ``[S, T, ...]`` of the projection (see :meth:`linear_split`), in
        which case the slices are summed, ``bias`` is added and the rotated q is written to
        ``q_out [T, heads * head_dim]``.
        """

    def qkv_rope_write(self, x, weight, bias, step: StepTensors, kv: KvSlot | None, rotary: RotaryTable | None,
                       num_heads: int, num_kv_heads: int, head_dim: int, q_out) -> None:
        """The q/k/v projection with what follows it: ``x @ weight.T + bias``, q and k rotated, q to
        ``q_out`` and k and v into their pages (if kv).  The default is the two ops after one another;
        a set may do it in the product's epilogue."""
        slices = self.linear_split(x, weight)
        self.rope_kv_write(slices, step, kv, rotary, num_heads, num_kv_heads, head_dim, bias=bias, q_out=q_out)

    def qkv_attention(self, x, weight, bias, step: StepTensors, kv: KvSlot, writes_cache: bool,
                      rotary: RotaryTable | None, num_heads: int, num_kv_heads: int, head_dim: int,
                      window: int | None, scale: float, out) -> None:
        """From the mixer's input to the attention's output: the q/k/v projection, bias, rotation, the new
        keys and values into their pages (if ``writes_cache``) and attention over the pages into ``out``.
        The default is the ops after one another; a set may merge them for some steps."""
        q = torch.empty((x.shape[0], num_heads * head_dim), dtype=out.dtype, device=x.device)
        self.qkv_rope_write(x, weight, bias, step, kv if writes_cache else None, rotary, num_heads, num_kv_heads,
                            head_dim, q)
        self.attention(q, out, step, kv, num_heads, num_kv_heads, head_dim, window, scale)

    @abstractmethod
    def attention(self, qkv, out, step: StepTensors, kv: KvSlot, num_heads: int, num_kv_heads: int,
                  head_dim: int, window: int | None, scale: float) -> None:
        """Causal (optionally windowed) attention of every token over its request's pages."""

    @abstractmethod
    def sample(self, logits, temperatures, uniforms, out_tokens) -> None:
        """Arg-max for rows with temperature <= 0, inverse-CDF draw at uniforms[row] otherwise."""

    def check_errors(self) -> None:
        """Raise if a kernel of an earlier launch reported a bad index (after a synchronise)."""
