"""The two kernel sets of the product: bfloat16 (serving) and float32 (true 32-bit).

Both drive the same hand-written launchers with a dtype code; they differ in the
element type of activations, weights and cache, and in the matrix products:

* bfloat16: products with float32 accumulation.  Plain ``x @ W.T`` goes to the
  library (cuBLAS through ``torch.mm``), as the reference's engine does for every
  product (worker/src/inference/qwen2/model.py:216-236); skinny and fused
  products use this package's own kernels where they are registered.
* float32: ``torch.mm`` with TF32 switched off, i.e. FMA-only float32 products;
  accurate ``expf``/``sincosf``/``rsqrtf`` in every kernel.

There is no CPU path here and no fallback: a missing library raises.
"""

from __future__ import annotations

import torch

from . import library
from .interface import KernelSet, StepTensors
from .library import KernelError, check, function

_CODE = {torch.float32: 0, torch.bfloat16: 1}
_DECODE_HEAD_DIMS = (16, 32, 64, 128, 256)
_PREFILL_HEAD_DIMS = (64, 128)  # tensor-core attention for portions of prompts (bfloat16)
_SKINNY_ROWS = 64               # weight-streaming products (tcgen05, weights as the 128-row operand) take up to 64 rows
_CLUSTER_SPLITS = 8             # splits of a decode attention that one cluster of CTAs merges itself
_TENSOR_CORE_ROWS = 128         # from here on the tcgen05 kernel's 128-row tiles are full; in between: the library

_ERROR_TEXT = {
    1: "a token id outside the vocabulary reached the embedding",
    2: "a new token's page is missing from its block table (cache write)",
    3: "a block table does not cover the keys a token attends to",
    4: "a block table does not cover the keys a decoded token attends to",
    6: "a tensor-core product gave up waiting for its own copies or instructions",
    5: "a block table does not cover the keys a portion of a prompt attends to",
}


class DeviceKernels(KernelSet):
    def __init__(self, dtype: torch.dtype, device: torch.device | str = "cuda:0") -> None:
        if dtype not in _CODE:
            raise KernelError(f"no kernel set for dtype {dtype}; the engine runs bfloat16 or float32")
        self.dtype = dtype
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise KernelError("distie_b200 runs on a CUDA device (sm_100a) only; no GPU is visible")
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise KernelError(f"kernels are built for sm_100a; device reports sm_{major}{minor}")
        self.code = _CODE[dtype]
        if dtype == torch.float32:
            # True 32-bit products: no TF32, no reduced-precision reductions.
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
            torch.set_float32_matmul_precision("highest")
        library.load_unit("base")
        if dtype == torch.bfloat16:
            library.load_unit("bf16")
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.launches = 0  # own kernels launched (library products are not counted)
        self.kernel_counts: dict[str, int] = {}  # the same, by launcher

    # -- helpers ------------------------------------------------------------
    @staticmethod
    def _stream() -> int:
        return torch.cuda.current_stream().cuda_stream

    def _ran(self, name: str, kernels: int = 1) -> None:
        self.launches += kernels
        self.kernel_counts[name] = self.kernel_counts.get(name, 0) + 1

    def check_errors(self) -> None:
        code = int(self.error_flag.item())
        if code:
            self.error_flag.zero_()
            raise KernelError(f"device-side check failed: {_ERROR_TEXT.get(code, code)}")

    # -- operations -----------------------------------------------------------
    def embed(self, step: StepTensors, table: torch.Tensor, residual: torch.Tensor) -> None:
        hidden = table.shape[1]
        check(
            function("distie_embed")(
                step.token_ids.data_ptr(), table.data_ptr(), residual.data_ptr(), step.num_tokens, hidden,
                table.shape[0], _CODE[table.dtype], self.error_flag.data_ptr(), self._stream(),
            ),
            "embed",
        )
        self._ran("embed")

    def add_rmsnorm(self, delta, residual, weight, eps, out, rows_index=None) -> None:
        rows = out.shape[0]
        rows_ptr = rows_index.data_ptr() if rows_index is not None else None
        if delta is not None and delta.dim() == 3:
            code = function("distie_add_rmsnorm_split")(
                delta.data_ptr(), delta.shape[0], delta.stride(0), residual.data_ptr(), weight.data_ptr(),
                out.data_ptr(), rows_ptr, rows, residual.shape[1], float(eps), self.code, self._stream(),
            )
            if code == 0:
                self._ran("add_rmsnorm_split")
                return
            if code != -2:
                check(code, "add_rmsnorm_split")
            # A width the fused kernel refuses: add the slices up here, in float32.
            summed = delta[0] if delta.shape[0] == 1 else delta.sum(0)
            if rows_index is None:
                residual.add_(summed)
                delta = None
            else:
                index = rows_index.long()
                residual, delta, rows_ptr = residual.index_select(0, index) + summed.index_select(0, index), None, None
        check(
            function("distie_add_rmsnorm")(
                delta.data_ptr() if delta is not None else None, residual.data_ptr(), weight.data_ptr(),
                out.data_ptr(), rows_ptr, rows, residual.shape[1], float(eps), self.code, self._stream(),
            ),
            "add_rmsnorm",
        )
        self._ran("add_rmsnorm")

    def linear_split(self, x, weight):
        if self._skinny(x, weight):
            m, n, k = x.shape[0], weight.shape[0], weight.shape[1]
            splits = function("distie_gemm_tcgen05_skinny_splits")(n, k, self.sm_count)
            out = torch.empty((splits, m, n), dtype=torch.float32, device=x.device)
            self._stream_weights(x, weight, None, out, 0)
            return out
        return super().linear_split(x, weight)

    def linear(self, x, weight, bias=None, out_dtype=None):
        out_dtype = out_dtype or self.dtype
        if weight.dtype == torch.float32:
            # float32 engine, or a matrix the checkpoint stores in 32-bit: a true float32 product.
            x32 = x if x.dtype == torch.float32 else x.float()
            y = torch.addmm(bias, x32, weight.t()) if bias is not None else torch.mm(x32, weight.t())
            return y if out_dtype == torch.float32 else self._bias_cast(y, None, out_dtype)
        if self._skinny(x, weight):
            out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
            self._stream_weights(x, weight, bias, out, 1)
            return out
        if self._tensor_core(x, weight) and (bias is None or out_dtype == torch.float32) and not self._underfilled(x, weight):
            out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
            self._gemm_tcgen05(x, weight, out, 1 if out_dtype == torch.float32 else 0)
            return out if bias is None else out.add_(bias)
        if bias is None and out_dtype == self.dtype:
            return torch.mm(x, weight.t())
        y32 = torch.mm(x, weight.t(), out_dtype=torch.float32)
        if out_dtype == torch.float32:
            return y32 if bias is None else y32.add_(bias)
        return self._bias_cast(y32, bias, out_dtype)

    def _tensor_core(self, x, weight) -> bool:
        """Products of more rows than the weight-streaming kernel takes: the tcgen05 kernel."""
        return (
            self.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
            and x.shape[0] >= _TENSOR_CORE_ROWS and weight.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and x.stride(1) == 1 and weight.is_contiguous()
        )

    def _underfilled(self, x, weight) -> bool:
        """A long-K product whose 256 x 256 tiles would leave most of the machine idle (a few hundred rows against
        a narrow weight, e.g. the down projection of a short portion): the library splits K over the idle SMs and
        is up to twice as fast there (measured at 256 to 1,024 rows of the 1.5B, 7B and 14B down projections)."""
        rows, n, k = x.shape[0], weight.shape[0], weight.shape[1]
        tiles = -(-rows // 256) * -(-n // 256)
        return k >= 4096 and tiles < 0.7 * (self.sm_count // 2)

    def _gemm_tcgen05(self, x, weight, out, epi: int, tile_width: int = 0) -> None:
        check(
            function("distie_gemm_tcgen05")(
                x.data_ptr(), x.stride(0), weight.data_ptr(), out.data_ptr(), out.stride(0), x.shape[0],
                weight.shape[0], weight.shape[1], epi, tile_width, self.sm_count, self.error_flag.data_ptr(),
                self._stream(),
            ),
            "gemm_tcgen05",
        )
        self._ran("gemm_tcgen05")

    def _skinny(self, x, weight) -> bool:
        return (
            self.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
            and x.shape[0] <= _SKINNY_ROWS and weight.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1
            and weight.is_contiguous()
        )

    def _stream_weights(self, x, weight, bias, out, mode: int) -> None:
        """mode 0: float32 slices; 1: x W^T + bias; 2: fused SwiGLU (see gemm_tcgen05.cu)."""
        check(
            function("distie_gemm_tcgen05_skinny")(
                x.data_ptr(), x.stride(0), weight.data_ptr(), bias.data_ptr() if bias is not None else None,
                out.data_ptr(), out.stride(-2), x.shape[0], weight.shape[0], weight.shape[1], mode,
                _CODE.get(out.dtype, 0), self.sm_count, self.error_flag.data_ptr(), self._stream(),
            ),
            "gemm_tcgen05_skinny",
        )
        self._ran("gemm_tcgen05_skinny")

    def linear_swiglu(self, x, weight):
        if self._skinny(x, weight) and weight.shape[0] % 2 == 0:
            out = torch.empty((x.shape[0], weight.shape[0] // 2), dtype=self.dtype, device=x.device)
            self._stream_weights(x, weight, None, out, 2)
            return out
        if self._tensor_core(x, weight) and weight.shape[0] % 2 == 0:
            out = torch.empty((x.shape[0], weight.shape[0] // 2), dtype=self.dtype, device=x.device)
            self._gemm_tcgen05(x, weight, out, 2)
            return out
        return super().linear_swiglu(x, weight)

    def _bias_cast(self, y32, bias, out_dtype):
        out = torch.empty(y32.shape, dtype=out_dtype, device=y32.device)
        check(
            function("distie_bias_cast")(
                y32.data_ptr(), bias.data_ptr() if bias is not None else None, out.data_ptr(), y32.shape[0],
                y32.shape[1], _CODE[out_dtype], self._stream(),
            ),
            "bias_cast",
        )
        self._ran("bias_cast")
        return out

    def swiglu(self, gate_up, out) -> None:
        check(
            function("distie_swiglu")(
                gate_up.data_ptr(), out.data_ptr(), gate_up.shape[0], out.shape[1], self.code, self._stream()
            ),
            "swiglu",
        )
        self._ran("swiglu")

    def rope_kv_write(self, qkv, step, kv, rotary, num_heads, num_kv_heads, head_dim, bias=None, q_out=None) -> None:
        write = kv is not None
        table = kv.block_table if write else step.seq_seat  # any valid pointer when nothing is written
        tail = [
            step.positions.data_ptr(), step.token_seq.data_ptr(), step.seq_seat.data_ptr(),
            table.data_ptr(), table.shape[-1] if write else 1,
            rotary.inv_freq.data_ptr() if rotary is not None else None,
            float(rotary.factor) if rotary is not None else 1.0,
            kv.k.data_ptr() if write else None, kv.v.data_ptr() if write else None,
        ]
        sizes = [
            num_heads, num_kv_heads, head_dim,
            rotary.rotary_dim if rotary is not None else 0,
            int(rotary.interleaved) if rotary is not None else 0,
            kv.page_size if write else 1, kv.num_pages if write else 1, int(write), self.code,
            self.error_flag.data_ptr(), self._stream(),
        ]
        if qkv.dim() == 3:
            if q_out is None:
                raise KernelError("rope_kv_write: slices of a projection need a q_out buffer")
            code = function("distie_rope_kv_write_split")(
                qkv.data_ptr(), qkv.shape[0], qkv.stride(0), qkv.stride(1),
                bias.data_ptr() if bias is not None else None, q_out.data_ptr(), q_out.stride(0),
                *tail, step.num_tokens, *sizes,
            )
            if code == 0:
                self._ran("rope_kv_write_split")
                return
            if code != -2:
                check(code, "rope_kv_write_split")
            # Sizes the fused kernel refuses: finish the projection here, rotate in place, copy q out.
            summed = qkv[0] if qkv.shape[0] == 1 else qkv.sum(0)
            if bias is not None:
                summed = summed + bias
            dense = summed.to(self.dtype)
            self.rope_kv_write(dense, step, kv, rotary, num_heads, num_kv_heads, head_dim)
            q_out.copy_(dense[:, : num_heads * head_dim])
            return
        check(
            function("distie_rope_kv_write")(qkv.data_ptr(), *tail, step.num_tokens, qkv.stride(0), *sizes),
            "rope_kv_write",
        )
        self._ran("rope_kv_write")
        if q_out is not None:
            q_out.copy_(qkv[:, : num_heads * head_dim])

    def qkv_rope_write(self, x, weight, bias, step, kv, rotary, num_heads, num_kv_heads, head_dim, q_out) -> None:
        """Prompt portions of 128 rows and more: bias, rotation and the stores of q, k and v happen in the
        epilogue of the tcgen05 product, which reads the step's angles and cache rows from a table made once
        per step.  Everything else: the product's float32 slices into the rotation kernel."""
        fused = (
            self._tensor_core(x, weight) and head_dim in (64, 128)
            and weight.shape[0] == (num_heads + 2 * num_kv_heads) * head_dim
            and (rotary is None or (rotary.rotary_dim == head_dim and not rotary.interleaved))
            and (bias is None or bias.dtype == torch.float32)
            and (kv is None or kv.k.dtype == torch.bfloat16)
            and q_out.dtype == torch.bfloat16 and q_out.stride(1) == 1 and q_out.stride(0) % 8 == 0
            and not self._underfilled(x, weight)
        )
        if not fused:
            return super().qkv_rope_write(x, weight, bias, step, kv, rotary, num_heads, num_kv_heads, head_dim, q_out)
        trig, cache_row = self._rope_rows(step, kv, rotary, num_kv_heads, head_dim)
        check(
            function("distie_gemm_tcgen05_qkv")(
                x.data_ptr(), x.stride(0), weight.data_ptr(), bias.data_ptr() if bias is not None else None,
                trig.data_ptr(), cache_row.data_ptr() if cache_row is not None else None, q_out.data_ptr(),
                q_out.stride(0), kv.k.data_ptr() if kv is not None else None, kv.v.data_ptr() if kv is not None else None,
                x.shape[0], weight.shape[0], weight.shape[1], num_heads, num_kv_heads, head_dim,
                kv.page_size if kv is not None else 1, self.sm_count, self.error_flag.data_ptr(), self._stream(),
            ),
            "gemm_tcgen05_qkv",
        )
        self._ran("gemm_tcgen05_qkv")

    def _rope_rows(self, step, kv, rotary, num_kv_heads: int, head_dim: int):
        """(trig [T, head_dim] float32, cache_row [T] int32 or None) of this step: made by the first layer that
        asks and kept with the step for the others of its cache group and encoding."""
        key = (
            "rope_rows", head_dim, num_kv_heads, kv.block_table.data_ptr() if kv is not None else 0,
            rotary.inv_freq.data_ptr() if rotary is not None else 0, float(rotary.factor) if rotary is not None else 1.0,
        )
        made = step.derived.get(key)
        if made is None:
            trig = torch.empty((step.num_tokens, head_dim), dtype=torch.float32, device=self.device)
            cache_row = torch.empty(step.num_tokens, dtype=torch.int32, device=self.device) if kv is not None else None
            check(
                function("distie_rope_rows")(
                    step.positions.data_ptr(), step.token_seq.data_ptr(), step.seq_seat.data_ptr(),
                    kv.block_table.data_ptr() if kv is not None else None, kv.block_table.shape[-1] if kv is not None else 1,
                    rotary.inv_freq.data_ptr() if rotary is not None else None,
                    float(rotary.factor) if rotary is not None else 1.0, step.num_tokens, head_dim, num_kv_heads,
                    kv.page_size if kv is not None else 1, kv.num_pages if kv is not None else 1, trig.data_ptr(),
                    cache_row.data_ptr() if cache_row is not None else None, self.error_flag.data_ptr(), self._stream(),
                ),
                "rope_rows",
            )
            self._ran("rope_rows")
            made = step.derived[key] = (trig, cache_row)
        return made

    def plan_splits(self, tokens: int, num_heads: int, num_kv_heads: int, max_kv_len: int) -> int:
        group = num_heads // num_kv_heads
        chunks = (group + 7) // 8 if group > 8 else 1
        blocks = max(1, tokens * num_kv_heads * chunks)
        by_machine = max(1, 2 * self.sm_count // blocks)  # two CTAs fit an SM; a second wave would wait for the first
        by_length = max(1, max_kv_len // 256)
        return max(1, min(by_machine, by_length, 64))

    def qkv_attention(self, x, weight, bias, step, kv, writes_cache, rotary, num_heads, num_kv_heads, head_dim,
                      window, scale, out) -> None:
        """A step of single tokens on the tensor-core kernels: the attention kernel starts from the
        projection's float32 slices itself (bias, rotation, the token's key and value into the cache and into
        its own tile), so the kernel between the projection and the attention is not launched."""
        merged = (
            step.num_decode_tokens == step.num_tokens and self.dtype == torch.bfloat16 and head_dim in _PREFILL_HEAD_DIMS
            and self._skinny(x, weight) and weight.shape[0] == (num_heads + 2 * num_kv_heads) * head_dim
            and (rotary is None or (rotary.rotary_dim == head_dim and not rotary.interleaved))
            and (bias is None or bias.dtype == torch.float32) and kv.k.dtype == torch.bfloat16
            and out.dtype == torch.bfloat16
        )
        if not merged:
            return super().qkv_attention(x, weight, bias, step, kv, writes_cache, rotary, num_heads, num_kv_heads,
                                         head_dim, window, scale, out)
        slices = self.linear_split(x, weight)
        window = int(window) if window else 0
        tokens = step.num_tokens
        splits = self.plan_splits(tokens, num_heads, num_kv_heads, step.max_kv_len)
        if splits <= 2 * _CLUSTER_SPLITS:
            splits = min(splits, _CLUSTER_SPLITS)  # merged inside the kernel, by a cluster of CTAs
        scratch = None
        if splits > _CLUSTER_SPLITS:
            floats = function("distie_attention_decode_scratch_floats")(tokens, num_heads, head_dim, splits)
            scratch = torch.empty(floats, dtype=torch.float32, device=x.device)
        check(
            function("distie_attention_decode_mma_qkv")(
                slices.data_ptr(), slices.shape[0], slices.stride(0), slices.stride(1),
                bias.data_ptr() if bias is not None else None,
                rotary.inv_freq.data_ptr() if rotary is not None else None,
                float(rotary.factor) if rotary is not None else 1.0, int(bool(writes_cache)),
                out.data_ptr(), out.stride(0), scratch.data_ptr() if scratch is not None else None,
                step.positions.data_ptr(), step.token_seq.data_ptr(), step.seq_seat.data_ptr(),
                kv.block_table.data_ptr(), kv.block_table.shape[-1], kv.k.data_ptr(), kv.v.data_ptr(), tokens,
                num_heads, num_kv_heads, head_dim, kv.page_size, kv.num_pages, window, float(scale), splits,
                self.error_flag.data_ptr(), self._stream(),
            ),
            "attention_decode_mma_qkv",
        )
        self._ran("attention_decode_mma", 1 if splits <= _CLUSTER_SPLITS else 2)
        self._ran("attention_decode_mma_qkv", 0)

    def attention(self, qkv, out, step, kv, num_heads, num_kv_heads, head_dim, window, scale) -> None:
        window = int(window) if window else 0
        n_dec = step.num_decode_tokens if head_dim in _DECODE_HEAD_DIMS else 0
        element = qkv.element_size()
        if n_dec > 0:
            splits = self.plan_splits(n_dec, num_heads, num_kv_heads, step.max_kv_len)
            tensor_cores = self.dtype == torch.bfloat16 and head_dim in _PREFILL_HEAD_DIMS
            if tensor_cores and splits <= 2 * _CLUSTER_SPLITS:
                splits = min(splits, _CLUSTER_SPLITS)  # merged inside the kernel, by a cluster of CTAs
            in_kernel_merge = splits == 1 or (tensor_cores and splits <= _CLUSTER_SPLITS)
            scratch = None
            if not in_kernel_merge:
                floats = function("distie_attention_decode_scratch_floats")(n_dec, num_heads, head_dim, splits)
                scratch = torch.empty(floats, dtype=torch.float32, device=qkv.device)
            head = [
                qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0),
                scratch.data_ptr() if scratch is not None else None, step.positions.data_ptr(),
                step.token_seq.data_ptr(), step.seq_seat.data_ptr(), kv.block_table.data_ptr(),
                kv.block_table.shape[-1], kv.k.data_ptr(), kv.v.data_ptr(), n_dec, num_heads, num_kv_heads,
                head_dim, kv.page_size, kv.num_pages, window, float(scale), splits,
            ]
            if tensor_cores:
                check(
                    function("distie_attention_decode_mma")(*head, self.error_flag.data_ptr(), self._stream()),
                    "attention_decode_mma",
                )
            else:
                check(
                    function("distie_attention_decode")(*head, self.code, self.error_flag.data_ptr(), self._stream()),
                    "attention_decode",
                )
            self._ran("attention_decode_mma" if tensor_cores else "attention_decode", 1 if in_kernel_merge else 2)
        rest = step.num_tokens - n_dec
        tiled = rest > 0 and self.dtype == torch.bfloat16 and head_dim in _PREFILL_HEAD_DIMS and step.num_q_tiles and n_dec == step.num_decode_tokens
        if tiled and self._attention_tcgen05(qkv, out, step, kv, num_heads, num_kv_heads, head_dim, window, scale):
            pass
        elif tiled:
            check(
                function("distie_attention_prefill")(
                    qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), step.q_tiles.data_ptr(),
                    step.num_q_tiles, step.positions.data_ptr(), step.token_seq.data_ptr(), step.seq_seat.data_ptr(),
                    kv.block_table.data_ptr(), kv.block_table.shape[-1], kv.k.data_ptr(), kv.v.data_ptr(), num_heads,
                    num_kv_heads, head_dim, kv.page_size, kv.num_pages, window, float(scale),
                    self.error_flag.data_ptr(), self._stream(),
                ),
                "attention_prefill",
            )
            self._ran("attention_prefill")
        elif rest > 0:
            check(
                function("distie_attention_generic")(
                    qkv.data_ptr() + n_dec * qkv.stride(0) * element, qkv.stride(0),
                    out.data_ptr() + n_dec * out.stride(0) * element, out.stride(0),
                    step.positions.data_ptr() + 4 * n_dec, step.token_seq.data_ptr() + 4 * n_dec,
                    step.seq_seat.data_ptr(), kv.block_table.data_ptr(), kv.block_table.shape[-1],
                    kv.k.data_ptr(), kv.v.data_ptr(), rest, num_heads, num_kv_heads, head_dim, kv.page_size,
                    kv.num_pages, window, float(scale), self.code, self.error_flag.data_ptr(), self._stream(),
                ),
                "attention_generic",
            )
            self._ran("attention_generic")

    def _attention_tcgen05(self, qkv, out, step, kv, num_heads, num_kv_heads, head_dim, window, scale) -> bool:
        """Prompt portions on the tcgen05 kernel; False when it refuses the page size or an alignment."""
        code = function("distie_attention_prefill_tcgen05")(
            qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), step.q_tiles.data_ptr(), step.num_q_tiles,
            step.positions.data_ptr(), step.token_seq.data_ptr(), step.seq_seat.data_ptr(),
            kv.block_table.data_ptr(), kv.block_table.shape[-1], kv.k.data_ptr(), kv.v.data_ptr(), qkv.shape[0],
            num_heads, num_kv_heads, head_dim, kv.page_size, kv.num_pages, window, float(scale),
            self.error_flag.data_ptr(), self._stream(),
        )
        if code == -2:
            return False
        check(code, "attention_prefill_tcgen05")
        self._ran("attention_prefill_tcgen05")
        return True

    def sample(self, logits, temperatures, uniforms, out_tokens) -> None:
        check(
            function("distie_sample")(
                logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1],
                temperatures.data_ptr() if temperatures is not None else None,
                uniforms.data_ptr() if uniforms is not None else None, out_tokens.data_ptr(), self._stream(),
            ),
            "sample",
        )
        self._ran("sample")
