"""Plain tensor-op versions of every kernel, with the kernels' own signatures.

Two uses.  The ``-m gpu`` tests check each CUDA kernel against the function of the
same name here, at sizes the engine does not use.  And the CPU tests hand a
:class:`RefKernels` to the engine in place of the CUDA set, so that cache
bookkeeping, batching, scheduling and trace replay run end to end on a machine
without a GPU.  The product never imports this file.
"""

from __future__ import annotations

import torch

from distie_b200.kernels.interface import KernelSet, KvSlot, RotaryTable, StepTensors


def embed(ids, table):
    return table[ids.long()].float()


def add_rmsnorm(delta, residual, weight, eps, dtype, rows_index=None):
    """Returns (new residual, normed).  With rows_index only those rows are normed and the residual is unchanged."""
    if delta is not None and delta.dim() == 3:  # float32 slices of a split product
        delta = delta.float().sum(0)
    summed = residual if delta is None else residual + delta.float()
    source = summed if rows_index is None else summed[rows_index.long()]
    variance = (source * source).mean(dim=-1, keepdim=True)
    normed = (source * torch.rsqrt(variance + eps)).to(dtype)
    out = (weight.float() * normed.float()).to(dtype)
    return (summed if rows_index is None else residual), out


def swiglu(gate_up):
    inter = gate_up.shape[1] // 2
    g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    return (g / (1 + torch.exp(-g)) * u).to(gate_up.dtype)


def rotate(x, positions, rotary: RotaryTable | None):
    """x [T, heads, d] -> rotated, float32 arithmetic, stored back in x.dtype."""
    if rotary is None:
        return x.clone()
    rot = rotary.rotary_dim
    angles = positions.float()[:, None] * rotary.inv_freq.float()[None, :]
    factor = float(getattr(rotary, "factor", 1.0))
    cos, sin = angles.cos()[:, None, :] * factor, angles.sin()[:, None, :] * factor
    xf = x.float()
    out = xf.clone()
    if rotary.interleaved:
        a, b = xf[..., 0:rot:2], xf[..., 1:rot:2]
        out[..., 0:rot:2] = a * cos - b * sin
        out[..., 1:rot:2] = b * cos + a * sin
    else:
        a, b = xf[..., : rot // 2], xf[..., rot // 2 : rot]
        out[..., : rot // 2] = a * cos - b * sin
        out[..., rot // 2 : rot] = b * cos + a * sin
    return out.to(x.dtype)


def rope_kv_write(qkv, step: StepTensors, kv: KvSlot | None, rotary, num_heads, num_kv_heads, head_dim,
                  bias=None, q_out=None):
    if qkv.dim() == 3:  # float32 slices of the projection: sum, add the bias, then as below on a copy
        dense = qkv.float().sum(0)
        if bias is not None:
            dense = dense + bias.float()
        dense = dense.to(q_out.dtype)
        rope_kv_write(dense, step, kv, rotary, num_heads, num_kv_heads, head_dim)
        q_out.copy_(dense[:, : num_heads * head_dim])
        return
    tokens = step.num_tokens
    q_end, k_end = num_heads * head_dim, (num_heads + num_kv_heads) * head_dim
    positions = step.positions[:tokens]
    q = rotate(qkv[:tokens, :q_end].reshape(tokens, num_heads, head_dim), positions, rotary)
    qkv[:tokens, :q_end] = q.reshape(tokens, q_end)
    if q_out is not None:
        q_out.copy_(qkv[:tokens, :q_end])
    if kv is None:
        return
    k = rotate(qkv[:tokens, q_end:k_end].reshape(tokens, num_kv_heads, head_dim), positions, rotary)
    v = qkv[:tokens, k_end:].reshape(tokens, num_kv_heads, head_dim)
    seats = step.seq_seat[step.token_seq[:tokens].long()].long()
    pos = positions.long()
    pages = kv.block_table[seats, pos // kv.page_size].long()
    if bool(((pages < 0) | (pages >= kv.num_pages)).any()):
        raise IndexError("a new token's page is missing from its block table")
    kv.k[pages, :, pos % kv.page_size, :] = k
    kv.v[pages, :, pos % kv.page_size, :] = v


def attention(qkv, step: StepTensors, kv: KvSlot, num_heads, num_kv_heads, head_dim, window, scale):
    """Token by token: gather the visible keys of the token's request from its pages, softmax in float32."""
    tokens = step.num_tokens
    out = torch.zeros((tokens, num_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    rep = num_heads // num_kv_heads
    for t in range(tokens):
        pos = int(step.positions[t])
        seat = int(step.seq_seat[int(step.token_seq[t])])
        first = max(0, pos - int(window) + 1) if window else 0
        keys = torch.arange(first, pos + 1, device=qkv.device)
        pages = kv.block_table[seat, keys // kv.page_size].long()
        if bool(((pages < 0) | (pages >= kv.num_pages)).any()):
            raise IndexError("a block table does not cover the keys a token attends to")
        k = kv.k[pages, :, keys % kv.page_size, :].float()  # [n, kv_heads, d]
        v = kv.v[pages, :, keys % kv.page_size, :].float()
        q = qkv[t, : num_heads * head_dim].reshape(num_heads, head_dim).float()
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
        scores = torch.einsum("hd,nhd->hn", q, k) * scale
        probs = torch.softmax(scores, dim=-1)
        out[t] = torch.einsum("hn,nhd->hd", probs, v).reshape(-1).to(qkv.dtype)
    return out


def sample(logits, temperatures, uniforms):
    picks = logits.float().argmax(dim=-1).to(torch.int32)
    if temperatures is None:
        return picks
    for row in range(logits.shape[0]):
        t = float(temperatures[row])
        if t > 0:
            z = logits[row].float() / t
            p = torch.exp(z - z.max())
            cdf = torch.cumsum(p.double(), dim=0)
            target = float(uniforms[row]) * float(cdf[-1])
            picks[row] = int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True).clamp(max=logits.shape[1] - 1))
    return picks


class RefKernels(KernelSet):
    """The interface of the CUDA kernel sets, computed with the functions above."""

    def __init__(self, dtype=torch.float32, device="cpu") -> None:
        self.dtype = dtype
        self.device = torch.device(device)
        self.launches = 0

    def embed(self, step, table, residual):
        residual[: step.num_tokens] = embed(step.token_ids[: step.num_tokens], table)

    def add_rmsnorm(self, delta, residual, weight, eps, out, rows_index=None):
        new_residual, normed = add_rmsnorm(delta, residual, weight, eps, self.dtype, rows_index)
        if rows_index is None and delta is not None:
            residual.copy_(new_residual)
        out.copy_(normed)

    def linear(self, x, weight, bias=None, out_dtype=None):
        y = torch.nn.functional.linear(x.float(), weight.float(), bias.float() if bias is not None else None)
        return y.to(out_dtype or self.dtype)

    def swiglu(self, gate_up, out):
        out.copy_(swiglu(gate_up))

    def rope_kv_write(self, qkv, step, kv, rotary, num_heads, num_kv_heads, head_dim, bias=None, q_out=None):
        rope_kv_write(qkv, step, kv, rotary, num_heads, num_kv_heads, head_dim, bias, q_out)

    def attention(self, qkv, out, step, kv, num_heads, num_kv_heads, head_dim, window, scale):
        out.copy_(attention(qkv, step, kv, num_heads, num_kv_heads, head_dim, window, scale))

    def sample(self, logits, temperatures, uniforms, out_tokens):
        out_tokens.copy_(sample(logits, temperatures, uniforms))

    def check_errors(self):
        return None
