"""The entry point that allocates nothing, called through its exported C symbol.

``distie_attention_decode_static`` is for callers of the library that cannot
allocate device memory where they need decode attention: processes whose device
memory was handed out completely at start-up, plug-ins that get tensors but no
allocator, loops that must not risk the synchronisation an allocation can bring.
It keeps the scratch of the split-KV kernel in an array inside the library.  The
test calls it twice in a row, with different inputs (so that what the first call
left in the shared array would show if it were read), and compares each result
with the ordinary entry point given a scratch buffer by the caller.  This file
sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def library() -> ctypes.CDLL:
    from distie_b200.csrc import build

    lib = ctypes.CDLL(build.build_cuda_unit("base"))
    lib.distie_attention_decode_static.argtypes = [P, I, P, I, P, P, P, P, I, P, P, I, I, I, I, I, I, I, F, I, I, P, P]
    lib.distie_attention_decode_static.restype = I
    lib.distie_attention_decode.argtypes = [P, I, P, I, P, P, P, P, P, I, P, P, I, I, I, I, I, I, I, F, I, I, P, P]
    lib.distie_attention_decode.restype = I
    lib.distie_attention_decode_scratch_floats.argtypes = [I, I, I, I]
    lib.distie_attention_decode_scratch_floats.restype = ctypes.c_longlong
    lib.distie_attention_decode_static_capacity.restype = ctypes.c_longlong
    lib.distie_no_alloc_error.argtypes = [I]
    lib.distie_no_alloc_error.restype = ctypes.c_char_p
    return lib


def case(seed: int, tokens: int, heads: int, kv_heads: int, head_dim: int, page: int, lengths: list[int]):
    g = torch.Generator(device="cuda").manual_seed(seed)
    pages_each = [-(-n // page) for n in lengths]
    pages = sum(pages_each) + 2
    k = torch.randn(pages, kv_heads, page, head_dim, generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn(pages, kv_heads, page, head_dim, generator=g, device="cuda").to(torch.bfloat16)
    table = torch.full((tokens, max(pages_each)), -1, dtype=torch.int32)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(seed)).to(torch.int32)
    at = 0
    for seat, count in enumerate(pages_each):
        table[seat, :count] = order[at : at + count]
        at += count
    q = torch.randn(tokens, (heads + 2 * kv_heads) * head_dim, generator=g, device="cuda").to(torch.bfloat16)
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device="cuda")
    rows = torch.arange(tokens, dtype=torch.int32, device="cuda")
    return q, k, v, table.cuda(), positions, rows, pages


def run(lib, static: bool, q, k, v, table, positions, rows, pages, heads, kv_heads, head_dim, page, splits):
    tokens = q.shape[0]
    out = torch.zeros(tokens, heads * head_dim, dtype=torch.bfloat16, device="cuda")
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    head = [q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0)]
    tail = [positions.data_ptr(), rows.data_ptr(), rows.data_ptr(), table.data_ptr(), table.shape[1], k.data_ptr(),
            v.data_ptr(), tokens, heads, kv_heads, head_dim, page, pages, 0, head_dim**-0.5, splits, 1, error.data_ptr(), stream]
    if static:
        code = lib.distie_attention_decode_static(*head, *tail)
    else:
        floats = lib.distie_attention_decode_scratch_floats(tokens, heads, head_dim, splits)
        scratch = torch.empty(max(1, floats), dtype=torch.float32, device="cuda")
        code = lib.distie_attention_decode(*head, scratch.data_ptr(), *tail)
    torch.cuda.synchronize()
    assert int(error.item()) == 0
    return code, out


def test_static_entry_point_matches_the_allocating_one_twice_in_a_row():
    lib = library()
    heads, kv_heads, head_dim, page = 12, 2, 128, 16
    first = case(1, 6, heads, kv_heads, head_dim, page, [700, 33, 1024, 257, 16, 480])
    second = case(2, 3, heads, kv_heads, head_dim, page, [90, 1500, 640])
    for inputs, splits in ((first, 8), (second, 5)):
        code, got = run(lib, True, *inputs, heads, kv_heads, head_dim, page, splits)
        assert code == 0, lib.distie_no_alloc_error(code).decode()
        code, want = run(lib, False, *inputs, heads, kv_heads, head_dim, page, splits)
        assert code == 0
        scale = float(want.float().abs().max())
        assert float((got.float() - want.float()).abs().max()) <= 1.6e-2 * scale
        assert torch.equal(got, want), "same kernels, same inputs: the results are the same bits"


def test_static_entry_point_refuses_what_does_not_fit():
    lib = library()
    heads, kv_heads, head_dim, page = 32, 8, 128, 16
    inputs = case(3, 64, heads, kv_heads, head_dim, page, [40] * 64)
    capacity = lib.distie_attention_decode_static_capacity()
    assert lib.distie_attention_decode_scratch_floats(64, heads, head_dim, 16) > capacity
    code, out = run(lib, True, *inputs, heads, kv_heads, head_dim, page, 16)
    assert code == -3 and "exceeds the built-in scratch" in lib.distie_no_alloc_error(code).decode()
    assert float(out.float().abs().sum()) == 0.0, "a refused call launches nothing"
    code, _ = run(lib, True, *inputs, heads, kv_heads, head_dim, page, 1)  # one split needs no scratch at all
    assert code == 0
