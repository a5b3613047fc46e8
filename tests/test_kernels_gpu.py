"""Each CUDA kernel alone against its plain reference, at sizes the engine's tiny models do not use."""

from __future__ import annotations

import pytest
import torch

import ref_kernels as ref

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 1.6e-2}  # relative to the largest magnitude of the expected result


@pytest.fixture(scope="module")
def kernel_sets():
    from distie_b200.kernels import make_kernels

    return {dtype: make_kernels(dtype, "cuda:0") for dtype in DTYPES}


def close(got, want, dtype, what=""):
    scale = max(1e-6, float(want.float().abs().max()))
    error = float((got.float() - want.float()).abs().max()) / scale
    assert error <= TOL[dtype], f"{what}: off by {error:.3e} of the scale"


def step_of(tokens_per_seq, pasts, seats, device="cuda"):
    """StepTensors for a batch in which request i brings tokens_per_seq[i] tokens after pasts[i] cached ones."""
    from distie_b200.kernels.interface import Q_TILE, StepTensors

    positions, token_seq = [], []
    order = sorted(range(len(tokens_per_seq)), key=lambda i: (tokens_per_seq[i] != 1, i))
    for row, i in enumerate(order):
        positions += list(range(pasts[i], pasts[i] + tokens_per_seq[i]))
        token_seq += [row] * tokens_per_seq[i]
    total = len(positions)
    as_i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)  # noqa: E731
    tiles, start = [], 0
    for i in order:
        n = tokens_per_seq[i]
        if n > 1:
            tiles += [(start + at, min(Q_TILE, n - at)) for at in range(0, n, Q_TILE)]
        start += n
    step = StepTensors(
        token_ids=torch.zeros(total, dtype=torch.int32, device=device),
        positions=as_i32(positions),
        token_seq=as_i32(token_seq),
        seq_seat=as_i32([seats[i] for i in order]),
        num_tokens=total,
        num_seqs=len(order),
        num_decode_tokens=sum(1 for n in tokens_per_seq if n == 1),
        max_kv_len=max(p + n for p, n in zip(pasts, tokens_per_seq)),
    )
    if tiles:
        step.q_tiles = as_i32(tiles).reshape(-1)
        step.num_q_tiles = len(tiles)
    return step


def make_cache(dtype, pages, kv_heads, page_size, head_dim, seats, width, fill=True, seed=0):
    from distie_b200.kernels.interface import KvSlot

    g = torch.Generator(device="cuda").manual_seed(seed)
    shape = (pages, kv_heads, page_size, head_dim)
    k = torch.randn(shape, generator=g, device="cuda").to(dtype) if fill else torch.zeros(shape, dtype=dtype, device="cuda")
    v = torch.randn(shape, generator=g, device="cuda").to(dtype) if fill else torch.zeros(shape, dtype=dtype, device="cuda")
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(seed))
    table = torch.full((seats, width), -1, dtype=torch.int32)
    table.view(-1)[: min(pages, seats * width)] = perm[: min(pages, seats * width)].to(torch.int32)
    return KvSlot(k, v, table.cuda(), page_size, pages)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,vocab", [(80, 97), (1536, 1000), (200, 33)])
def test_embed(kernel_sets, dtype, hidden, vocab):
    ks = kernel_sets[dtype]
    table = torch.randn(vocab, hidden, device="cuda").to(dtype)
    step = step_of([11], [0], [0])
    step.token_ids = torch.randint(0, vocab, (11,), dtype=torch.int32, device="cuda")
    out = torch.empty(11, hidden, dtype=torch.float32, device="cuda")
    ks.embed(step, table, out)
    assert torch.equal(out, ref.embed(step.token_ids, table))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize(
    "rows,hidden,eps",
    [(5, 96, 1e-5), (33, 1536, 1e-6), (2, 8200, 1e-6), (7, 50, 1e-3), (1203, 1536, 1e-6), (1070, 3584, 1e-5), (1025, 96, 1e-6),
     (1024, 5120, 1e-6)],
)
def test_add_rmsnorm(kernel_sets, dtype, rows, hidden, eps):
    ks = kernel_sets[dtype]
    residual = torch.randn(rows, hidden, device="cuda") * 3
    delta = torch.randn(rows, hidden, device="cuda").to(dtype)
    weight = 1 + 0.1 * torch.randn(hidden, device="cuda")
    for with_delta in (True, False):
        res = residual.clone()
        out = torch.empty(rows, hidden, dtype=dtype, device="cuda")
        ks.add_rmsnorm(delta if with_delta else None, res, weight, eps, out)
        want_res, want = ref.add_rmsnorm(delta if with_delta else None, residual, weight, eps, dtype)
        assert torch.allclose(res, want_res, atol=1e-6, rtol=1e-6)
        close(out, want, dtype, "rmsnorm")
    rows_index = torch.tensor([rows - 1, 0, rows // 2], dtype=torch.int32, device="cuda")
    res = residual.clone()
    out = torch.empty(3, hidden, dtype=dtype, device="cuda")
    ks.add_rmsnorm(delta, res, weight, eps, out, rows_index)
    _, want = ref.add_rmsnorm(delta, residual, weight, eps, dtype, rows_index)
    assert torch.equal(res, residual), "row-selected norm must leave the residual alone"
    close(out, want, dtype, "rmsnorm rows")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden,splits", [(8, 1536, 4), (3, 96, 1), (5, 50, 3), (2, 8200, 2), (1100, 1536, 3), (8, 1536, 11)])
def test_add_rmsnorm_sums_slices_of_a_split_product(kernel_sets, dtype, rows, hidden, splits):
    ks = kernel_sets[dtype]
    residual = torch.randn(rows, hidden, device="cuda") * 3
    slices = torch.randn(splits, rows, hidden, device="cuda")
    weight = 1 + 0.1 * torch.randn(hidden, device="cuda")
    res = residual.clone()
    out = torch.empty(rows, hidden, dtype=dtype, device="cuda")
    ks.add_rmsnorm(slices, res, weight, 1e-6, out)
    want_res, want = ref.add_rmsnorm(slices, residual, weight, 1e-6, dtype)
    assert torch.allclose(res, want_res, atol=1e-5, rtol=1e-5)
    close(out, want, dtype, "rmsnorm of slices")
    rows_index = torch.tensor([rows - 1, 0], dtype=torch.int32, device="cuda")
    out2 = torch.empty(2, hidden, dtype=dtype, device="cuda")
    res2 = residual.clone()
    ks.add_rmsnorm(slices, res2, weight, 1e-6, out2, rows_index)
    assert torch.equal(res2, residual)
    close(out2, ref.add_rmsnorm(slices, residual, weight, 1e-6, dtype, rows_index)[1], dtype, "rmsnorm of slices, rows")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,k,n", [(8, 1536, 2048), (1, 8960, 1536), (16, 200, 57), (5, 96, 40), (30, 96, 40)])
def test_linear_split_slices_add_up(kernel_sets, dtype, m, k, n):
    ks = kernel_sets[dtype]
    x = torch.randn(m, k, device="cuda").to(dtype)
    w = (torch.randn(n, k, device="cuda") * 0.1).to(dtype)
    slices = ks.linear_split(x, w)
    assert slices.dim() == 3 and slices.dtype == torch.float32 and slices.shape[1:] == (m, n)
    want = torch.nn.functional.linear(x.double(), w.double())
    close(slices.sum(0), want, torch.float32 if dtype == torch.float32 else dtype, "sum of slices")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,inter", [(3, 224), (70, 8960), (1, 17)])
def test_swiglu(kernel_sets, dtype, tokens, inter):
    ks = kernel_sets[dtype]
    gate_up = (torch.randn(tokens, 2 * inter, device="cuda") * 2).to(dtype)
    out = torch.empty(tokens, inter, dtype=dtype, device="cuda")
    ks.swiglu(gate_up, out)
    close(out, ref.swiglu(gate_up), dtype, "swiglu")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize(
    "m,k,n,bias",
    [(5, 96, 40, True), (64, 1536, 2048, True), (7, 224, 96, False), (130, 80, 1000, False), (1, 1536, 2048, True),
     (16, 200, 57, True), (9, 8960, 1536, False), (8, 1536, 1000, False), (3, 72, 9, True), (17, 96, 40, True)],
)
def test_linear(kernel_sets, dtype, m, k, n, bias):
    ks = kernel_sets[dtype]
    x = torch.randn(m, k, device="cuda").to(dtype)
    w = (torch.randn(n, k, device="cuda") * 0.1).to(dtype)
    b = torch.randn(n, device="cuda") if bias else None
    want = torch.nn.functional.linear(x.double(), w.double(), b.double() if bias else None)
    close(ks.linear(x, w, b), want, dtype, "linear")
    got32 = ks.linear(x, w, b, out_dtype=torch.float32)
    assert got32.dtype == torch.float32
    close(got32, want, dtype, "linear float32 out")
    if dtype == torch.bfloat16:  # a matrix stored in 32-bit keeps a 32-bit product
        w32 = w.float() + 1e-4 * torch.randn(n, k, device="cuda")
        want32 = torch.nn.functional.linear(x.double(), w32.double(), b.double() if bias else None)
        close(ks.linear(x, w32, b, out_dtype=torch.float32), want32, torch.float32, "float32-stored matrix")


@pytest.mark.parametrize(
    "m,k,n", [(128, 64, 128), (17, 96, 40), (130, 1536, 2048), (2048, 1536, 1536), (300, 8960, 1536), (64, 200, 1000), (513, 72, 264)]
)
def test_tensor_core_product(kernel_sets, m, k, n):
    """The tcgen05 kernel alone: bfloat16 and float32 results, ragged edges in every dimension."""
    ks = kernel_sets[torch.bfloat16]
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.1).to(torch.bfloat16)
    want = torch.nn.functional.linear(x.double(), w.double())
    for out_dtype, epi in ((torch.bfloat16, 0), (torch.float32, 1)):
        out = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
        ks._gemm_tcgen05(x, w, out, epi)
        ks.check_errors()
        close(out, want, torch.bfloat16 if epi == 0 else torch.float32, f"tcgen05 product, epilogue {epi}")
    if n % 2 == 0:
        inter = n // 2
        out = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
        ks._gemm_tcgen05(x, w, out, 2)
        ks.check_errors()
        close(out, torch.nn.functional.silu(want[:, :inter]) * want[:, inter:], torch.bfloat16, "tcgen05 product with SwiGLU")


@pytest.mark.parametrize(
    "m,k,n", [(1, 64, 128), (8, 1536, 2048), (16, 200, 1000), (17, 96, 40), (3, 8960, 1536), (40, 1536, 264),
              (64, 72, 130), (33, 4096, 512), (5, 8, 6), (48, 264, 520)]
)
def test_weight_streaming_product(kernel_sets, m, k, n):
    """The tcgen05 kernel for few rows alone: slices, stored result with bias, and SwiGLU, ragged everywhere."""
    ks = kernel_sets[torch.bfloat16]
    backing = torch.randn(m, k + 8, device="cuda").to(torch.bfloat16)
    x = backing[:, :k]  # a row stride that is not K
    w = (torch.randn(n, k, device="cuda") * 0.1).to(torch.bfloat16)
    b = torch.randn(n, device="cuda")
    want = torch.nn.functional.linear(x.double(), w.double())
    from distie_b200.kernels.library import function

    splits = function("distie_gemm_tcgen05_skinny_splits")(n, k, ks.sm_count)
    slices = torch.full((splits, m, n), float("nan"), dtype=torch.float32, device="cuda")
    ks._stream_weights(x, w, None, slices, 0)
    ks.check_errors()
    assert slices.dim() == 3 and slices.dtype == torch.float32
    close(slices.sum(0), want, torch.float32, "weight streaming, slices")
    for out_dtype in (torch.bfloat16, torch.float32):
        out = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
        ks._stream_weights(x, w, b, out, 1)
        ks.check_errors()
        close(out, want + b.double(), out_dtype, "weight streaming, stored with bias")
    if n % 2 == 0:
        inter = n // 2
        out = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
        ks._stream_weights(x, w, None, out, 2)
        ks.check_errors()
        close(out, torch.nn.functional.silu(want[:, :inter]) * want[:, inter:], torch.bfloat16, "weight streaming, SwiGLU")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,k,inter", [(3, 96, 100), (8, 1536, 8960), (13, 200, 57), (40, 96, 224), (1, 64, 8)])
def test_linear_swiglu(kernel_sets, dtype, m, k, inter):
    ks = kernel_sets[dtype]
    x = torch.randn(m, k, device="cuda").to(dtype)
    w = (torch.randn(2 * inter, k, device="cuda") * 0.1).to(dtype)
    gate_up = torch.nn.functional.linear(x.double(), w.double())
    want = torch.nn.functional.silu(gate_up[:, :inter]) * gate_up[:, inter:]
    close(ks.linear_swiglu(x, w), want, dtype, "fused gate/up + SwiGLU")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize(
    "heads,kv_heads,head_dim,rotary_dim,interleaved,page,factor",
    [(4, 2, 16, 16, False, 16, 1.0), (3, 1, 32, 32, False, 8, 1.0), (12, 2, 128, 128, False, 16, 1.0), (5, 5, 48, 24, True, 4, 1.0),
     (6, 3, 80, 80, False, 32, 1.0), (4, 2, 64, 64, False, 16, 1.25), (2, 1, 48, 16, True, 8, 0.8)],
)
def test_rope_kv_write(kernel_sets, dtype, heads, kv_heads, head_dim, rotary_dim, interleaved, page, factor):
    from distie_b200.kernels.interface import RotaryTable

    ks = kernel_sets[dtype]
    tokens_per_seq, pasts, seats = [1, 9, 1, 20], [37, 0, page * 2 - 1, page - 3], [2, 0, 3, 1]
    step = step_of(tokens_per_seq, pasts, seats)
    width = 16
    kv = make_cache(dtype, 64, kv_heads, page, head_dim, 4, width, fill=False)
    kv_ref = make_cache(dtype, 64, kv_heads, page, head_dim, 4, width, fill=False)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))).cuda()
    rotary = RotaryTable(inv_freq, rotary_dim, interleaved, factor)  # the factor scales cos and sin
    qkv = torch.randn(step.num_tokens, (heads + 2 * kv_heads) * head_dim, device="cuda").to(dtype)
    mine, theirs = qkv.clone(), qkv.clone()
    ks.rope_kv_write(mine, step, kv, rotary, heads, kv_heads, head_dim)
    ref.rope_kv_write(theirs, step, kv_ref, rotary, heads, kv_heads, head_dim)
    ks.check_errors()
    close(mine, theirs, dtype, "rotated q (k and v columns untouched)")
    close(kv.k, kv_ref.k, dtype, "cached keys")
    assert torch.equal(kv.v, kv_ref.v), "values are copied bit for bit"
    assert float(kv.k.float().abs().sum()) > 0
    # The same from float32 slices of the projection plus a bias, q into its own buffer: a few slices,
    # and more than the kernel sums in one round of loads.
    for count in (3, 10):
        slices = torch.randn(count, step.num_tokens, qkv.shape[1], device="cuda")
        bias = torch.randn(qkv.shape[1], device="cuda")
        kv_a = make_cache(dtype, 64, kv_heads, page, head_dim, 4, width, fill=False)
        kv_b = make_cache(dtype, 64, kv_heads, page, head_dim, 4, width, fill=False)
        q_a = torch.zeros(step.num_tokens, heads * head_dim, dtype=dtype, device="cuda")
        q_b = torch.zeros_like(q_a)
        ks.rope_kv_write(slices, step, kv_a, rotary, heads, kv_heads, head_dim, bias=bias, q_out=q_a)
        ref.rope_kv_write(slices, step, kv_b, rotary, heads, kv_heads, head_dim, bias=bias, q_out=q_b)
        ks.check_errors()
        close(q_a, q_b, dtype, f"rotated q from {count} slices")
        close(kv_a.k, kv_b.k, dtype, f"cached keys from {count} slices")
        close(kv_a.v, kv_b.v, dtype, f"cached values from {count} slices")
    # Nothing is written when the call only reads the cache; no rotation without a table.
    kv_none = make_cache(dtype, 64, kv_heads, page, head_dim, 4, width, fill=False)
    again = qkv.clone()
    ks.rope_kv_write(again, step, None, None, heads, kv_heads, head_dim)
    assert torch.equal(again, qkv) and float(kv_none.k.float().abs().sum()) == 0


@pytest.mark.parametrize(
    "heads,kv_heads,head_dim,hidden,page,tokens,pasts,with_bias,with_table,factor",
    [(12, 2, 128, 1536, 16, [200, 1, 90], [13, 70, 0], True, True, 1.0),      # pairs of CTAs, 2,048 columns
     (3, 1, 64, 200, 8, [150], [5], True, True, 1.25),                         # one CTA; 320 columns: a tile's second half ends inside v
     (5, 5, 64, 72, 4, [129, 2, 140], [0, 9, 30], False, True, 1.0),           # as many kv heads as heads, no bias, pages of 4
     (2, 2, 128, 264, 32, [300], [31], True, False, 1.0),                      # no rotation: bias and stores only
     (7, 1, 128, 96, 16, [128], [0], True, True, 0.8)],                        # exactly one tile of rows; 1,152 columns
)
def test_qkv_projection_with_fused_rotation_and_cache_write(kernel_sets, heads, kv_heads, head_dim, hidden, page, tokens,
                                                            pasts, with_bias, with_table, factor):
    """The q/k/v product whose epilogue adds the bias, rotates and stores (128 rows and more, bfloat16) against
    the plain product followed by the plain rotation and cache write; also without a cache to write."""
    from distie_b200.kernels.interface import RotaryTable

    ks = kernel_sets[torch.bfloat16]
    step = step_of(tokens, pasts, list(range(len(tokens))))
    width = max(-(-(p + n) // page) for p, n in zip(pasts, tokens)) + 1
    pages = len(tokens) * width
    n = (heads + 2 * kv_heads) * head_dim
    x = torch.randn(step.num_tokens, hidden, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, hidden, device="cuda") / hidden**0.5).to(torch.bfloat16)
    bias = torch.randn(n, device="cuda") if with_bias else None
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))).cuda()
    rotary = RotaryTable(inv_freq, head_dim, False, factor) if with_table else None
    product = torch.nn.functional.linear(x.float(), w.float()).unsqueeze(0)
    for write in (True, False):
        kv_a = make_cache(torch.bfloat16, pages, kv_heads, page, head_dim, len(tokens), width, fill=False)
        kv_b = make_cache(torch.bfloat16, pages, kv_heads, page, head_dim, len(tokens), width, fill=False)
        q_a = torch.full((step.num_tokens, heads * head_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
        q_b = torch.zeros_like(q_a)
        before = ks.kernel_counts.get("gemm_tcgen05_qkv", 0)
        step.derived.clear()
        ks.qkv_rope_write(x, w, bias, step, kv_a if write else None, rotary, heads, kv_heads, head_dim, q_a)
        ks.check_errors()
        assert ks.kernel_counts.get("gemm_tcgen05_qkv", 0) == before + 1, "the fused kernel was meant to run"
        ref.rope_kv_write(product, step, kv_b if write else None, rotary, heads, kv_heads, head_dim, bias=bias, q_out=q_b)
        close(q_a, q_b, torch.bfloat16, "rotated q")
        close(kv_a.k, kv_b.k, torch.bfloat16, "cached keys")
        close(kv_a.v, kv_b.v, torch.bfloat16, "cached values")
        assert (float(kv_a.k.float().abs().sum()) > 0) == write
        # every slot that the reference left alone is still zero: nothing was written beside the tokens' slots
        assert torch.equal(kv_a.k == 0, kv_b.k == 0) or float(((kv_a.k != 0) & (kv_b.k == 0)).sum()) == 0
        assert float(((kv_a.v != 0) & (kv_b.v == 0)).sum()) == 0


def filled_cache_for(dtype, kv_heads, head_dim, page, lengths, seed=1):
    """A cache whose tables cover `lengths[i]` tokens for seat i, pages in scrambled order."""
    pages_each = [-(-n // page) for n in lengths]
    total = sum(pages_each) + 3
    kv = make_cache(dtype, total, kv_heads, page, head_dim, len(lengths), max(pages_each) + 1, seed=seed)
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(seed)).to(torch.int32)
    table = torch.full((len(lengths), max(pages_each) + 1), -1, dtype=torch.int32)
    at = 0
    for seat, count in enumerate(pages_each):
        table[seat, :count] = perm[at : at + count]
        at += count
    kv.block_table = table.cuda()
    return kv


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize(
    "heads,kv_heads,head_dim,page,window",
    [(4, 2, 16, 16, None), (3, 1, 32, 8, None), (12, 2, 128, 16, None), (6, 1, 64, 16, 37), (5, 5, 48, 4, None), (16, 2, 256, 32, 100), (14, 2, 80, 16, None)],
)
def test_attention_mixed_batch(kernel_sets, dtype, heads, kv_heads, head_dim, page, window):
    """Portions beside single tokens: every token against its own request's pages only."""
    ks = kernel_sets[dtype]
    tokens_per_seq, pasts = [1, 23, 1, 2, 1], [130, 45, 0, 310, 63]
    lengths = [p + n for p, n in zip(pasts, tokens_per_seq)]
    kv = filled_cache_for(dtype, kv_heads, head_dim, page, lengths)
    step = step_of(tokens_per_seq, pasts, list(range(5)))
    qkv = torch.randn(step.num_tokens, (heads + 2 * kv_heads) * head_dim, device="cuda").to(dtype)
    out = torch.zeros(step.num_tokens, heads * head_dim, dtype=dtype, device="cuda")
    ks.attention(qkv, out, step, kv, heads, kv_heads, head_dim, window, head_dim**-0.5)
    ks.check_errors()
    want = ref.attention(qkv, step, kv, heads, kv_heads, head_dim, window, head_dim**-0.5)
    close(out, want, dtype, "attention")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim,heads,kv_heads", [(128, 12, 2), (64, 6, 1), (128, 40, 2)])
@pytest.mark.parametrize("splits", [1, 2, 3, 8, 13, 17, 40])
def test_decode_attention_at_every_split_count(kernel_sets, dtype, head_dim, heads, kv_heads, splits, monkeypatch):
    """Single tokens with the keys cut into a given number of splits: merged by one CTA, by a cluster, by the merge kernel."""
    ks = kernel_sets[dtype]
    pasts = [699, 32, 1499, 0, 15]
    kv = filled_cache_for(dtype, kv_heads, head_dim, 16, [p + 1 for p in pasts], seed=11)
    step = step_of([1] * len(pasts), pasts, list(range(len(pasts))))
    monkeypatch.setattr(ks, "plan_splits", lambda *args: splits)
    qkv = torch.randn(step.num_tokens, (heads + 2 * kv_heads) * head_dim, device="cuda").to(dtype)
    out = torch.zeros(step.num_tokens, heads * head_dim, dtype=dtype, device="cuda")
    ks.attention(qkv, out, step, kv, heads, kv_heads, head_dim, None, head_dim**-0.5)
    ks.check_errors()
    want = ref.attention(qkv, step, kv, heads, kv_heads, head_dim, None, head_dim**-0.5)
    close(out, want, dtype, f"decode attention in {splits} splits")


@pytest.mark.parametrize(
    "heads,kv_heads,head_dim,hidden,page,with_bias,with_table,factor",
    [(12, 2, 128, 1536, 16, True, True, 1.0), (6, 1, 64, 200, 8, True, True, 1.25), (5, 5, 64, 72, 16, False, True, 1.0),
     (40, 2, 128, 264, 32, True, False, 1.0), (4, 4, 128, 96, 4, True, True, 0.8)],
)
@pytest.mark.parametrize("splits", [1, 2, 4, 8, 13])
def test_decode_attention_from_the_projection(kernel_sets, heads, kv_heads, head_dim, hidden, page, with_bias, with_table,
                                              factor, splits, monkeypatch):
    """A step of single tokens through the merged op (projection slices -> bias, rotation, the token's key and
    value into the cache and into the attention itself) against the plain ops one after the other: the outputs,
    the cache rows that were written, and that no other row was touched.  Positions at the start of a request,
    at the first and last row of a page and of a group of 16 keys; with and without a write of the cache, and
    with a window of 100 keys."""
    from distie_b200.kernels.interface import KvSlot, RotaryTable

    ks = kernel_sets[torch.bfloat16]
    pasts = [699, 32, 1499, 0, 15, 16, 31, 255, 256]
    step = step_of([1] * len(pasts), pasts, list(range(len(pasts))))
    monkeypatch.setattr(ks, "plan_splits", lambda *args: splits)
    n = (heads + 2 * kv_heads) * head_dim
    x = torch.randn(step.num_tokens, hidden, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, hidden, device="cuda") / hidden**0.5).to(torch.bfloat16)
    bias = torch.randn(n, device="cuda") if with_bias else None
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))).cuda()
    rotary = RotaryTable(inv_freq, head_dim, False, factor) if with_table else None
    product = torch.nn.functional.linear(x.float(), w.float()).unsqueeze(0)
    scale = head_dim**-0.5
    for writes, window in ((True, None), (False, None), (True, 100)):
        kv_a = filled_cache_for(torch.bfloat16, kv_heads, head_dim, page, [p + 1 for p in pasts], seed=13)
        kv_b = KvSlot(kv_a.k.clone(), kv_a.v.clone(), kv_a.block_table, kv_a.page_size, kv_a.num_pages)
        before_k, before_v = kv_a.k.clone(), kv_a.v.clone()
        out = torch.full((step.num_tokens, heads * head_dim), float("nan"), dtype=torch.bfloat16, device="cuda")
        count = ks.kernel_counts.get("attention_decode_mma_qkv", 0)
        ks.qkv_attention(x, w, bias, step, kv_a, writes, rotary, heads, kv_heads, head_dim, window, scale, out)
        ks.check_errors()
        assert ks.kernel_counts.get("attention_decode_mma_qkv", 0) == count + 1, "the merged kernel was meant to run"
        q = torch.zeros_like(out)
        ref.rope_kv_write(product, step, kv_b if writes else None, rotary, heads, kv_heads, head_dim, bias=bias, q_out=q)
        want = ref.attention(q, step, kv_b, heads, kv_heads, head_dim, window, scale)
        close(out, want, torch.bfloat16, f"merged decode attention, {splits} splits, writes {writes}, window {window}")
        close(kv_a.k, kv_b.k, torch.bfloat16, "cached keys")
        close(kv_a.v, kv_b.v, torch.bfloat16, "cached values")
        changed = (kv_a.k != before_k).any(-1) | (kv_a.v != before_v).any(-1)   # [pages, kv_heads, rows]
        expected = (kv_b.k != before_k).any(-1) | (kv_b.v != before_v).any(-1)
        assert not bool((changed & ~expected).any()), "a row other than the tokens' own was written"
        assert bool(changed.any()) == writes


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim,page,far", [(128, 16, 3), (64, 16, 511), (32, 8, 256), (128, 16, 1008)])
def test_attention_finds_one_far_key(kernel_sets, dtype, head_dim, page, far):
    """One key among a thousand is made to stand out; the output must be its value (a page edge included)."""
    ks = kernel_sets[dtype]
    heads, kv_heads, length = 4, 2, 1024
    kv = filled_cache_for(dtype, kv_heads, head_dim, page, [length], seed=5)
    kv.k.mul_(0.05)
    step = step_of([1], [length - 1], [0])
    qkv = torch.zeros(1, (heads + 2 * kv_heads) * head_dim, dtype=dtype, device="cuda")
    qkv[0, : heads * head_dim] = 1.0
    page_id = int(kv.block_table[0, far // page])
    kv.k[page_id, :, far % page, :] = 6.0  # score head_dim * 6 * scale: far above everything else
    for splits_len in (length, 1):  # many splits and a single one
        step.max_kv_len = splits_len
        out = torch.zeros(1, heads * head_dim, dtype=dtype, device="cuda")
        ks.attention(qkv, out, step, kv, heads, kv_heads, head_dim, None, head_dim**-0.5)
        want = kv.v[page_id, :, far % page, :].repeat_interleave(heads // kv_heads, dim=0).reshape(1, -1)
        close(out, want, dtype, f"far key {far}")
    # The same key just outside a window must not be seen; just inside it must.
    for window, seen in ((length - 1 - far, False), (length - far, True)):
        if window < 1:
            continue
        out = torch.zeros(1, heads * head_dim, dtype=dtype, device="cuda")
        ks.attention(qkv, out, step, kv, heads, kv_heads, head_dim, window, head_dim**-0.5)
        want = kv.v[page_id, :, far % page, :].repeat_interleave(heads // kv_heads, dim=0).reshape(1, -1)
        error = float((out.float() - want.float()).abs().max())
        assert (error < 0.05) == seen, f"window {window}: key {far} seen={error < 0.05}, expected {seen}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim,page,window", [(128, 16, None), (64, 8, None), (128, 16, 70), (64, 16, 200), (128, 32, 1),
                                                  (128, 4, None), (64, 24, 100)])
def test_prompt_portion_attention_long_context(kernel_sets, dtype, head_dim, page, window):
    """A portion of 150 tokens after 900 cached ones beside a whole short prompt: tiles, diagonal, window edges.
    Pages of 4 and of 24 rows are sizes the tcgen05 kernel refuses: in bfloat16 the mma.sync kernel takes over."""
    ks = kernel_sets[dtype]
    before = dict(ks.kernel_counts)
    heads, kv_heads = 6, 2
    tokens_per_seq, pasts = [150, 1, 70, 64], [900, 40, 0, 64]
    kv = filled_cache_for(dtype, kv_heads, head_dim, page, [p + n for p, n in zip(pasts, tokens_per_seq)], seed=3)
    step = step_of(tokens_per_seq, pasts, list(range(4)))
    qkv = torch.randn(step.num_tokens, (heads + 2 * kv_heads) * head_dim, device="cuda").to(dtype)
    out = torch.zeros(step.num_tokens, heads * head_dim, dtype=dtype, device="cuda")
    want = ref.attention(qkv, step, kv, heads, kv_heads, head_dim, window, head_dim**-0.5)
    if window:
        # A cache with a window gives pages back once every later token's window has passed them: the pages
        # wholly before the oldest key that a request's first new token sees are gone from its block table,
        # and the kernels must not ask for them (a tile's first block of keys starts before that key).
        table = kv.block_table.clone()
        for seat, past in enumerate(pasts):
            gone = max(0, past - window + 1) // page
            table[seat, :gone] = -1
        kv.block_table = table
    ks.attention(qkv, out, step, kv, heads, kv_heads, head_dim, window, head_dim**-0.5)
    ks.check_errors()
    close(out, want, dtype, "attention over a long context")
    if dtype == torch.bfloat16:
        ran = {name for name, count in ks.kernel_counts.items() if count > before.get(name, 0)}
        assert ("attention_prefill" if page in (4, 24) else "attention_prefill_tcgen05") in ran, sorted(ran)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far", [5, 511, 512, 959, 1000])
def test_prompt_portion_finds_one_far_key(kernel_sets, dtype, far):
    """Rows of a portion whose one far key stands out must return that key's value, rows before it must not."""
    ks = kernel_sets[dtype]
    heads, kv_heads, head_dim, page, past, count = 4, 2, 128, 16, 960, 64
    kv = filled_cache_for(dtype, kv_heads, head_dim, page, [past + count], seed=6)
    kv.k.mul_(0.05)
    page_id = int(kv.block_table[0, far // page])
    kv.k[page_id, :, far % page, :] = 6.0
    step = step_of([count], [past], [0])
    qkv = torch.zeros(count, (heads + 2 * kv_heads) * head_dim, dtype=dtype, device="cuda")
    qkv[:, : heads * head_dim] = 1.0
    value = kv.v[page_id, :, far % page, :].repeat_interleave(heads // kv_heads, dim=0).reshape(1, -1).float()
    for window in (None, 40):
        out = torch.zeros(count, heads * head_dim, dtype=dtype, device="cuda")
        ks.attention(qkv, out, step, kv, heads, kv_heads, head_dim, window, head_dim**-0.5)
        for row in range(count):
            pos = past + row
            seen = far <= pos and (window is None or far > pos - window)
            hit = float((out[row].float() - value[0]).abs().max()) < 0.05
            assert hit == seen, f"far {far} window {window}: row at position {pos} saw it={hit}, expected {seen}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_kernel_equals_generic_kernel(kernel_sets, dtype):
    """The split-KV kernel and the size-agnostic kernel are two routes to the same numbers."""
    ks = kernel_sets[dtype]
    heads, kv_heads, head_dim, page = 12, 2, 128, 16
    pasts = [5, 1000, 255, 256, 15, 16, 700, 0]
    kv = filled_cache_for(dtype, kv_heads, head_dim, page, [p + 1 for p in pasts], seed=9)
    step = step_of([1] * 8, pasts, list(range(8)))
    qkv = torch.randn(8, (heads + 2 * kv_heads) * head_dim, device="cuda").to(dtype)
    fast = torch.zeros(8, heads * head_dim, dtype=dtype, device="cuda")
    slow = torch.zeros_like(fast)
    ks.attention(qkv, fast, step, kv, heads, kv_heads, head_dim, None, head_dim**-0.5)
    step.num_decode_tokens = 0  # every token through the other kernel
    ks.attention(qkv, slow, step, kv, heads, kv_heads, head_dim, None, head_dim**-0.5)
    close(fast, slow, dtype, "decode vs generic")


@pytest.mark.parametrize("vocab", [100, 384, 32771, 151936])
def test_sampling(kernel_sets, vocab):
    ks = kernel_sets[torch.float32]
    rows = 6
    logits = torch.randn(rows, vocab, device="cuda") * 3
    logits[1, 7] = logits[1, 3] = logits[1].max() + 1  # a tie: the lowest index wins
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    ks.sample(logits, None, None, out)
    greedy = logits.argmax(dim=-1).tolist()
    assert [t for r, t in enumerate(out.tolist()) if r != 1] == [t for r, t in enumerate(greedy) if r != 1]
    assert out[1].item() == 3
    temperatures = torch.tensor([0.0, 0.7, 1.0, 1.5, 0.3, 2.0], device="cuda")
    uniforms = torch.tensor([0.5, 0.0, 0.999999, 0.25, 0.5, 0.75], device="cuda")
    ks.sample(logits, temperatures, uniforms, out)
    picks = out.tolist()
    assert picks[0] == int(logits[0].argmax())
    for row in range(1, rows):
        z = logits[row].double() / float(temperatures[row])
        p = torch.exp(z - z.max())
        cdf = torch.cumsum(p, 0) / p.sum()
        u, i = float(uniforms[row]), picks[row]
        below = float(cdf[i - 1]) if i > 0 else 0.0
        assert below - 1e-5 <= u <= float(cdf[i]) + 1e-5, f"row {row}: picked {i}, cdf [{below}, {float(cdf[i])}], u {u}"
    # The distribution over many draws follows the softmax.
    small = torch.tensor([[0.0, 1.0, 2.0, -1.0]], device="cuda").repeat(4000, 1)
    us = torch.rand(4000, device="cuda")
    outs = torch.empty(4000, dtype=torch.int32, device="cuda")
    ks.sample(small, torch.ones(4000, device="cuda"), us, outs)
    freq = torch.bincount(outs.long(), minlength=4).float() / 4000
    assert torch.allclose(freq.cpu(), torch.softmax(small[0].cpu(), -1), atol=0.03)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim,tokens", [(32, 1), (128, 1), (48, 3), (128, 3)])
def test_position_beyond_the_block_table_sets_the_error_word(kernel_sets, dtype, head_dim, tokens):
    """A token whose position lies past the last column of its block table reads nothing outside the
    table: its keys count as missing pages and the error word says so (every attention kernel checks the
    column before it reads the table)."""
    from distie_b200.kernels.library import KernelError

    ks = kernel_sets[dtype]
    page, heads, kv_heads = 16, 4, 2
    kv = filled_cache_for(dtype, kv_heads, head_dim, page, [40, 40])
    width = kv.block_table.shape[1]
    pasts = [40 - tokens, width * page + 5]
    step = step_of([tokens, tokens], pasts, [0, 1])
    qkv = torch.randn(step.num_tokens, (heads + 2 * kv_heads) * head_dim, device="cuda").to(dtype)
    out = torch.zeros(step.num_tokens, heads * head_dim, dtype=dtype, device="cuda")
    ks.attention(qkv, out, step, kv, heads, kv_heads, head_dim, None, head_dim**-0.5)
    with pytest.raises(KernelError, match="block table"):
        ks.check_errors()
    ks.check_errors()  # the word was cleared
    assert torch.isfinite(out.float()).all()

@pytest.mark.parametrize("tokens", [1, 140])
def test_merged_ops_beyond_the_block_table_set_the_error_word(kernel_sets, tokens):
    """The same for the ops that start from the projection: a position past the block table writes no key or value
    anywhere, reads no page, and leaves the error word set (single tokens: the merged attention kernel; a
    portion: the product with the cache write in its epilogue, then the attention)."""
    from distie_b200.kernels.interface import KvSlot, RotaryTable
    from distie_b200.kernels.library import KernelError

    ks = kernel_sets[torch.bfloat16]
    page, heads, kv_heads, head_dim, hidden = 16, 4, 2, 128, 256
    kv = filled_cache_for(torch.bfloat16, kv_heads, head_dim, page, [200, 200])
    before_k, before_v = kv.k.clone(), kv.v.clone()
    width = kv.block_table.shape[1]
    pasts = [200 - tokens, width * page + 5]
    step = step_of([tokens, tokens], pasts, [0, 1])
    n = (heads + 2 * kv_heads) * head_dim
    x = torch.randn(step.num_tokens, hidden, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, hidden, device="cuda") / hidden**0.5).to(torch.bfloat16)
    bias = torch.randn(n, device="cuda")
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))).cuda()
    out = torch.zeros(step.num_tokens, heads * head_dim, dtype=torch.bfloat16, device="cuda")
    ks.qkv_attention(x, w, bias, step, kv, True, RotaryTable(inv_freq, head_dim), heads, kv_heads, head_dim, None, head_dim**-0.5, out)
    with pytest.raises(KernelError, match="block table"):
        ks.check_errors()
    ks.check_errors()
    assert torch.isfinite(out.float()).all()
    # Only the first request's own slots changed.
    changed = ((kv.k != before_k).any(-1) | (kv.v != before_v).any(-1)).nonzero()
    own_pages = set(int(p) for p in kv.block_table[0].tolist() if p >= 0)
    assert len(changed) > 0 and all(int(row[0]) in own_pages for row in changed)
