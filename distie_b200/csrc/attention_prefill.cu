// Tensor-core attention for portions of prompts over the paged cache (bfloat16).
//
// A portion is cut into tiles of 64 consecutive tokens of one request.  One CTA
// (4 warps, 16 query rows each) handles one tile and one query head: it walks the
// keys the tile can see in blocks of 64, S = Q K^T and O += P V on the tensor cores
// (mma.sync.m16n8k16, bfloat16 in, float32 accumulate), with the online softmax in
// float32 registers in between.  Keys and values come straight from the pages: every
// key row is located through the block table and copied with cp.async into
// shared memory (two stages, so the next block loads while this one is computed);
// rows past the last visible key are zero-filled.  Any page size works, because rows
// are addressed one by one.
//
// Visibility is decided per (query row, key): key j is seen by the row at position p
// iff j <= p and (no window or j > p - window).  It depends on positions only, so the
// result does not depend on how the prompt was cut.  head_dim 64 or 128; other sizes
// are refused and the caller uses the size-agnostic kernel.
#include "common.cuh"

namespace distie {

constexpr int kPrefillWarps = 4;
constexpr int kTileM = 64;
constexpr int kTileN = 64;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a [rows][D] bfloat16 tile; chunks are
// XOR-swizzled with the row so that ldmatrix reads hit different banks.
template <int D>
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
  return (uint32_t)((row * (D / 8) + (chunk ^ (row & 7))) * 16);
}

template <int D>
__global__ void __launch_bounds__(kPrefillWarps * 32)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride, __nv_bfloat16* __restrict__ out,
                         int out_row_stride, const int* __restrict__ q_tiles, const int* __restrict__ positions,
                         const int* __restrict__ token_seq, const int* __restrict__ seq_seat,
                         const int* __restrict__ block_table, int table_width,
                         const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                         int group_size, int num_kv_heads, int page_size, int page_shift, int num_pages,
                         int window, float scale_log2, int* __restrict__ error) {
  constexpr int CHUNKS = D / 8;                       // 16-byte chunks per row
  constexpr int TILE_BYTES = kTileN * D * 2;
  constexpr int ROWS_PER_PASS = kPrefillWarps * 32 / CHUNKS;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* k_s = smem;                          // two stages
  unsigned char* v_s = smem + 2 * TILE_BYTES;         // two stages
  unsigned char* q_s = v_s + TILE_BYTES;              // the query tile borrows stage 1 of V: it is read into
                                                      // registers before the first load into that stage

  // Tiles late in a request see the most keys and take longest: start them first.  A tile of the list
  // holds up to 2 * kTileM rows: two CTAs take its halves.
  const int slot = gridDim.y - 1 - blockIdx.y, head = blockIdx.x;
  const int tile = slot >> 1, half = slot & 1;
  const int kv_head = head / group_size;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int t0 = q_tiles[2 * tile] + half * kTileM;
  const int rows = min(kTileM, q_tiles[2 * tile + 1] - half * kTileM);
  if (rows <= 0) return;
  const int p0 = positions[t0];
  const int seat = seq_seat[token_seq[t0]];
  const int* table = block_table + (size_t)seat * table_width;
  const int p_last = p0 + rows - 1;
  const int first_key = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;
  const int kb_start = (first_key / kTileN) * kTileN;
  const int num_blocks = (p_last - kb_start) / kTileN + 1;

  const int my_chunk = threadIdx.x % CHUNKS;
  const int my_row0 = threadIdx.x / CHUNKS;

  // ---- loaders --------------------------------------------------------------------------
  auto load_q = [&]() {
#pragma unroll
    for (int r = my_row0; r < kTileM; r += ROWS_PER_PASS) {
      const bool ok = r < rows;
      const __nv_bfloat16* src = q + (size_t)(t0 + (ok ? r : 0)) * q_row_stride + (size_t)head * D + my_chunk * 8;
      cp_async_16(smem_addr(q_s + tile_offset<D>(r, my_chunk)), src, ok ? 16 : 0);
    }
  };
  auto load_kv = [&](int block, int stage) {
    const int kb = kb_start + block * kTileN;
#pragma unroll
    for (int r = my_row0; r < kTileN; r += ROWS_PER_PASS) {
      const int key = kb + r;
      // (keys before every row's window are not looked up: a cache with a window may have given their page
      // back; their rows are filled with zeros and masked)
      bool ok = key <= p_last && key >= first_key;
      size_t at = 0;
      if (ok) {
        // page_shift >= 0: the page size is a power of two, so no division per row.
        const int column = page_shift >= 0 ? key >> page_shift : key / page_size;
        const int within = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
        const int page = column < table_width ? table[column] : -1;
        if (page < 0 || page >= num_pages) {
          if (error) atomicExch(error, 5);
          ok = false;
        } else {
          at = (((size_t)page * num_kv_heads + kv_head) * page_size + within) * D + my_chunk * 8;
        }
      }
      const uint32_t off = stage * TILE_BYTES + tile_offset<D>(r, my_chunk);
      cp_async_16(smem_addr(k_s + off), k_cache + at, ok ? 16 : 0);
      cp_async_16(smem_addr(v_s + off), v_cache + at, ok ? 16 : 0);
    }
  };

  load_q();
  load_kv(0, 0);
  cp_async_commit();

  uint32_t qf[D / 16][4];
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int r = 0; r < 4; ++r) o[i][r] = 0.f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};
  const int pos_row[2] = {p0 + warp * 16 + g, p0 + warp * 16 + g + 8};

  cp_async_wait<0>();
  __syncthreads();
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    ldmatrix_x4(qf[ks], smem_addr(q_s + tile_offset<D>(row, 2 * ks + (lane >> 4))));
  }
  __syncthreads();  // every warp has its query fragments: stage 1 of V may be overwritten

  for (int block = 0; block < num_blocks; ++block) {
    const int stage = block & 1;
    if (block + 1 < num_blocks) load_kv(block + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    // ---- S = Q K^T ------------------------------------------------------------------------
    float s[kTileN / 8][4];
#pragma unroll
    for (int i = 0; i < kTileN / 8; ++i)
#pragma unroll
      for (int r = 0; r < 4; ++r) s[i][r] = 0.f;
    const unsigned char* k_tile = k_s + stage * TILE_BYTES;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
      for (int np = 0; np < kTileN / 16; ++np) {
        uint32_t b[4];
        const int key_row = np * 16 + (lane & 7) + (lane >> 4) * 8;
        ldmatrix_x4(b, smem_addr(k_tile + tile_offset<D>(key_row, 2 * ks + ((lane >> 3) & 1))));
        mma_16816(s[2 * np], qf[ks], b[0], b[1]);
        mma_16816(s[2 * np + 1], qf[ks], b[2], b[3]);
      }
    }

    // ---- mask, online softmax (base-2 exponentials of scale * log2(e) * S) ------------------
    // Only blocks that touch the diagonal or the window's edge need the per-element test: a block
    // is wholly visible to this warp when its last key is no later than the warp's first row and
    // its first key is inside the window of the warp's last row.
    const int kb = kb_start + block * kTileN;
    const int warp_first = p0 + warp * 16, warp_last = warp_first + 15;
    const bool whole = kb + kTileN - 1 <= warp_first && (window <= 0 || kb > warp_last - window);
    float tile_max[2] = {-INFINITY, -INFINITY};
    if (whole) {
#pragma unroll
      for (int i = 0; i < kTileN / 8; ++i)
#pragma unroll
        for (int r = 0; r < 4; ++r) tile_max[r >> 1] = fmaxf(tile_max[r >> 1], s[i][r]);
    } else {
#pragma unroll
      for (int i = 0; i < kTileN / 8; ++i) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int key = kb + i * 8 + 2 * c + (r & 1);
          const int p = pos_row[r >> 1];
          const bool seen = key <= p && (window <= 0 || key > p - window);
          s[i][r] = seen ? s[i][r] : -INFINITY;
          tile_max[r >> 1] = fmaxf(tile_max[r >> 1], s[i][r]);
        }
      }
    }
    // row_max holds scale_log2 * (largest raw score so far); the scale is positive, so the order is the same.
    float corr[2], shift[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float m = tile_max[h];
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      const float m_new = fmaxf(row_max[h], m * scale_log2);
      corr[h] = (m_new == -INFINITY) ? 1.f : exp2f(row_max[h] - m_new);
      row_max[h] = m_new;
      row_sum[h] *= corr[h];
      shift[h] = m_new == -INFINITY ? 0.f : -m_new;
    }
#pragma unroll
    for (int i = 0; i < kTileN / 8; ++i) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float p = exp2f(fmaf(s[i][r], scale_log2, shift[r >> 1]));  // exp2(-inf) = 0 for hidden keys
        s[i][r] = p;
        row_sum[r >> 1] += p;
      }
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0];
      o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }

    // ---- O += P V ---------------------------------------------------------------------------
    const unsigned char* v_tile = v_s + stage * TILE_BYTES;
#pragma unroll
    for (int kk = 0; kk < kTileN / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        uint32_t b[4];
        const int key_row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldmatrix_x4_trans(b, smem_addr(v_tile + tile_offset<D>(key_row, 2 * dp + (lane >> 4))));
        mma_16816(o[2 * dp], a, b[0], b[1]);
        mma_16816(o[2 * dp + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();  // this stage is overwritten by the load issued two iterations from now
  }
  cp_async_wait<0>();

  // ---- normalise and store ----------------------------------------------------------------------
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float l = row_sum[h];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const int row = warp * 16 + g + 8 * h;
    if (row < rows) {
      __nv_bfloat16* dst = out + (size_t)(t0 + row) * out_row_stride + (size_t)head * D + 2 * c;
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
    }
  }
}

template <int D>
int launch_prefill(const void* q, int q_row_stride, void* out, int out_row_stride, const int* q_tiles, int num_tiles,
                   const int* positions, const int* token_seq, const int* seq_seat, const int* block_table,
                   int table_width, const void* k_cache, const void* v_cache, int num_heads, int num_kv_heads,
                   int page_size, int num_pages, int window, float scale, int* error, cudaStream_t stream) {
  const int shared = 4 * kTileN * D * 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attention_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page_size; ++page_shift) {
    }
  const dim3 grid(num_heads, 2 * num_tiles);
  attention_prefill_kernel<D><<<grid, kPrefillWarps * 32, shared, stream>>>(
      (const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, out_row_stride, q_tiles, positions, token_seq,
      seq_seat, block_table, table_width, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
      num_heads / num_kv_heads, num_kv_heads, page_size, page_shift, num_pages, window,
      scale * 1.4426950408889634f, error);
  DISTIE_LAUNCH_CHECK();
  return 0;
}

}  // namespace distie

using namespace distie;

// Tokens per tile of `q_tiles` ([num_tiles, 2] int32: first token of the tile, number of rows).
extern "C" int distie_attention_prefill_tile(void) { return 2 * kTileM; }

extern "C" int distie_attention_prefill(const void* q, int q_row_stride, void* out, int out_row_stride,
                                        const int* q_tiles, int num_tiles, const int* positions,
                                        const int* token_seq, const int* seq_seat, const int* block_table,
                                        int table_width, const void* k_cache, const void* v_cache, int num_heads,
                                        int num_kv_heads, int head_dim, int page_size, int num_pages, int window,
                                        float scale, int* error, cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads != 0 || page_size < 1 || table_width < 1 ||
      2 * num_tiles > 65535 || (q_row_stride & 7) || (out_row_stride & 1))
    return DISTIE_ERR_ARG;
#define DISTIE_PREFILL(DV)                                                                                        \
  return launch_prefill<DV>(q, q_row_stride, out, out_row_stride, q_tiles, num_tiles, positions, token_seq,       \
                            seq_seat, block_table, table_width, k_cache, v_cache, num_heads, num_kv_heads,        \
                            page_size, num_pages, window, scale, error, stream)
  switch (head_dim) {
    case 64: DISTIE_PREFILL(64);
    case 128: DISTIE_PREFILL(128);
    default: return DISTIE_ERR_UNSUPPORTED;
  }
#undef DISTIE_PREFILL
}
