// Attention of prompt portions over the paged cache on the 5th-generation tensor cores, bfloat16.
//
// A CTA takes one tile of up to 128 consecutive query tokens of a request and one query head, and walks
// the keys the tile may see in blocks of 128:
//
//   S = Q K^T        tcgen05.mma, M = 128 query rows, N = 128 keys, reduction over head_dim;
//                    Q and K are K-major tiles in shared memory (TMA, 128-byte swizzle); S lands in
//                    tensor memory (two buffers of 128 columns, so the next S is computed while the
//                    softmax of this one runs)
//   P = softmax part eight warps, two threads per query row (64 keys each; the row maxima and, at the end,
//                    the row sums of the two meet in shared memory): tcgen05.ld of the row, mask,
//                    running maximum and sum in float32, exp2, P as bfloat16 into shared memory in the
//                    K-major swizzled layout of an A operand
//   O += P V         tcgen05.mma, N = head_dim, reduction over the 128 keys; V stays as the cache holds
//                    it (a key per row, head_dim contiguous), which for this product is an MN-major
//                    B operand; O accumulates in tensor memory
//
// Keys and values come straight from their pages: a page of the cache is page_size rows of head_dim, so
// one TMA box of [page_size x 64] per page and half of the head fills its rows of the 128-key tile.
// Pages past the last key the tile needs are not fetched.
//
// The running maximum is only raised when a row's new maximum exceeds the one in use by more than 8
// (in base-2 units): P then stays below 2^8, the sums stay exact in float32, and O needs to be read,
// scaled and written back only on those blocks.  Normalisation by the row sum happens once, at the end.
//
// Rows of V that belong to no key of the request (the rest of its last page, pages that were not
// fetched) are set to zero in shared memory before the product, since 0 * garbage need not be 0.
//
//   warp 0      producer: TMA loads of Q, then K and V blocks through two stages each (a lane per page)
//   warp 1      allocates tensor memory; one lane issues the MMAs and commits them to mbarriers
//   warps 2..9  softmax, correction of O, final normalisation and store
//
// Every wait on an mbarrier is bounded; when one runs out the CTA sets the error word to 6, every role
// stops at its next wait, the producer waits (bounded) for its copies in flight, and tensor memory is
// released.  head_dim 64 or 128; page sizes 8, 16, ..., 128.
#include "tcgen05.cuh"

namespace distie {

constexpr int kAttnRows = 128;     // query rows of a tile = lanes of tensor memory
constexpr int kAttnKeys = 128;     // keys per block
constexpr int kAttnSoftmaxWarps = 8;
constexpr int kAttnThreads = (2 + kAttnSoftmaxWarps) * 32;
constexpr int kAttnStages = 2;
constexpr int kAttnHalf = kAttnRows * 128;  // bytes of one [128 rows x 64 elements] swizzled half tile
constexpr float kAttnRaise = 8.f;  // the maximum in use is raised when a row exceeds it by this much (base 2)

template <int D>
struct AttnShared {
  alignas(1024) unsigned char q[kAttnRows * D * 2];
  alignas(1024) unsigned char k[kAttnStages][kAttnKeys * D * 2];
  alignas(1024) unsigned char v[kAttnStages][kAttnKeys * D * 2];
  alignas(1024) unsigned char p[kAttnRows * kAttnKeys * 2];
  uint64_t q_full;
  uint64_t k_full[kAttnStages], k_empty[kAttnStages];
  uint64_t v_full[kAttnStages], v_empty[kAttnStages];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full, pv_done;
  uint64_t max_ready[2], sum_ready;
  float row_max[2][2][kAttnRows];  // [S buffer][side][row]: the maxima the two threads of a row exchange
  float row_sum[2][kAttnRows];
  uint32_t tmem_base;
  uint32_t failed;
};

__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                                 int out_row_stride, const int* __restrict__ q_tiles,
                                 const int* __restrict__ positions, const int* __restrict__ token_seq,
                                 const int* __restrict__ seq_seat, const int* __restrict__ block_table,
                                 int table_width, int group_size, int num_kv_heads, int page_shift, int num_pages,
                                 int window, float scale_log2, int* __restrict__ error) {
  extern __shared__ unsigned char raw[];
  auto& sm = *reinterpret_cast<AttnShared<D>*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  constexpr int HALVES = D / 64;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t O_COL = 256;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile uint32_t* failed = &sm.failed;

  if (threadIdx.x == 0) {
    mbar_init(&sm.q_full, 1);
    for (int s = 0; s < kAttnStages; ++s) {
      mbar_init(&sm.k_full[s], 1);
      mbar_init(&sm.k_empty[s], 1);
      mbar_init(&sm.v_full[s], 1);
      mbar_init(&sm.v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.s_full[b], 1);
      mbar_init(&sm.s_empty[b], kAttnSoftmaxWarps);  // one arrival per softmax warp
      mbar_init(&sm.max_ready[b], kAttnSoftmaxWarps);
    }
    mbar_init(&sm.sum_ready, kAttnSoftmaxWarps);
    mbar_init(&sm.p_full, kAttnSoftmaxWarps);
    mbar_init(&sm.pv_done, 1);
    sm.failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = sm.tmem_base;

  grid_dependency_release();
  grid_dependency_wait();  // q and the newest keys and values come from the kernel before this one

  // Tiles late in a request see the most keys and take longest: they start first, for every head
  // (blockIdx.x, the heads, runs fastest in the order in which CTAs are handed out).
  const int tile = gridDim.y - 1 - blockIdx.y, head = blockIdx.x;
  const int kv_head = head / group_size;
  const int t0 = q_tiles[2 * tile], rows = q_tiles[2 * tile + 1];
  const int pos0 = positions[t0];
  const int seat = seq_seat[token_seq[t0]];
  const int last_pos = pos0 + rows - 1;
  const int first_key = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const int block_first = first_key / kAttnKeys;
  const int blocks = last_pos / kAttnKeys - block_first + 1;
  const int page_size = 1 << page_shift;

  if (warp == 0) {
    // ---- producer: lane pg looks up page pg of a block and issues its copies -------------------------------
    if (lane == 0) {
      mbar_expect_tx(&sm.q_full, kAttnRows * D * 2);
      for (int h = 0; h < HALVES; ++h) tma_load_2d(sm.q + h * kAttnHalf, &map_q, &sm.q_full, head * D + h * 64, t0);
    }
    const int* table = block_table + (size_t)seat * table_width;
    const int pages_per_block = kAttnKeys >> page_shift;  // at most 16
    int issued_k = 0, issued_v = 0;  // blocks whose K (V) copies have been issued
    bool ok = true;
    // Pages of block j that hold keys the tile needs, this lane's page and its first row in the cache.
    int count = 0, row = 0;
    auto look_up = [&](int j) {
      const int key0 = (block_first + j) * kAttnKeys;
      count = min(pages_per_block, ((last_pos - key0) >> page_shift) + 1);
      const int column = (key0 >> page_shift) + lane;
      const int page = (lane < count && column < table_width) ? table[column] : -1;
      row = (page * num_kv_heads + kv_head) * page_size;
      if (__any_sync(0xffffffffu, lane < count && (page < 0 || page >= num_pages))) {
        if (lane == 0 && error) atomicExch(error, 4);
        return false;
      }
      return true;
    };
    auto copy = [&](unsigned char* stage, const CUtensorMap* map, uint64_t* full, uint64_t* empty, int j, int& issued) {
      if (!__all_sync(0xffffffffu, mbar_wait_unless(empty, ((j >> 1) & 1) ^ 1, failed))) return false;
      if (lane == 0) mbar_expect_tx(full, (uint32_t)count * page_size * D * 2);
      __syncwarp();
      if (lane < count)
        for (int h = 0; h < HALVES; ++h)
          tma_load_2d(stage + h * kAttnHalf + lane * page_size * 128, map, full, h * 64, row);
      issued = j + 1;
      return true;
    };
    // K runs a block ahead of V: K of block j + 1 only waits for S of block j - 1, which is done early,
    // while V of block j waits for the product of block j - 2.
    ok = look_up(0) && copy(sm.k[0], &map_k, &sm.k_full[0], &sm.k_empty[0], 0, issued_k);
    for (int j = 0; j < blocks && ok; ++j) {
      const int s = j & 1;
      const int count_now = count, row_now = row;
      if (j + 1 < blocks) {
        ok = look_up(j + 1) && copy(sm.k[s ^ 1], &map_k, &sm.k_full[s ^ 1], &sm.k_empty[s ^ 1], j + 1, issued_k);
        if (!ok) break;
      }
      const int count_next = count, row_next = row;
      count = count_now;
      row = row_now;
      ok = copy(sm.v[s], &map_v, &sm.v_full[s], &sm.v_empty[s], j, issued_v);
      count = count_next;
      row = row_next;
    }
    if (!ok) atomicExch(&sm.failed, 1u);
    if (sm.failed && lane == 0) {
      // Copies already under way must land before the CTA may leave: wait (bounded) for the last few.
      mbar_wait(&sm.q_full, 0);
      for (int j = max(0, issued_k - 2); j < issued_k; ++j) mbar_wait(&sm.k_full[j & 1], (j >> 1) & 1);
      for (int j = max(0, issued_v - 2); j < issued_v; ++j) mbar_wait(&sm.v_full[j & 1], (j >> 1) & 1);
    }
  } else if (warp == 1) {
    // ---- MMA issuer ------------------------------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = instr_desc(kAttnKeys);
      constexpr uint32_t idesc_o = instr_desc(D, true);
      const uint64_t q_desc = smem_desc(sm.q), p_desc = smem_desc(sm.p);
      bool ok = mbar_wait_unless(&sm.q_full, 0, failed);
      auto issue_s = [&](int j) {
        const int s = j & 1;
        if (!mbar_wait_unless(&sm.k_full[s], (j >> 1) & 1, failed)) return false;
        if (!mbar_wait_unless(&sm.s_empty[s], ((j >> 1) & 1) ^ 1, failed)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t k_desc = smem_desc(sm.k[s]);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t step = (uint64_t)(((kk >> 2) * kAttnHalf + (kk & 3) * 32) >> 4);
          umma_bf16(tmem + s * kAttnKeys, q_desc + step, k_desc + step, idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&sm.k_empty[s]);
        umma_commit(&sm.s_full[s]);
        return true;
      };
      ok = ok && issue_s(0);
      for (int j = 0; j < blocks && ok; ++j) {
        const int s = j & 1;
        if (j + 1 < blocks) ok = issue_s(j + 1);
        if (!ok) break;
        if (!mbar_wait_unless(&sm.p_full, j & 1, failed)) { ok = false; break; }
        if (!mbar_wait_unless(&sm.v_full[s], (j >> 1) & 1, failed)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t v_desc = smem_desc_mn(sm.v[s], kAttnHalf, 1024);
#pragma unroll
        for (int kk = 0; kk < kAttnKeys / 16; ++kk) {
          const uint64_t p_step = (uint64_t)(((kk >> 2) * kAttnHalf + (kk & 3) * 32) >> 4);
          const uint64_t v_step = (uint64_t)((kk * 16 * 128) >> 4);
          umma_bf16(tmem + O_COL, p_desc + p_step, v_desc + v_step, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&sm.v_empty[s]);
        umma_commit(&sm.pv_done);
      }
      if (!ok) atomicExch(&sm.failed, 1u);
    }
  } else {
    // ---- softmax, correction, epilogue: two threads per query row, 64 keys (and half of O) each ---------------
    const int quadrant = warp & 3;
    const int side = (warp - 2) >> 2;  // which half of the block's keys and of O's columns
    const int r = quadrant * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(quadrant * 32) << 16);
    const int limit = min(pos0 + r, last_pos);                      // newest key this row may see
    const int oldest = window > 0 ? pos0 + r - window + 1 : 0;      // oldest key inside its window
    constexpr int SIDE_KEYS = kAttnKeys / 2, SIDE_DIMS = D / 2;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    // The warp waits as one: the tensor-memory instructions below need all of its lanes.
    auto wait_all = [&](uint64_t* bar, uint32_t parity) {
      return __all_sync(0xffffffffu, mbar_wait_unless(bar, parity, failed));
    };
    for (int j = 0; j < blocks; ++j) {
      const int s = j & 1;
      const int key0 = (block_first + j) * kAttnKeys + side * SIDE_KEYS;  // first key of this thread's half
      if (!wait_all(&sm.s_full[s], (j >> 1) & 1)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // No row of the tile needs a mask when every key of the block is old enough and inside every window.
      const int block_key0 = (block_first + j) * kAttnKeys;
      const bool unmasked =
          block_key0 + kAttnKeys - 1 <= pos0 && (window <= 0 || block_key0 >= last_pos - window + 1);
      const uint32_t s_addr = lane_base + s * kAttnKeys + side * SIDE_KEYS;
      // Pass 1: the row's maximum over this half of the block (kept in registers for pass 2); the two
      // halves meet in shared memory.  Four running maxima, so that the chain of dependent operations is short.
      uint32_t sv[SIDE_KEYS];
      tmem_load_64(s_addr, sv);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      // This warp has its part of S in registers: the buffer may be overwritten.
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.s_empty[s]);
      if (!unmasked) {
#pragma unroll
        for (int i = 0; i < SIDE_KEYS; ++i) {
          const int key = key0 + i;
          if (!(key <= limit && key >= oldest)) sv[i] = 0xff800000u;  // -inf
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < SIDE_KEYS; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[i]));
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      sm.row_max[s][side][r] = mx;
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.max_ready[s]);  // release: the store above is ordered before it
      if (!wait_all(&sm.max_ready[s], (j >> 1) & 1)) { ok = false; break; }
      mx = fmaxf(mx, sm.row_max[s][side ^ 1][r]);
      const float m_new = fmaxf(m_used, mx * scale_log2);
      const bool raise = m_new > m_used + kAttnRaise || (m_used == -INFINITY && m_new > -INFINITY);
      float corr = 1.f;
      if (raise) {
        corr = m_used == -INFINITY ? 0.f : exp2_approx(m_used - m_new);
        m_used = m_new;
      }
      l *= corr;
      const bool any_raise = __any_sync(0xffffffffu, raise);
      // P and O are in use by the product of the block before this one until it has completed.
      if (j > 0) {
        if (!wait_all(&sm.pv_done, (j - 1) & 1)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (any_raise) {
#pragma unroll
          for (int c0 = 0; c0 < SIDE_DIMS; c0 += 32) {
            uint32_t v[32];
            tmem_load_32(lane_base + O_COL + side * SIDE_DIMS + c0, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
            tmem_store_32(lane_base + O_COL + side * SIDE_DIMS + c0, v);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
      }
      // Pass 2: P = exp2(S * scale - maximum in use), its sum, and P as bfloat16 into the A-operand tile
      // (this thread's 64 keys are one swizzled half of it).  A masked S is -inf and gives 0.
      const float shift = m_used == -INFINITY ? 0.f : m_used;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      unsigned char* row_base = sm.p + side * kAttnHalf + r * 128;
#pragma unroll
      for (int c0 = 0; c0 < SIDE_KEYS; c0 += 8) {
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          const float p0 = exp2_approx(fmaf(__uint_as_float(sv[c0 + i]), scale_log2, -shift));
          const float p1 = exp2_approx(fmaf(__uint_as_float(sv[c0 + i + 1]), scale_log2, -shift));
          sum4[(i >> 1) & 3] += p0 + p1;
          const __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
          packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&pair);
        }
        const int chunk = c0 >> 3;
        *reinterpret_cast<uint4*>(row_base + ((chunk ^ (r & 7)) << 4)) =
            make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      // Rows of V past the last key the tile needs: zero, so that P = 0 gives 0 (side 0 does it).
      if (block_key0 + kAttnKeys - 1 > last_pos && side == 0) {
        if (!wait_all(&sm.v_full[s], (j >> 1) & 1)) { ok = false; break; }
        if (block_key0 + r > last_pos) {
#pragma unroll
          for (int h = 0; h < HALVES; ++h) {
            uint4* dst = reinterpret_cast<uint4*>(sm.v[s] + h * kAttnHalf + r * 128);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      }
      // P (and the zeroed rows) written by this thread become visible to the tensor core's reads.
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.p_full);
    }
    if (!ok) atomicExch(&sm.failed, 1u);
    // ---- epilogue: O / l; the two sides of a row add their sums -----------------------------------------------
    sm.row_sum[side][r] = l;
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.sum_ready);
    if (ok && wait_all(&sm.sum_ready, 0) && wait_all(&sm.pv_done, (blocks - 1) & 1)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      l += sm.row_sum[side ^ 1][r];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = out + (size_t)(t0 + r) * out_row_stride + (size_t)head * D + side * SIDE_DIMS;
#pragma unroll
      for (int c0 = 0; c0 < SIDE_DIMS; c0 += 32) {
        uint32_t v[32];
        tmem_load_32(lane_base + O_COL + side * SIDE_DIMS + c0, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (r < rows) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            float y[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = __uint_as_float(v[i + e]) * inv;
            store8(dst + c0 + i, y);
          }
        }
      }
    } else {
      atomicExch(&sm.failed, 1u);
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
  }
  if (threadIdx.x == 0 && sm.failed && error) atomicCAS(error, 0, 6);
}

template <int D>
static int launch_attention_tc(const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v, void* out,
                               int out_row_stride, const int* q_tiles, int num_tiles, const int* positions,
                               const int* token_seq, const int* seq_seat, const int* block_table, int table_width,
                               int num_heads, int num_kv_heads, int page_shift, int num_pages, int window,
                               float scale_log2, int* error, cudaStream_t stream) {
  const size_t shared = sizeof(AttnShared<D>) + 1024;
  static bool configured = false;
  if (!configured) {
    const cudaError_t err = cudaFuncSetAttribute(attention_prefill_tcgen05_kernel<D>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  const cudaError_t err = launch_dependent_family(
      32, attention_prefill_tcgen05_kernel<D>, dim3(num_heads, num_tiles), dim3(kAttnThreads), shared, stream, map_q,
      map_k, map_v, (__nv_bfloat16*)out, out_row_stride, q_tiles, positions, token_seq, seq_seat, block_table,
      table_width, num_heads / num_kv_heads, num_kv_heads, page_shift, num_pages, window, scale_log2, error);
  return err == cudaSuccess ? 0 : (int)err;
}

}  // namespace distie

using namespace distie;

// Tokens per tile of `q_tiles` ([num_tiles, 2] int32: first token of the tile, number of rows <= 128).
// q is [tokens, >= num_heads * head_dim] bfloat16 with row stride q_row_stride; the caches are
// [num_pages, num_kv_heads, page_size, head_dim].  Returns DISTIE_ERR_UNSUPPORTED for a head_dim other
// than 64 and 128 or a page size that is not 8, 16, ..., 128.
extern "C" int distie_attention_prefill_tcgen05(const void* q, int q_row_stride, void* out, int out_row_stride,
                                                const int* q_tiles, int num_tiles, const int* positions,
                                                const int* token_seq, const int* seq_seat, const int* block_table,
                                                int table_width, const void* k_cache, const void* v_cache, int tokens,
                                                int num_heads, int num_kv_heads, int head_dim, int page_size,
                                                int num_pages, int window, float scale, int* error,
                                                cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (tokens < 1 || num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads != 0 || table_width < 1 ||
      num_pages < 1 || num_tiles > 65535)
    return DISTIE_ERR_ARG;
  if ((head_dim != 64 && head_dim != 128) || page_size < 8 || page_size > 128 || (page_size & (page_size - 1)) ||
      (q_row_stride & 7) || (out_row_stride & 7) || ((uintptr_t)q & 15) || ((uintptr_t)out & 15) ||
      ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
    return DISTIE_ERR_UNSUPPORTED;
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  CUtensorMap map_q, map_k, map_v;
  int status = make_map(&map_q, q, tokens, num_heads * head_dim, q_row_stride, kAttnRows);
  if (status != 0) return status;
  const long long cache_rows = (long long)num_pages * num_kv_heads * page_size;
  if (cache_rows > 0x7fffffffLL) return DISTIE_ERR_UNSUPPORTED;
  if ((status = make_map(&map_k, k_cache, (int)cache_rows, head_dim, head_dim, page_size)) != 0) return status;
  if ((status = make_map(&map_v, v_cache, (int)cache_rows, head_dim, head_dim, page_size)) != 0) return status;
  const float scale_log2 = scale * 1.4426950408889634f;
  if (head_dim == 64)
    return launch_attention_tc<64>(map_q, map_k, map_v, out, out_row_stride, q_tiles, num_tiles, positions, token_seq,
                                   seq_seat, block_table, table_width, num_heads, num_kv_heads, page_shift, num_pages,
                                   window, scale_log2, error, stream);
  return launch_attention_tc<128>(map_q, map_k, map_v, out, out_row_stride, q_tiles, num_tiles, positions, token_seq,
                                  seq_seat, block_table, table_width, num_heads, num_kv_heads, page_shift, num_pages,
                                  window, scale_log2, error, stream);
}
