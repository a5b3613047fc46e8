// Attention of prompt portions over the paged cache on the 5th-generation tensor cores, bfloat16.
//
// A CTA takes one tile of up to 128 consecutive query tokens of a request and one query head, and walks
// the keys the tile may see in blocks of 128:
//
//   S = Q K^T        tcgen05.mma, M = 128 query rows, N = 128 keys, reduction over head_dim;
//                    Q and K are K-major tiles in shared memory (TMA, 128-byte swizzle); S lands in
//                    tensor memory (two buffers of 128 columns, so the next S is computed while the
//                    softmax of this one runs)
//   P = softmax part eight warps in two groups of four: group 0 owns keys 0..63 of every block, group 1 keys
//                    64..127, a thread per query row in each.  The groups are two softmax streams of
//                    their own -- running maximum, sum and an O accumulator each -- and never wait
//                    for one another inside the loop, so one group's exponentials (16 a clock and SM)
//                    overlap the other's loads, maxima and waits.  P goes back into the first 32 of the
//                    group's 64 columns of S as bfloat16, two keys to a column
//   O_g += P_g V_g   tcgen05.mma with P as the A operand straight from tensor memory, N = head_dim,
//                    reduction over the group's 64 keys; V stays as the cache holds it (a key per row,
//                    head_dim contiguous), which for this product is an MN-major B operand
//   end              the two partial results of a row are brought to a common maximum, added and
//                    divided by the common sum
//
//   tensor memory    S0 | S1 | O of group 0 | O of group 1 (128 + 128 + head_dim + head_dim columns)
//   MMA order        PV0(j), PV1(j), S(j + 2): the S that overwrites a block's P is issued behind the
//                    products that read it (MMAs of one thread execute in the order of issue)
//
// Keys and values come straight from their pages: a page of the cache is page_size rows of head_dim, so
// one TMA box of [page_size x 64] per page and half of the head fills its rows of the 128-key tile.
// Pages past the last key the tile needs are not fetched.  The page ids of a block are read from the
// table one block ahead of their use, by two producer warps (K and V), so that neither the look-up nor
// the other operand's stage stands between a stage becoming free and its copies being issued.
//
// The running maximum is only raised when a row's new maximum exceeds the one in use by more than 8
// (in base-2 units): P then stays below 2^8, the sums stay exact in float32, and O needs to be read,
// scaled and written back only on those blocks.  Normalisation by the row sum happens once, at the end.
//
// Rows of V that belong to no key of the request (the rest of its last page, pages that were not
// fetched) are set to zero in shared memory before the product, since 0 * garbage need not be 0.
//
//   warp 0      producer: TMA loads of Q, then K blocks through two stages (a lane per page)
//   warp 1      allocates tensor memory; one lane issues the MMAs and commits them to mbarriers
//   warps 2..9  softmax, correction of O, final merge and store
//   warp 10     producer of the V blocks, three stages
//
// Every wait on an mbarrier is bounded; when one runs out the CTA sets the error word to 6, every role
// stops at its next wait, the producers wait (bounded) for their copies in flight, and tensor memory is
// released.  head_dim 64 or 128; page sizes 8, 16, ..., 128.
#include "tcgen05.cuh"

namespace distie {

constexpr int kAttnRows = 128;     // query rows of a tile = lanes of tensor memory
constexpr int kAttnKeys = 128;     // keys per block
constexpr int kAttnGroupKeys = kAttnKeys / 2;  // keys of a block that one softmax group owns
constexpr int kAttnSoftmaxWarps = 8;
constexpr int kAttnVProducerWarp = 2 + kAttnSoftmaxWarps;  // behind the softmax warps
constexpr int kAttnThreads = (3 + kAttnSoftmaxWarps) * 32;
constexpr int kAttnKStages = 2, kAttnVStages = 3;  // V of a block is needed a block time after its stage is freed, K two
constexpr int kAttnHalf = kAttnRows * 128;  // bytes of one [128 rows x 64 elements] swizzled half tile
constexpr float kAttnRaise = 8.f;  // the maximum in use is raised when a row exceeds it by this much (base 2)

template <int D>
struct AttnShared {
  alignas(1024) unsigned char q[kAttnRows * D * 2];
  alignas(1024) unsigned char k[kAttnKStages][kAttnKeys * D * 2];
  alignas(1024) unsigned char v[kAttnVStages][kAttnKeys * D * 2];
  uint64_t q_full;
  uint64_t k_full[kAttnKStages], k_empty[kAttnKStages];
  uint64_t v_full[kAttnVStages], v_empty[kAttnVStages];
  uint64_t s_full[2];
  uint64_t p_full[2][2];  // [group][S buffer]
  uint64_t pv_done[2];    // [group]
  uint64_t merge_ready;
  uint64_t store_ready;   // the eight softmax warps have put their part of the output tile into shared memory
  float row_max[2][kAttnRows], row_sum[2][kAttnRows];  // [group][row]: what the groups exchange at the end
  uint32_t tmem_base;
  uint32_t failed;
};

__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// The softmax warps are bound by the number of instructions they issue (two warps to a scheduler, long chains of
// dependent operations), so the loop over a block's scores uses the forms that do two things at once: the maximum
// of three values, and float32 arithmetic on pairs of values in a 64-bit register (same rounding per value).
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t pair_of(float lo, float hi) {
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void halves_of(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_pairs(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_pairs(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

template <int D>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v,
                                 const __grid_constant__ CUtensorMap map_out, __nv_bfloat16* __restrict__ out,
                                 int out_row_stride, const int* __restrict__ q_tiles,
                                 const int* __restrict__ positions, const int* __restrict__ token_seq,
                                 const int* __restrict__ seq_seat, const int* __restrict__ block_table,
                                 int table_width, int group_size, int num_kv_heads, int page_shift, int num_pages,
                                 int window, float scale_log2, int* __restrict__ error) {
  extern __shared__ unsigned char raw[];
  auto& sm = *reinterpret_cast<AttnShared<D>*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  constexpr int HALVES = D / 64;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t O_COL = 256;  // S0 | S1 | O of group 0 | O of group 1
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile uint32_t* failed = &sm.failed;

  if (threadIdx.x == 64) {
    prefetch_tensor_map(&map_q);
    prefetch_tensor_map(&map_k);
    prefetch_tensor_map(&map_v);
    prefetch_tensor_map(&map_out);
  }
  if (threadIdx.x == 0) {
    mbar_init(&sm.q_full, 1);
    for (int s = 0; s < kAttnKStages; ++s) {
      mbar_init(&sm.k_full[s], 1);
      mbar_init(&sm.k_empty[s], 1);
    }
    for (int s = 0; s < kAttnVStages; ++s) {
      mbar_init(&sm.v_full[s], 1);
      mbar_init(&sm.v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.s_full[b], 1);
      // One barrier per group and S buffer: a group may be a block ahead of the MMA issuer, never two
      // on one buffer (the S of block j + 2 is issued only after the P of block j has been seen).
      mbar_init(&sm.p_full[0][b], kAttnSoftmaxWarps / 2);  // one arrival per warp of the group
      mbar_init(&sm.p_full[1][b], kAttnSoftmaxWarps / 2);
      mbar_init(&sm.pv_done[b], 1);
    }
    mbar_init(&sm.merge_ready, kAttnSoftmaxWarps);
    mbar_init(&sm.store_ready, kAttnSoftmaxWarps);
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
  // The tile's place in the step (tiles, positions, seats and block tables are inputs of the step, written by
  // no kernel) is looked up before the wait for the kernel that makes q and the newest keys and values: four
  // loads that depend on one another, which then cost the CTAs of the first wave nothing.
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
  const int* table = block_table + (size_t)seat * table_width;
  const int pages_per_block = kAttnKeys >> page_shift;  // at most 16
  auto pages_of = [&](int j) {  // pages of block j up to the last one that holds keys the tile needs
    return min(pages_per_block, ((last_pos - (block_first + j) * kAttnKeys) >> page_shift) + 1);
  };
  // Pages of the first block that lie wholly before the oldest key any row of the tile sees: a cache with a
  // window may have given them back already, so they are neither looked up nor fetched (their rows of the
  // tile are masked as keys and cleared as values).
  const int skipped0 = (first_key - block_first * kAttnKeys) >> page_shift;
  auto skipped = [&](int j) { return j == 0 ? skipped0 : 0; };
  auto read_table = [&](int j) {  // this lane's page of block j, -1 outside the block's pages
    if (j >= blocks) return -1;
    const int column = (((block_first + j) * kAttnKeys) >> page_shift) + lane;
    return (lane >= skipped(j) && lane < pages_of(j) && column < table_width) ? __ldg(table + column) : -1;
  };
  const bool producer = warp == 0 || warp == kAttnVProducerWarp;
  int page_ahead = producer ? read_table(0) : -1;
  grid_dependency_wait();  // q and the newest keys and values come from the kernel before this one

  if (producer) {
    // ---- producers: warp 0 fetches Q and K, the last warp V; lane pg takes page pg of a block -----------------
    const bool for_k = warp == 0;
    if (for_k && lane == 0) {
      mbar_expect_tx(&sm.q_full, kAttnRows * D * 2);
      for (int h = 0; h < HALVES; ++h) tma_load_2d(sm.q + h * kAttnHalf, &map_q, &sm.q_full, head * D + h * 64, t0);
    }
    const int stages = for_k ? kAttnKStages : kAttnVStages;
    const CUtensorMap* map = for_k ? &map_k : &map_v;
    uint64_t* full = for_k ? sm.k_full : sm.v_full;
    uint64_t* empty = for_k ? sm.k_empty : sm.v_empty;
    int issued = 0;
    bool ok = true;
    for (int j = 0; j < blocks && ok; ++j) {
      const int s = j % stages, use = j / stages;
      const int page = page_ahead;
      page_ahead = read_table(j + 1);
      const int count = pages_of(j), from = skipped(j);
      if (__any_sync(0xffffffffu, lane >= from && lane < count && (page < 0 || page >= num_pages))) {
        if (lane == 0 && error) atomicExch(error, 5);
        ok = false;
        break;
      }
      if (!__all_sync(0xffffffffu, mbar_wait_unless(&empty[s], (use & 1) ^ 1, failed))) { ok = false; break; }
      if (lane == 0) mbar_expect_tx(&full[s], (uint32_t)(count - from) * page_size * D * 2);
      __syncwarp();
      if (lane >= from && lane < count) {
        unsigned char* stage = (for_k ? sm.k[s] : sm.v[s]) + lane * page_size * 128;
        const int row = (page * num_kv_heads + kv_head) * page_size;
        for (int h = 0; h < HALVES; ++h) tma_load_2d(stage + h * kAttnHalf, map, &full[s], h * 64, row);
      }
      issued = j + 1;
    }
    if (!ok) atomicExch(&sm.failed, 1u);
    if (sm.failed && lane == 0) {
      // Copies already under way must land before the CTA may leave: wait (bounded) for the last few.
      if (for_k) mbar_wait(&sm.q_full, 0);
      for (int j = max(0, issued - stages); j < issued; ++j) mbar_wait(&full[j % stages], (j / stages) & 1);
    }
  } else if (warp == 1) {
    // ---- MMA issuer ------------------------------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = instr_desc(kAttnKeys);
      constexpr uint32_t idesc_o = instr_desc(D, true);
      const uint64_t q_desc = smem_desc(sm.q);
      bool ok = mbar_wait_unless(&sm.q_full, 0, failed);
      // S of block j into buffer j & 1.  Both groups have that buffer's last S in registers and their P
      // consumed: the caller has seen both P of block j - 2 and issued the products that read them.
      auto issue_s = [&](int j) {
        const int s = j & 1, ks = j % kAttnKStages;
        if (!mbar_wait_unless(&sm.k_full[ks], (j / kAttnKStages) & 1, failed)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t k_desc = smem_desc(sm.k[ks]);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t step = (uint64_t)(((kk >> 2) * kAttnHalf + (kk & 3) * 32) >> 4);
          umma_bf16(tmem + s * kAttnKeys, q_desc + step, k_desc + step, idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&sm.k_empty[ks]);
        umma_commit(&sm.s_full[s]);
        return true;
      };
      ok = ok && issue_s(0);
      if (ok && blocks > 1) ok = issue_s(1);
      for (int j = 0; j < blocks && ok; ++j) {
        const int s = j & 1, vs = j % kAttnVStages;
        if (!mbar_wait_unless(&sm.v_full[vs], (j / kAttnVStages) & 1, failed)) { ok = false; break; }
        const uint64_t v_desc = smem_desc_mn(sm.v[vs], kAttnHalf, 1024);
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          if (!mbar_wait_unless(&sm.p_full[g][s], (j >> 1) & 1, failed)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int kk = 0; kk < kAttnGroupKeys / 16; ++kk) {
            // P of the group: 32 columns at the start of its half of the S buffer, 16 keys are 8 columns;
            // its keys are rows g * 64 ... of the V block.
            const uint64_t v_step = (uint64_t)(((g * kAttnGroupKeys + kk * 16) * 128) >> 4);
            umma_bf16_ts(tmem + O_COL + g * D, tmem + s * kAttnKeys + g * kAttnGroupKeys + kk * 8, v_desc + v_step,
                         idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&sm.pv_done[g]);
        }
        if (!ok) break;
        umma_commit(&sm.v_empty[vs]);
        if (j + 2 < blocks) ok = issue_s(j + 2);
      }
      if (!ok) atomicExch(&sm.failed, 1u);
    }
  } else if (warp < kAttnVProducerWarp) {
    // ---- softmax, correction, epilogue: group g owns 64 keys of every block, thread = query row ---------------
    const int quadrant = warp & 3;
    const int g = (warp - 2) >> 2;
    const int r = quadrant * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(quadrant * 32) << 16);
    const uint32_t o_addr = lane_base + O_COL + g * D;
    const int limit = min(pos0 + r, last_pos);                      // newest key this row may see
    const int oldest = window > 0 ? pos0 + r - window + 1 : 0;      // oldest key inside its window
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    // One lane polls the barrier; the warp continues as one (the tensor-memory instructions need all lanes).
    auto wait_all = [&](uint64_t* bar, uint32_t parity) {
      int done = 1;
      if (lane == 0) done = mbar_wait_unless(bar, parity, failed) ? 1 : 0;
      done = __shfl_sync(0xffffffffu, done, 0);
      __syncwarp();
      return done != 0;
    };
    for (int j = 0; j < blocks; ++j) {
      const int s = j & 1, vs = j % kAttnVStages;
      const int block_key0 = (block_first + j) * kAttnKeys;
      const int key0 = block_key0 + g * kAttnGroupKeys;  // first key of this group's part
      const uint32_t s_addr = lane_base + s * kAttnKeys + g * kAttnGroupKeys;
      if (!wait_all(&sm.s_full[s], (j >> 1) & 1)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // No row of the tile needs a mask when every key of the block is old enough and inside every window.
      const bool unmasked =
          block_key0 + kAttnKeys - 1 <= pos0 && (window <= 0 || block_key0 >= last_pos - window + 1);
      uint32_t sv[kAttnGroupKeys];
      tmem_load_64(s_addr, sv);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (!unmasked) {
#pragma unroll
        for (int i = 0; i < kAttnGroupKeys; ++i) {
          const int key = key0 + i;
          if (!(key <= limit && key >= oldest)) sv[i] = 0xff800000u;  // -inf
        }
      }
      // The row's maximum over the group's keys: four running maxima keep the chain of dependent operations short.
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < kAttnGroupKeys; i += 2)
        mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m_used, mx * scale_log2);
      const bool raise = m_new > m_used + kAttnRaise || (m_used == -INFINITY && m_new > -INFINITY);
      float corr = 1.f;
      if (raise) {
        corr = m_used == -INFINITY ? 0.f : exp2_approx(m_used - m_new);
        m_used = m_new;
      }
      l *= corr;
      // The group's O is in use by its product of the block before this one until that has completed.
      if (j > 0 && __any_sync(0xffffffffu, raise)) {
        if (!wait_all(&sm.pv_done[g], (j - 1) & 1)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t v[32];
          tmem_load_32(o_addr + c0, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
          tmem_store_32(o_addr + c0, v);
        }
      }
      // P = exp2(S * scale - maximum in use) and its sum; P as bfloat16, two keys to a column, into the
      // first 32 of the group's 64 columns of this S buffer (the thread has its S in registers).  A
      // masked S is -inf and gives 0.
      const float shift = m_used == -INFINITY ? 0.f : m_used;
      uint64_t sum4[4] = {0ull, 0ull, 0ull, 0ull};  // four pairs of running sums
      const uint64_t scale2 = pair_of(scale_log2, scale_log2), shift2 = pair_of(-shift, -shift);
      uint32_t packed[kAttnGroupKeys / 2];
#pragma unroll
      for (int i = 0; i < kAttnGroupKeys; i += 2) {
        float x0, x1;
        halves_of(fma_pairs(pair_of(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), scale2, shift2), x0, x1);
        const float p0 = exp2_approx(x0), p1 = exp2_approx(x1);
        sum4[(i >> 1) & 3] = add_pairs(sum4[(i >> 1) & 3], pair_of(p0, p1));
        const __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
        packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&pair);
      }
      tmem_store_32(s_addr, packed);
      {
        float even, odd;
        halves_of(add_pairs(add_pairs(sum4[0], sum4[1]), add_pairs(sum4[2], sum4[3])), even, odd);
        l += even + odd;
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      // Rows of V past the last key the tile needs, and rows of pages that were not fetched because they lie
      // before every row's window: zero, so that P = 0 gives 0.  Each group clears the rows of its own keys.
      const int first_fetched = block_key0 + (skipped(j) << page_shift);
      if (block_key0 + kAttnKeys - 1 > last_pos || first_fetched > block_key0) {
        if (!wait_all(&sm.v_full[vs], (j / kAttnVStages) & 1)) { ok = false; break; }
        const int row = g * kAttnGroupKeys + (r & (kAttnGroupKeys - 1));
        if (r < kAttnGroupKeys && (block_key0 + row > last_pos || block_key0 + row < first_fetched)) {
#pragma unroll
          for (int h = 0; h < HALVES; ++h) {
            uint4* dst = reinterpret_cast<uint4*>(sm.v[vs] + h * kAttnHalf + row * 128);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.p_full[g][s]);
    }
    if (!ok) atomicExch(&sm.failed, 1u);
    // ---- epilogue: the two groups' parts of a row at a common maximum, added, divided by the common sum -------
    sm.row_max[g][r] = m_used;
    sm.row_sum[g][r] = l;
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.merge_ready);  // release: the stores above are ordered before it
    if (ok && wait_all(&sm.merge_ready, 0) && wait_all(&sm.pv_done[0], (blocks - 1) & 1) &&
        wait_all(&sm.pv_done[1], (blocks - 1) & 1)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float m0 = sm.row_max[0][r], m1 = sm.row_max[1][r];
      const float m_all = fmaxf(m0, m1);
      const float w0 = m0 == -INFINITY ? 0.f : exp2_approx(m0 - m_all);
      const float w1 = m1 == -INFINITY ? 0.f : exp2_approx(m1 - m_all);
      const float l_all = sm.row_sum[0][r] * w0 + sm.row_sum[1][r] * w1;
      const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
      const float f0 = w0 * inv, f1 = w1 * inv;
      // Group g writes columns g * D / 2 ... of the row, from both accumulators.  A whole tile of 128 rows goes
      // into the shared memory that held Q (all products with Q are done), in the layout of a tile copy, and
      // leaves as one: 128 rows of whole lines, where the threads' own stores are 16 bytes of 32 different
      // rows per instruction and take a microsecond and a half to drain.  A partial tile (the end of a
      // request) is stored by the threads, row by row.
      constexpr int SIDE_DIMS = D / 2;
      const bool whole = rows == kAttnRows;  // (the same for every thread of the CTA)
      __nv_bfloat16* dst = out + (size_t)(t0 + r) * out_row_stride + (size_t)head * D + g * SIDE_DIMS;
#pragma unroll
      for (int c0 = 0; c0 < SIDE_DIMS; c0 += 32) {
        uint32_t a[32], b[32];
        tmem_load_32(lane_base + O_COL + g * SIDE_DIMS + c0, a);
        tmem_load_32(lane_base + O_COL + D + g * SIDE_DIMS + c0, b);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (whole || r < rows) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            float y[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = __uint_as_float(a[i + e]) * f0 + __uint_as_float(b[i + e]) * f1;
            if (whole) {
              const int dim = g * SIDE_DIMS + c0 + i;  // 8 dims = one 16-byte piece of the row's 128-byte line
              const uint32_t at = smem_u32(sm.q) + (dim >> 6) * kAttnHalf + r * 128 + ((((dim & 63) >> 3) ^ (r & 7)) << 4);
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const __nv_bfloat162 pair = __floats2bfloat162_rn(y[2 * e], y[2 * e + 1]);
                w[e] = *reinterpret_cast<const uint32_t*>(&pair);
              }
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(at), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
            } else {
              store8(dst + c0 + i, y);
            }
          }
        }
      }
      if (whole) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the stores above, before the copy reads them
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.store_ready);
        if (warp == 2 && wait_all(&sm.store_ready, 0) && lane == 0) {
#pragma unroll
          for (int h = 0; h < HALVES; ++h)
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&map_out),
                         "r"(head * D + h * 64), "r"(t0), "r"(smem_u32(sm.q + h * kAttnHalf)) : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // shared memory is read before the CTA may end
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
static int launch_attention_tc(const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v,
                               const CUtensorMap& map_out, void* out,
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
      map_k, map_v, map_out, (__nv_bfloat16*)out, out_row_stride, q_tiles, positions, token_seq, seq_seat, block_table,
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
  CUtensorMap map_q, map_k, map_v, map_out;
  int status = make_map(&map_q, q, tokens, num_heads * head_dim, q_row_stride, kAttnRows);
  if (status != 0) return status;
  if ((status = make_map(&map_out, out, tokens, num_heads * head_dim, out_row_stride, kAttnRows)) != 0) return status;
  const long long cache_rows = (long long)num_pages * num_kv_heads * page_size;
  if (cache_rows > 0x7fffffffLL) return DISTIE_ERR_UNSUPPORTED;
  if ((status = make_map(&map_k, k_cache, (int)cache_rows, head_dim, head_dim, page_size)) != 0) return status;
  if ((status = make_map(&map_v, v_cache, (int)cache_rows, head_dim, head_dim, page_size)) != 0) return status;
  const float scale_log2 = scale * 1.4426950408889634f;
  if (head_dim == 64)
    return launch_attention_tc<64>(map_q, map_k, map_v, map_out, out, out_row_stride, q_tiles, num_tiles, positions, token_seq,
                                   seq_seat, block_table, table_width, num_heads, num_kv_heads, page_shift, num_pages,
                                   window, scale_log2, error, stream);
  return launch_attention_tc<128>(map_q, map_k, map_v, map_out, out, out_row_stride, q_tiles, num_tiles, positions, token_seq,
                                  seq_seat, block_table, table_width, num_heads, num_kv_heads, page_shift, num_pages,
                                  window, scale_log2, error, stream);
}
