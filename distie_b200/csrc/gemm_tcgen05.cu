// Products of many rows (prompt portions) on the 5th-generation tensor cores:
//   C[M, N] = A[M, K] (bfloat16 activations) x W[N, K]^T (bfloat16 weights), float32 accumulation.
//
// A CTA computes 128 x BN tiles of C, one after the other (persistent, one CTA per SM).  Operands are staged in shared memory by
// TMA (cp.async.bulk.tensor, 128-byte swizzle, K-major boxes of 64 elements) through a
// ring of stages; one elected thread issues tcgen05.mma (M = 128, N = BN, K = 16 per
// instruction) with the accumulator in tensor memory; four warps read the accumulator
// back with tcgen05.ld and run the epilogue in registers.
//
//   warp 0      producer: waits for a free stage, arms its mbarrier with the byte count, issues the TMA loads
//   warp 1      allocates tensor memory; one lane issues the MMAs of each stage as its barrier completes and
//               commits them to the stage's "empty" barrier, at the end to the "accumulator ready" barrier
//   warps 2..9  epilogue: warps w and w + 4 read TMEM lanes 32 * (w % 4) .. + 31 (their rows of the tile), half
//               of the columns each, 32 at a time, and write bfloat16, float32, or silu(gate) * up
//
// With the SwiGLU epilogue the weight is [2 * inter, K] (gate rows, then up rows) and a tile holds 128
// gate rows and the 128 matching up rows (two TMA loads per stage), so gate and up of one output
// element meet in the same thread.
//
// Rows and columns past the matrices are zero-filled by TMA and masked at the store; K needs to be a
// multiple of 8 only.  Every wait on an mbarrier is bounded: when a wait runs out, the kernel sets
// the error word to 6, stops issuing work, waits (bounded) for the copies it has in flight, releases
// its tensor memory and returns.
#include "tcgen05.cuh"

namespace distie {

constexpr int kGemmBM = 128;
constexpr int kGemmBK = 64;
constexpr int kGemmThreads = 192;      // the weight-streaming kernel: producer, MMA issuer, four epilogue warps
constexpr int kGemmWideThreads = 320;  // the tile kernels: producer, MMA issuer, eight epilogue warps

constexpr int GEMM_EPI_BF16 = 0;
constexpr int GEMM_EPI_F32 = 1;
constexpr int GEMM_EPI_SWIGLU = 2;
constexpr int GEMM_EPI_QKV = 3;  // bias, rotation and the write of q, k and v (store_qkv_rope); tiles of 256 columns

template <int BN, int STAGES>
struct GemmShared {
  alignas(1024) unsigned char a[STAGES][kGemmBM * kGemmBK * 2];
  alignas(1024) unsigned char b[STAGES][BN * kGemmBK * 2];
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t accum_full[2];
  uint64_t accum_empty[2];
  uint32_t tmem_base;
  uint32_t failed;
};

// 32 consecutive bfloat16 results of one row: 64 bytes per thread, whole sectors, in pieces of 16 bytes
// when the row allows it.
__device__ __forceinline__ void store_row_bf16(const float (&v)[32], __nv_bfloat16* __restrict__ dst, int cols_valid,
                                               bool aligned) {
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    if (j + 8 <= cols_valid && aligned) {
      float piece[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) piece[e] = v[j + e];
      store8(dst + j, piece);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (j + e < cols_valid) dst[j + e] = __float2bfloat16_rn(v[j + e]);
    }
  }
}

// 32 consecutive float32 results of one row with 256-bit stores: every store writes a whole 32-byte
// sector, so nothing is written in part (16-byte stores of a row fill each sector in two instructions
// that other rows' stores come between).  dst must be 32-byte aligned.
__device__ __forceinline__ void store_row_f32(const float (&v)[32], float* __restrict__ dst) {
#pragma unroll
  for (int j = 0; j < 32; j += 8)
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(dst + j), "f"(v[j]), "f"(v[j + 1]),
                 "f"(v[j + 2]), "f"(v[j + 3]), "f"(v[j + 4]), "f"(v[j + 5]), "f"(v[j + 6]), "f"(v[j + 7])
                 : "memory");
}

// The epilogue of one warp: its 32 rows (from row `row0` of the output) of a 128 x BN accumulator
// (tensor-memory address `lane_base`, first output column `n0`) to global memory as bfloat16, float32, or
// silu(gate) * up with the gate in columns [0, BN / 2) and the up values in [BN / 2, BN).
// Two warps share a quarter of the rows: `part` (0 or 1) selects this warp's half of the output columns.
//
// float32 results leave through `stage`, 4 KB of shared memory of the warp's own: a thread holds 32 columns of
// one row, and stored from there an instruction would touch 32 rows with 32 bytes each, which the memory
// system takes four times as long to absorb as whole lines.  So the 32 x 32 piece goes into shared memory
// (16-byte pieces, piece ^ (row & 7): no bank conflicts either way) and comes back with eight lanes to a
// row: an instruction then writes four whole 128-byte lines.
constexpr int kEpilogueStageBytes = 32 * 32 * 4;  // per epilogue warp

template <int BN, int EPI>
__device__ __forceinline__ void store_accumulator(uint32_t lane_base, int row0, int lane, int n0,
                                                  void* __restrict__ out, int ldo, int M, int N, int inter, int part,
                                                  unsigned char* stage) {
  const int rows_valid = M - row0;
  if (EPI == GEMM_EPI_SWIGLU) {
    constexpr int HALF = BN / 2;
    for (int c0 = part * (HALF / 2); c0 < (part + 1) * (HALF / 2); c0 += 32) {
      uint32_t gate[32], up[32];
      tmem_load_32(lane_base + c0, gate);
      tmem_load_32(lane_base + HALF + c0, up);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float g = __uint_as_float(gate[j]), u = __uint_as_float(up[j]);
        v[j] = __fdividef(g * u, 1.f + __expf(-g));
      }
      const int col = n0 + c0;
      if (lane < rows_valid && col < inter)
        store_row_bf16(v, (__nv_bfloat16*)out + (size_t)(row0 + lane) * ldo + col, inter - col, ((ldo | col) & 7) == 0);
    }
  } else {
    // The warp's whole part of the accumulator comes out of tensor memory behind one wait.
    constexpr int CHUNKS = BN / 64;
    uint32_t whole[CHUNKS][32];
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) tmem_load_32(lane_base + part * (BN / 2) + 32 * i, whole[i]);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
      const int c0 = part * (BN / 2) + 32 * i;
      uint32_t(&acc)[32] = whole[i];
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]);
      const int col = n0 + c0;
      if (rows_valid > 0 && col < N) {
        if (EPI == GEMM_EPI_F32) {
          // (uniform over the warp: whole rows of 32 columns, rows 16 bytes apart in alignment)
          if (col + 32 <= N && ((ldo | col) & 3) == 0 && ((uintptr_t)out & 15) == 0) {
            const uint32_t base = smem_u32(stage);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + lane * 128 + ((j ^ (lane & 7)) << 4)),
                           "r"(acc[4 * j]), "r"(acc[4 * j + 1]), "r"(acc[4 * j + 2]), "r"(acc[4 * j + 3]) : "memory");
            __syncwarp();
            const int piece = lane & 7;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int row = 4 * i + (lane >> 3);
              uint32_t w0, w1, w2, w3;
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3)
                           : "r"(base + row * 128 + ((piece ^ (row & 7)) << 4)) : "memory");
              if (row < rows_valid)
                asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"((float*)out + (size_t)(row0 + row) * ldo + col + 4 * piece),
                             "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
            }
            __syncwarp();  // before the next piece overwrites the stage
          } else if (lane < rows_valid) {
            float* dst = (float*)out + (size_t)(row0 + lane) * ldo + col;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col + j < N) dst[j] = v[j];
          }
        }
        else if (lane < rows_valid)
          store_row_bf16(v, (__nv_bfloat16*)out + (size_t)(row0 + lane) * ldo + col, N - col, ((ldo | col) & 7) == 0);
      }
    }
  }
}

// What the q/k/v epilogue needs beside the accumulator: see store_qkv_rope.
struct QkvEpilogue {
  const float* bias;     // [N] or null
  const float* trig;     // [M, head_dim]: cos of the row's angles in the first half, sin in the second (already scaled)
  const int* cache_row;  // [M]: row of the token's slot in the cache for kv head 0 (page * kv_heads * page_size + pos % page_size), -1: none
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  int num_heads, num_kv_heads, head_dim, page_size;
};

// The epilogue of the q/k/v projection of prompt portions: bias, rotation of q and k (pairs (j, j + head_dim / 2),
// cos and sin of the row's position from a table made once per step), q to its buffer and k and v straight into
// the token's slot of the paged cache, all as bfloat16.  The float32 product never goes to memory, and the
// rotation kernel that used to read it back is not launched.
//
// A warp has 32 rows of the tile; the two warps of a quarter of the rows split every head of the tile's 256
// columns by pairs: warp `part` takes pairs [part * HD / 4, (part + 1) * HD / 4) of each head, so it needs
// only that quarter of the cos and of the sin of its rows.  It copies them into shared memory of its own
// (qkv_stage_trig, asynchronously, while the MMAs of the tile still run), because 32 rows reading their
// own 512 bytes of the table from L2 piece by piece would wait for every piece.  `out` is the q buffer.
constexpr int kQkvStageFloats = 32 * (128 / 2 + 4);  // per epilogue warp: 32 rows of (cos quarter | sin quarter), padded

template <int HD>
__device__ __forceinline__ void qkv_stage_trig(float* stage, int row0, int lane, int part, int M, const float* trig) {
  constexpr int QW = HD / 4, STRIDE = HD / 2 + 4, PIECES = QW / 4;  // 16-byte pieces per row and segment
#pragma unroll
  for (int idx = lane; idx < 32 * 2 * PIECES; idx += 32) {
    const int row = idx / (2 * PIECES), rem = idx % (2 * PIECES), seg = rem / PIECES, piece = rem % PIECES;
    if (row0 + row < M) {
      const float* src = trig + (size_t)(row0 + row) * HD + seg * (HD / 2) + part * QW + piece * 4;
      asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(stage + row * STRIDE + seg * QW + piece * 4)),
                   "l"(src) : "memory");
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

template <int HD>
__device__ __forceinline__ void store_qkv_rope(uint32_t lane_base, int row0, int lane, int n0, int part,
                                               __nv_bfloat16* __restrict__ q_out, int ldq, int M, int N,
                                               const QkvEpilogue& e, const float* stage) {
  constexpr int QW = HD / 4, STRIDE = HD / 2 + 4;
  const int t = row0 + lane;
  const bool valid = t < M;
  const int slot = (valid && e.cache_row) ? e.cache_row[t] : -1;
  const float* cs_row = stage + lane * STRIDE;
  const float* sn_row = cs_row + QW;
  const int lo_off = part * QW, hi_off = HD / 2 + part * QW;
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncwarp();
#pragma unroll
  for (int h = 0; h < 256 / HD; ++h) {
    const int col0 = h * HD;               // first column of the head inside the tile
    if (n0 + col0 >= N) break;             // (uniform over the warp)
    const int head = (n0 + col0) / HD;     // q heads, then k heads, then v heads
    const bool is_q = head < e.num_heads, is_k = !is_q && head < e.num_heads + e.num_kv_heads;
    const int kv_head = head - e.num_heads - (is_k ? 0 : e.num_kv_heads);
    __nv_bfloat16* dst = nullptr;
    if (valid) {
      if (is_q)
        dst = q_out + (size_t)t * ldq + (size_t)head * HD;
      else if (slot >= 0)
        dst = (is_k ? e.k_cache : e.v_cache) + ((size_t)slot + (size_t)kv_head * e.page_size) * HD;
    }
    const float* bias = e.bias ? e.bias + (size_t)head * HD : nullptr;
    uint32_t lo[QW], hi[QW];
    if constexpr (QW == 32) {
      tmem_load_32(lane_base + col0 + lo_off, reinterpret_cast<uint32_t(&)[32]>(lo));
      tmem_load_32(lane_base + col0 + hi_off, reinterpret_cast<uint32_t(&)[32]>(hi));
    } else {
      tmem_load_16(lane_base + col0 + lo_off, reinterpret_cast<uint32_t(&)[16]>(lo));
      tmem_load_16(lane_base + col0 + hi_off, reinterpret_cast<uint32_t(&)[16]>(hi));
    }
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    if (dst != nullptr) {
#pragma unroll
      for (int j = 0; j < QW; j += 8) {
        float a[8], b[8], y_lo[8], y_hi[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          a[i] = __uint_as_float(lo[j + i]);
          b[i] = __uint_as_float(hi[j + i]);
        }
        if (bias) {
          float ba[8], bb[8];
          load8(bias + lo_off + j, ba);
          load8(bias + hi_off + j, bb);
#pragma unroll
          for (int i = 0; i < 8; ++i) { a[i] += ba[i]; b[i] += bb[i]; }
        }
        if (is_q || is_k) {
          float cs[8], sn[8];
          load8(cs_row + j, cs);
          load8(sn_row + j, sn);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            y_lo[i] = a[i] * cs[i] - b[i] * sn[i];
            y_hi[i] = b[i] * cs[i] + a[i] * sn[i];
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) { y_lo[i] = a[i]; y_hi[i] = b[i]; }
        }
        store8(dst + lo_off + j, y_lo);
        store8(dst + hi_off + j, y_hi);
      }
    }
    __syncwarp();  // the loads from tensor memory are warp-wide: rows without a destination rejoin here
  }
}

// Persistent: a CTA walks the tiles blockIdx.x, blockIdx.x + gridDim.x, ...  The accumulator is
// double-buffered in tensor memory (2 x 256 columns), so the epilogue of one tile runs while the
// MMAs of the next fill the other buffer; the ring of shared-memory stages runs across tiles.
template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(kGemmWideThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    void* __restrict__ out, int ldo, int M, int N, int K, int inter, int m_tiles, int num_tiles,
                    const QkvEpilogue qkv, int* __restrict__ error) {
  extern __shared__ unsigned char raw[];
  auto& sm = *reinterpret_cast<GemmShared<BN, STAGES>*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  constexpr uint32_t TMEM_COLS = 512;   // two accumulators, the second at column 256
  constexpr uint32_t ACC_STRIDE = 256;
  constexpr uint32_t STAGE_BYTES = (kGemmBM + BN) * kGemmBK * 2;
  constexpr int PER_TILE = EPI == GEMM_EPI_SWIGLU ? BN / 2 : BN;  // output columns per tile
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_blocks = (K + kGemmBK - 1) / kGemmBK;

  if (threadIdx.x == 64) {
    prefetch_tensor_map(&map_a);
    prefetch_tensor_map(&map_b);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.accum_full[b], 1);
      mbar_init(&sm.accum_empty[b], 8);  // one arrival per epilogue warp
    }
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
  // Launched as a dependent kernel: everything up to here overlaps the end of the kernel before this
  // one.  Its results (the activations) are read, and anything is written, only after the wait; the
  // weights are written by no kernel, so the producer has the first ring of weight tiles on its way
  // before it waits.
  grid_dependency_release();

  if (warp == 0) {
    // ---- producer ----------------------------------------------------------------------------------------
    if (lane == 0) {
      uint32_t it = 0;  // stages filled so far, over all tiles
      bool ok = true;
      auto load_w = [&](int s, int kb, int n0) {
        if (EPI == GEMM_EPI_SWIGLU) {
          tma_load_2d(sm.b[s], &map_b, &sm.full[s], kb * kGemmBK, n0);
          tma_load_2d(sm.b[s] + (BN / 2) * kGemmBK * 2, &map_b, &sm.full[s], kb * kGemmBK, inter + n0);
        } else {
          tma_load_2d(sm.b[s], &map_b, &sm.full[s], kb * kGemmBK, n0);
        }
      };
      const int early = blockIdx.x < num_tiles ? min(k_blocks, STAGES) : 0;  // of this CTA's first tile
      for (int kb = 0; kb < early; ++kb) {
        mbar_expect_tx(&sm.full[kb], STAGE_BYTES);
        load_w(kb, kb, (blockIdx.x / m_tiles) * PER_TILE);
      }
      grid_dependency_wait();
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * kGemmBM;
        const int n0 = (tile / m_tiles) * PER_TILE;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (it >= (uint32_t)early) {
            if (!mbar_wait(&sm.empty[s], ((it / STAGES) & 1) ^ 1)) { atomicExch(&sm.failed, 1u); ok = false; break; }
            mbar_expect_tx(&sm.full[s], STAGE_BYTES);
            load_w(s, kb, n0);
          }
          tma_load_2d(sm.a[s], &map_a, &sm.full[s], kb * kGemmBK, m0);
        }
      }
      if (!ok) {
        // Copies already issued still land in shared memory: give them a bounded time before leaving.
        for (uint32_t back = (it > (uint32_t)STAGES ? it - STAGES : 0); back < it; ++back)
          mbar_wait(&sm.full[back % STAGES], (back / STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----------------------------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(BN);
      uint32_t it = 0, round = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++round) {
        const uint32_t buffer = round & 1;
        // The epilogue must have drained this accumulator (two tiles ago).
        if (!mbar_wait(&sm.accum_empty[buffer], ((round >> 1) & 1) ^ 1)) { atomicExch(&sm.failed, 1u); break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem + buffer * ACC_STRIDE;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&sm.full[s], (it / STAGES) & 1)) { atomicExch(&sm.failed, 1u); ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t a_desc = smem_desc(sm.a[s]), b_desc = smem_desc(sm.b[s]);
#pragma unroll
          for (int k = 0; k < kGemmBK / 16; ++k)  // 32 bytes further along K inside the swizzled row: +2 in the address field
            umma_bf16(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&sm.empty[s]);  // arrives when these MMAs have read the stage
        }
        umma_commit(&sm.accum_full[buffer]);  // arrives when the accumulator is complete
      }
    }
  } else {
    // ---- epilogue: warps w and w + 4 share rows 32 * (w % 4) .. + 31 and take half of the columns each ------
    grid_dependency_wait();  // nothing is written before the earlier kernels are done
    const int quadrant = warp & 3, part = (warp - 2) >> 2;
    unsigned char* behind = reinterpret_cast<unsigned char*>(&sm) + ((sizeof(sm) + 15) & ~size_t(15));  // behind the stages:
    float* trig_stage = reinterpret_cast<float*>(behind) + (warp - 2) * kQkvStageFloats;  // asked for by the q/k/v epilogue,
    unsigned char* epilogue_stage = behind + (warp - 2) * kEpilogueStageBytes;            // by the float32 epilogue
    uint32_t round = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++round) {
      const uint32_t buffer = round & 1;
      const int m0 = (tile % m_tiles) * kGemmBM;
      const int n0 = (tile / m_tiles) * PER_TILE;
      if (EPI == GEMM_EPI_QKV) {  // this warp's cos and sin, on their way while the tile's MMAs run
        if (qkv.head_dim == 128) qkv_stage_trig<128>(trig_stage, m0 + quadrant * 32, lane, part, M, qkv.trig);
        else qkv_stage_trig<64>(trig_stage, m0 + quadrant * 32, lane, part, M, qkv.trig);
      }
      if (!mbar_wait(&sm.accum_full[buffer], (round >> 1) & 1) || sm.failed) { atomicExch(&sm.failed, 1u); break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_base = tmem + buffer * ACC_STRIDE + ((uint32_t)(quadrant * 32) << 16);
      if (EPI == GEMM_EPI_QKV) {
        if (qkv.head_dim == 128) store_qkv_rope<128>(lane_base, m0 + quadrant * 32, lane, n0, part, (__nv_bfloat16*)out, ldo, M, N, qkv, trig_stage);
        else store_qkv_rope<64>(lane_base, m0 + quadrant * 32, lane, n0, part, (__nv_bfloat16*)out, ldo, M, N, qkv, trig_stage);
      } else {
        store_accumulator<BN, EPI>(lane_base, m0 + quadrant * 32, lane, n0, out, ldo, M, N, inter, part, epilogue_stage);
      }
      // This warp has read its part of the accumulator: hand the buffer back to the MMA issuer.
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.accum_empty[buffer]);
    }
    if (EPI == GEMM_EPI_QKV) asm volatile("cp.async.wait_all;" ::: "memory");  // (a loop left early: nothing stays in flight)
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
  }
  if (threadIdx.x == 0 && sm.failed && error) atomicExch(error, 6);
}

// ---------------------------------------------------------------------------------------------------------------
// The same product on pairs of CTAs (clusters of two, tcgen05 with cta_group::2): a pair computes 256 x BN
// tiles.  Each CTA stages its own 128 rows of A and half of the tile's rows of W, so a stage costs a CTA
// 16 KB + BN / 2 * 128 bytes instead of 16 KB + BN * 128 for the same number of MMA cycles: the product
// is bound by what an SM can pull out of L2, and this is where the pair wins.  The MMA is issued by the
// first CTA of the pair for both; it reads both CTAs' shared memory and writes 128 rows of the
// accumulator into each CTA's tensor memory, which each CTA's epilogue warps store.
//
//   full[s]          in the first CTA: armed there with the bytes of both CTAs; both CTAs' copies count on it
//   empty[s]         in each CTA: tcgen05.commit of the stage's MMAs arrives on both
//   accum_full[b]    in each CTA: tcgen05.commit after a tile's last MMA arrives on both
//   accum_empty[b]   in the first CTA: the sixteen epilogue warps of the pair arrive on it
// ---------------------------------------------------------------------------------------------------------------
template <int BN, int STAGES, int KB>
struct PairShared {
  alignas(1024) unsigned char a[STAGES][KB][kGemmBM * kGemmBK * 2];  // KB boxes of 64 along K per stage
  alignas(1024) unsigned char b[STAGES][KB][(BN / 2) * kGemmBK * 2];
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t accum_full[2];
  uint64_t accum_empty[2];
  uint32_t tmem_base;
  uint32_t failed;
};

template <int BN, int STAGES, int KB, int EPI>
__global__ void __launch_bounds__(kGemmWideThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         void* __restrict__ out, int ldo, int M, int N, int K, int inter, int m_tiles, int num_tiles,
                         const QkvEpilogue qkv, int* __restrict__ error) {
  extern __shared__ unsigned char raw[];
  auto& sm = *reinterpret_cast<PairShared<BN, STAGES, KB>*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  constexpr uint32_t TMEM_COLS = 512;   // two accumulators, the second at column 256
  constexpr uint32_t ACC_STRIDE = 256;
  constexpr uint32_t STAGE_BYTES_PAIR = 2 * KB * (kGemmBM + BN / 2) * kGemmBK * 2;
  constexpr int STAGE_K = KB * kGemmBK;
  constexpr int PER_TILE = EPI == GEMM_EPI_SWIGLU ? BN / 2 : BN;  // output columns per tile
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_blocks = (K + STAGE_K - 1) / STAGE_K;
  const uint32_t rank = cluster_cta_rank();       // 0: issues the MMAs
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

  if (threadIdx.x == 64) {
    prefetch_tensor_map(&map_a);
    prefetch_tensor_map(&map_b);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.accum_full[b], 1);
      mbar_init(&sm.accum_empty[b], 16);  // one arrival per epilogue warp of the pair
    }
    sm.failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  cluster_barrier();  // both CTAs' barriers are initialised and tensor memory is allocated
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = sm.tmem_base;
  grid_dependency_release();  // (the wait: by the producers behind their first weight tiles, by the epilogue warps)

  if (warp == 0) {
    // ---- producer (both CTAs) -------------------------------------------------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      // Rows of W this CTA stages: with SwiGLU the first CTA takes the gate rows, the second the up rows.
      auto rows_of_w = [&](int tile) {
        const int n_tile = (tile / m_tiles) * PER_TILE;
        return EPI == GEMM_EPI_SWIGLU ? (rank == 0 ? n_tile : inter + n_tile) : n_tile + (int)rank * (BN / 2);
      };
      // The weights are written by no kernel: the first ring of them is on its way before the wait for
      // the kernel that makes the activations.  (A copy of the second CTA may land on the first CTA's
      // barrier before that one has announced the bytes; the phase cannot end before it has.)
      const int early = pair < num_tiles ? min(k_blocks, STAGES) : 0;
      for (int kb = 0; kb < early; ++kb) {
        if (rank == 0) mbar_expect_tx(&sm.full[kb], STAGE_BYTES_PAIR);
        const uint32_t full_addr = cluster_address(&sm.full[kb], 0);
#pragma unroll
        for (int box = 0; box < KB; ++box)
          tma_load_2d_pair(sm.b[kb][box], &map_b, full_addr, kb * STAGE_K + box * kGemmBK, rows_of_w(pair));
      }
      grid_dependency_wait();
      for (int tile = pair; tile < num_tiles && ok; tile += pairs) {
        const int m0 = (tile % m_tiles) * 2 * kGemmBM + (int)rank * kGemmBM;
        const int w0 = rows_of_w(tile);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const bool ahead = it < (uint32_t)early;  // this stage's weights are under way already
          if (!ahead) {
            if (!mbar_wait_unless(&sm.empty[s], ((it / STAGES) & 1) ^ 1, &sm.failed)) { ok = false; break; }
            if (rank == 0) mbar_expect_tx(&sm.full[s], STAGE_BYTES_PAIR);
          }
          const uint32_t full_addr = cluster_address(&sm.full[s], 0);
#pragma unroll
          for (int box = 0; box < KB; ++box) {  // a box past K is filled with zeros and still counted
            tma_load_2d_pair(sm.a[s][box], &map_a, full_addr, kb * STAGE_K + box * kGemmBK, m0);
            if (!ahead) tma_load_2d_pair(sm.b[s][box], &map_b, full_addr, kb * STAGE_K + box * kGemmBK, w0);
          }
        }
      }
      if (!ok) {
        atomicExch(&sm.failed, 1u);
        // Copies already issued still land in shared memory: the first CTA, whose barriers count them,
        // gives them a bounded time before the pair leaves.
        if (rank == 0)
          for (uint32_t back = (it > (uint32_t)STAGES ? it - STAGES : 0); back < it; ++back)
            mbar_wait(&sm.full[back % STAGES], (back / STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer (first CTA only) --------------------------------------------------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = instr_desc_pair(BN);
      uint32_t it = 0, round = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++round) {
        const uint32_t buffer = round & 1;
        if (!mbar_wait_unless(&sm.accum_empty[buffer], ((round >> 1) & 1) ^ 1, &sm.failed)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem + buffer * ACC_STRIDE;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait_unless(&sm.full[s], (it / STAGES) & 1, &sm.failed)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int box = 0; box < KB; ++box) {
            const uint64_t a_desc = smem_desc(sm.a[s][box]), b_desc = smem_desc(sm.b[s][box]);
#pragma unroll
            for (int k = 0; k < kGemmBK / 16; ++k)
              umma_bf16_pair(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || box > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(&sm.empty[s], 3);
        }
        if (ok) umma_commit_pair(&sm.accum_full[buffer], 3);
      }
      if (!ok) atomicExch(&sm.failed, 1u);
    }
  } else {
    // ---- epilogue (both CTAs, each its own 128 rows; two warps per quarter of the rows, half the columns each) --
    grid_dependency_wait();  // nothing is written before the earlier kernels are done
    const int quadrant = warp & 3, part = (warp - 2) >> 2;
    unsigned char* behind = reinterpret_cast<unsigned char*>(&sm) + ((sizeof(sm) + 15) & ~size_t(15));  // behind the stages:
    float* trig_stage = reinterpret_cast<float*>(behind) + (warp - 2) * kQkvStageFloats;  // asked for by the q/k/v epilogue,
    unsigned char* epilogue_stage = behind + (warp - 2) * kEpilogueStageBytes;            // by the float32 epilogue
    uint32_t round = 0;
    for (int tile = pair; tile < num_tiles; tile += pairs, ++round) {
      const uint32_t buffer = round & 1;
      const int m0 = (tile % m_tiles) * 2 * kGemmBM + (int)rank * kGemmBM;
      const int n0 = (tile / m_tiles) * PER_TILE;
      if (EPI == GEMM_EPI_QKV) {  // this warp's cos and sin, on their way while the tile's MMAs run
        if (qkv.head_dim == 128) qkv_stage_trig<128>(trig_stage, m0 + quadrant * 32, lane, part, M, qkv.trig);
        else qkv_stage_trig<64>(trig_stage, m0 + quadrant * 32, lane, part, M, qkv.trig);
      }
      const bool ready = __all_sync(0xffffffffu, mbar_wait_unless(&sm.accum_full[buffer], (round >> 1) & 1, &sm.failed));
      if (!ready) { atomicExch(&sm.failed, 1u); break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_base = tmem + buffer * ACC_STRIDE + ((uint32_t)(quadrant * 32) << 16);
      if (EPI == GEMM_EPI_QKV) {
        if (qkv.head_dim == 128) store_qkv_rope<128>(lane_base, m0 + quadrant * 32, lane, n0, part, (__nv_bfloat16*)out, ldo, M, N, qkv, trig_stage);
        else store_qkv_rope<64>(lane_base, m0 + quadrant * 32, lane, n0, part, (__nv_bfloat16*)out, ldo, M, N, qkv, trig_stage);
      } else {
        store_accumulator<BN, EPI>(lane_base, m0 + quadrant * 32, lane, n0, out, ldo, M, N, inter, part, epilogue_stage);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster_relaxed(cluster_address(&sm.accum_empty[buffer], 0));
    }
    if (EPI == GEMM_EPI_QKV) asm volatile("cp.async.wait_all;" ::: "memory");  // (a loop left early: nothing stays in flight)
  }

  // Neither CTA may leave while the other can still reach its shared memory, barriers or tensor memory.
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (sm.failed && threadIdx.x == 0) {
    // Tell the other CTA, so that its waits end at once, and give copies in flight time to land.
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_address(&sm.failed, rank ^ 1)), "r"(1u) : "memory");
    __nanosleep(20000);
  }
  cluster_barrier_exit();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
  }
  if (threadIdx.x == 0 && sm.failed && error) atomicExch(error, 6);
}

// ---------------------------------------------------------------------------------------------------------------
// The same machinery turned around for few rows of x (decoding): the weights are the 128-row operand and
// stream through a deep ring of TMA stages (16 KB each), the rows of x are the narrow operand
// (N = 16, 32 or 64), and the accumulator is D[weight row, row of x].  A product like this is bound by
// reading W once; what it needs is many bytes in flight per SM, which the ring gives without spending
// registers.  K may be split over gridDim.y CTAs: each then writes its float32 slice [M, N] and the
// consumer adds the slices up.
//
//   EPI_SLICE   out is [splits, M, N] float32 (row stride N), no bias
//   EPI_STORE   out is [M, N] bfloat16 or float32 with bias (one split)
//   EPI_SWIGLU  W is [2 * inter, K]; a tile holds 64 gate rows and the 64 matching up rows; out[M, inter]
//
// Launched as a dependent kernel: the producer warp issues the first weight stages before it waits for
// the kernel that writes x.
// ---------------------------------------------------------------------------------------------------------------
constexpr int SKINNY_EPI_SLICE = 0;
constexpr int SKINNY_EPI_STORE = 1;
constexpr int SKINNY_EPI_SWIGLU = 2;

template <int BN, int STAGES>
struct SkinnyShared {
  alignas(1024) unsigned char w[STAGES][kGemmBM * kGemmBK * 2];
  alignas(1024) unsigned char x[STAGES][BN * kGemmBK * 2];
  float exchange[kGemmBM][17];  // SwiGLU: gate and up rows meet here, 16 rows of x at a time
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t accum;
  uint32_t tmem_base;
  uint32_t failed;
};

template <int BN, int STAGES, int EPI, typename OutT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                           const float* __restrict__ bias, OutT* __restrict__ out, int ldo, int M, int N, int K,
                           int inter, int* __restrict__ error) {
  extern __shared__ unsigned char raw[];
  auto& sm = *reinterpret_cast<SkinnyShared<BN, STAGES>*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  constexpr uint32_t W_BYTES = kGemmBM * kGemmBK * 2, X_BYTES = BN * kGemmBK * 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
  const int k_blocks_all = (K + kGemmBK - 1) / kGemmBK;
  const int per_split = (k_blocks_all + splits - 1) / splits;
  const int kb_begin = split * per_split;
  const int kb_end = min(k_blocks_all, kb_begin + per_split);
  const int k_blocks = max(0, kb_end - kb_begin);
  // Weight rows of the tile: [r0, r0 + 128), or with SwiGLU 64 gate rows and the 64 matching up rows.
  const int r0 = EPI == SKINNY_EPI_SWIGLU ? tile * 64 : tile * kGemmBM;

  grid_dependency_release();
  if (threadIdx.x == 32) {
    prefetch_tensor_map(&map_w);
    prefetch_tensor_map(&map_x);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    mbar_init(&sm.accum, 1);
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

  if (warp == 0) {
    // ---- producer ----------------------------------------------------------------------------------------
    // The copies of a stage are issued by as many lanes in one instruction (lane 0: the weights, or with
    // SwiGLU the gate rows; lane 1: the up rows; the next lane: x): one thread issuing them one after
    // the other takes several hundred clocks a stage, which is as long as the stage's bytes take at
    // this SM's share of the memory bandwidth.
    constexpr int X_LANE = EPI == SKINNY_EPI_SWIGLU ? 2 : 1;
    auto load_w = [&](int kb, int s) {
      const int k = (kb_begin + kb) * kGemmBK;
      if (EPI == SKINNY_EPI_SWIGLU) {
        if (lane == 0) tma_load_2d(sm.w[s], &map_w, &sm.full[s], k, r0);
        if (lane == 1) tma_load_2d(sm.w[s] + 64 * kGemmBK * 2, &map_w, &sm.full[s], k, inter + r0);
      } else {
        if (lane == 0) tma_load_2d(sm.w[s], &map_w, &sm.full[s], k, r0);
      }
    };
    // The weights are written by no kernel: the first ring of stages starts before the wait.
    const int early = min(k_blocks, STAGES);
    for (int kb = 0; kb < early; ++kb) {
      if (lane == 0) mbar_expect_tx(&sm.full[kb], W_BYTES + X_BYTES);
      __syncwarp();
      load_w(kb, kb);
    }
    grid_dependency_wait();
    if (lane == X_LANE)
      for (int kb = 0; kb < early; ++kb) tma_load_2d(sm.x[kb], &map_x, &sm.full[kb], (kb_begin + kb) * kGemmBK, 0);
    int issued = early;
    for (int kb = early; kb < k_blocks; ++kb) {
      const int s = kb % STAGES;
      int ready = 1;
      if (lane == 0) {
        ready = mbar_wait(&sm.empty[s], ((kb / STAGES) & 1) ^ 1) ? 1 : 0;
        if (ready) mbar_expect_tx(&sm.full[s], W_BYTES + X_BYTES);
      }
      if (!__shfl_sync(0xffffffffu, ready, 0)) { atomicExch(&sm.failed, 1u); break; }
      load_w(kb, s);
      if (lane == X_LANE) tma_load_2d(sm.x[s], &map_x, &sm.full[s], (kb_begin + kb) * kGemmBK, 0);
      issued = kb + 1;
    }
    __syncwarp();
    if (sm.failed && lane == 0) {
      for (int kb = max(0, issued - STAGES); kb < issued; ++kb) mbar_wait(&sm.full[kb % STAGES], (kb / STAGES) & 1);
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----------------------------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(BN);
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % STAGES;
        if (!mbar_wait(&sm.full[s], (kb / STAGES) & 1)) { atomicExch(&sm.failed, 1u); break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t a_desc = smem_desc(sm.w[s]), b_desc = smem_desc(sm.x[s]);
#pragma unroll
        for (int k = 0; k < kGemmBK / 16; ++k)
          umma_bf16(tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        umma_commit(&sm.empty[s]);
      }
      umma_commit(&sm.accum);
    }
  } else {
    // ---- epilogue: lane = weight row of the tile, columns = rows of x --------------------------------------
    grid_dependency_wait();  // nothing is written before the earlier kernels are done
    const bool ready = mbar_wait(&sm.accum, 0);
    if (!ready) atomicExch(&sm.failed, 1u);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int quadrant = warp & 3;
    const int local_row = quadrant * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(quadrant * 32) << 16);
    const bool valid = ready && !sm.failed && k_blocks > 0;
    const int row = r0 + local_row;
    const float b = (EPI == SKINNY_EPI_STORE && bias && row < N) ? bias[row] : 0.f;
    // The whole accumulator of the row comes out of tensor memory at once (one wait, not one per sixteen
    // columns: with 64 rows of x the waits were a microsecond at the end of every CTA); it is then handled
    // sixteen rows of x at a time.
    uint32_t whole[BN];
    if (valid) {
#pragma unroll
      for (int c0 = 0; c0 < BN; c0 += 16) tmem_load_16(lane_base + c0, *reinterpret_cast<uint32_t(*)[16]>(&whole[c0]));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    }
#pragma unroll
    for (int c0 = 0; c0 < BN; c0 += 16) {
      if (c0 >= M) break;
      float acc[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = valid ? __uint_as_float(whole[c0 + j]) : 0.f;
      if (EPI == SKINNY_EPI_SWIGLU) {
#pragma unroll
        for (int j = 0; j < 16; ++j) sm.exchange[local_row][j] = acc[j];
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps only
        // Output column r0 + (local_row % 64); the two halves of the threads share the sixteen rows of x.
        const int pair = local_row & 63, j0 = (local_row >> 6) * 8;
        const int col = r0 + pair;
        if (col < inter) {
#pragma unroll
          for (int j = j0; j < j0 + 8; ++j) {
            if (c0 + j < M) {
              const float g = sm.exchange[pair][j], u = sm.exchange[64 + pair][j];
              out[(size_t)(c0 + j) * ldo + col] = from_float<OutT>(__fdividef(g * u, 1.f + __expf(-g)));
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // before the next sixteen overwrite the exchange
      } else if (row < N) {
        OutT* dst = out + (EPI == SKINNY_EPI_SLICE ? (size_t)split * M * ldo : 0) + row;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (c0 + j < M) dst[(size_t)(c0 + j) * ldo] = from_float<OutT>(acc[j] + b);
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
  }
  if (threadIdx.x == 0 && sm.failed && error) atomicExch(error, 6);
}

// ---- host side ---------------------------------------------------------------------------------------------
template <int BN, int STAGES, int EPI>
static int launch_gemm(const CUtensorMap& map_a, const CUtensorMap& map_b, void* out, int ldo, int M, int N, int K,
                       int inter, int sm_count, int* error, cudaStream_t stream, const QkvEpilogue& qkv = QkvEpilogue()) {
  const size_t shared = sizeof(GemmShared<BN, STAGES>) + 1024 + (EPI == GEMM_EPI_QKV ? 16 + 8 * kQkvStageFloats * sizeof(float) : 0) +
                        (EPI == GEMM_EPI_F32 ? 16 + 8 * kEpilogueStageBytes : 0);
  static bool configured = false;
  if (!configured) {
    const cudaError_t err =
        cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  const int m_tiles = (M + kGemmBM - 1) / kGemmBM;
  const int columns = EPI == GEMM_EPI_SWIGLU ? inter : N;
  const int per_tile = EPI == GEMM_EPI_SWIGLU ? BN / 2 : BN;
  const int num_tiles = m_tiles * ((columns + per_tile - 1) / per_tile);
  const int grid = num_tiles < sm_count ? num_tiles : sm_count;
  const cudaError_t err =
      launch_dependent_family(64, gemm_tcgen05_kernel<BN, STAGES, EPI>, dim3(grid), dim3(kGemmWideThreads), shared, stream,
                              map_a, map_b, out, ldo, M, N, K, inter, m_tiles, num_tiles, qkv, error);
  return err == cudaSuccess ? 0 : (int)err;
}

template <int BN, int STAGES, int KB, int EPI>
static int launch_gemm_pair(const CUtensorMap& map_a, const CUtensorMap& map_b, void* out, int ldo, int M, int N, int K,
                            int inter, int sm_count, int* error, cudaStream_t stream, const QkvEpilogue& qkv = QkvEpilogue()) {
  const size_t shared = sizeof(PairShared<BN, STAGES, KB>) + 1024 + (EPI == GEMM_EPI_QKV ? 16 + 8 * kQkvStageFloats * sizeof(float) : 0) +
                        (EPI == GEMM_EPI_F32 ? 16 + 8 * kEpilogueStageBytes : 0);
  static bool configured = false;
  static int resident_pairs = 0;  // pairs that can run at the same time (an SM left over in a GPC hosts none)
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<BN, STAGES, KB, EPI>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
    cudaLaunchConfig_t probe = {};
    probe.gridDim = dim3(2 * (sm_count / 2));
    probe.blockDim = dim3(kGemmWideThreads);
    probe.dynamicSmemBytes = shared;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = 2;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    probe.attrs = attribute;
    probe.numAttrs = 1;
    err = cudaOccupancyMaxActiveClusters(&resident_pairs, gemm_tcgen05_pair_kernel<BN, STAGES, KB, EPI>, &probe);
    if (err != cudaSuccess) return (int)err;
    if (resident_pairs < 1) return DISTIE_ERR_UNSUPPORTED;
    configured = true;
  }
  const int m_tiles = (M + 2 * kGemmBM - 1) / (2 * kGemmBM);
  const int columns = EPI == GEMM_EPI_SWIGLU ? inter : N;
  const int per_tile = EPI == GEMM_EPI_SWIGLU ? BN / 2 : BN;
  const int num_tiles = m_tiles * ((columns + per_tile - 1) / per_tile);
  const int slots = resident_pairs < sm_count / 2 ? resident_pairs : sm_count / 2;
  const int pairs = num_tiles < slots ? num_tiles : slots;
  const cudaError_t err = launch_dependent_cluster(64, dim3(2, 1, 1), gemm_tcgen05_pair_kernel<BN, STAGES, KB, EPI>,
                                                   dim3(2 * pairs), dim3(kGemmWideThreads), shared, stream, map_a, map_b, out,
                                                   ldo, M, N, K, inter, m_tiles, num_tiles, qkv, error);
  return err == cudaSuccess ? 0 : (int)err;
}

// Tile width (128, 192 or 256 columns).  Pairs of CTAs take 256 as soon as the product is more than one wave of
// tiles: measured at the projection and feed-forward shapes of 1.5B, 7B and 14B models with 512 to 2,048 rows,
// 256-wide tiles were the fastest or within 4 % of it there, while a count of waves alone picked 128 for
// [2048 x 7168 x 5120] and lost a third of the time to operand traffic (a narrow tile re-reads A once per 128
// columns).  A product that is a single wave either way takes the narrowest tiles that still are one wave:
// every pair then has less to do (2,048 x 1,536 x 1,536: 12.3 against 12.9 us with 192; 512 rows of it: 11.7
// against 13.6 us with 128).  A single CTA per tile (fewer than 256 rows) takes the width whose waves of
// `slots` tiles cost least.
static int pick_tile_width(int M, int N, int tile_rows, int slots) {
  if (tile_rows > kGemmBM) {
    const int m_tiles = (M + tile_rows - 1) / tile_rows;
    for (int width : {128, 192})  // (a few pairs fewer than there are: an SM left over in a GPC hosts no pair)
      if ((long long)m_tiles * ((N + width - 1) / width) <= slots - 4) return width;
    return 256;
  }
  const int m_tiles = (M + tile_rows - 1) / tile_rows;
  int best = 256;
  long long best_cost = -1;
  for (int width : {256, 192, 128}) {
    const long long tiles = (long long)m_tiles * ((N + width - 1) / width);
    const long long cost = ((tiles + slots - 1) / slots) * width;
    if (best_cost < 0 || cost < best_cost) {
      best = width;
      best_cost = cost;
    }
  }
  return best;
}

}  // namespace distie

using namespace distie;

// out = x[M, K] w[N, K]^T.  epi 0: bfloat16 [M, N]; 1: float32 [M, N]; 2: w is [2 * inter, K] and
// out[M, inter] = silu(x Wg^T) * (x Wu^T) in bfloat16 (N = 2 * inter).  x and w are bfloat16 with row
// strides ldx and K; K must be a multiple of 8 and the pointers 16-byte aligned.
// `tile_width` 128, 192 or 256 picks the width of the output tiles; 0 leaves the choice to the kernel.
extern "C" int distie_gemm_tcgen05(const void* x, int ldx, const void* w, void* out, int ldo, int M, int N, int K,
                                   int epi, int tile_width, int sm_count, int* error, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (N < 1 || K < 8 || (K & 7) || (ldx & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
    return DISTIE_ERR_UNSUPPORTED;
  if (epi == GEMM_EPI_SWIGLU && (N & 1)) return DISTIE_ERR_ARG;
  if (sm_count < 1) sm_count = 148;
  CUtensorMap map_a, map_b;
  int status = make_map(&map_a, x, M, K, ldx, kGemmBM);
  if (status != 0) return status;
  if (M >= 2 * kGemmBM && sm_count >= 2) {
    // Pairs of CTAs on 256-row tiles; each CTA stages half of the tile's rows of W.
    if (epi == GEMM_EPI_SWIGLU) {
      if ((status = make_map(&map_b, w, N, K, K, 128)) != 0) return status;
      return launch_gemm_pair<256, 6, 1, GEMM_EPI_SWIGLU>(map_a, map_b, out, ldo, M, N, K, N / 2, sm_count, error, stream);
    }
    if (epi != GEMM_EPI_F32 && epi != GEMM_EPI_BF16) return DISTIE_ERR_ARG;
    const int width = tile_width ? tile_width : pick_tile_width(M, N, 2 * kGemmBM, sm_count / 2);
    if (width != 128 && width != 192 && width != 256) return DISTIE_ERR_ARG;
    if ((status = make_map(&map_b, w, N, K, K, width / 2)) != 0) return status;
    // (stages: what fits beside the float32 epilogue's 32 KB of staging, where that is asked for)
#define DISTIE_GEMM_PAIR(BNV, STAGESV, STAGES32)                                                                          \
  return epi == GEMM_EPI_F32                                                                                             \
             ? launch_gemm_pair<BNV, STAGES32, 1, GEMM_EPI_F32>(map_a, map_b, out, ldo, M, N, K, 0, sm_count, error, stream) \
             : launch_gemm_pair<BNV, STAGESV, 1, GEMM_EPI_BF16>(map_a, map_b, out, ldo, M, N, K, 0, sm_count, error, stream)
    if (width == 256) { DISTIE_GEMM_PAIR(256, 6, 6); }
    if (width == 192) { DISTIE_GEMM_PAIR(192, 7, 6); }
    DISTIE_GEMM_PAIR(128, 8, 8);
#undef DISTIE_GEMM_PAIR
  }
  if (epi == GEMM_EPI_SWIGLU) {
    status = make_map(&map_b, w, N, K, K, 128);
    if (status != 0) return status;
    return launch_gemm<256, 4, GEMM_EPI_SWIGLU>(map_a, map_b, out, ldo, M, N, K, N / 2, sm_count, error, stream);
  }
  if (epi != GEMM_EPI_F32 && epi != GEMM_EPI_BF16) return DISTIE_ERR_ARG;
  const int width = tile_width ? tile_width : pick_tile_width(M, N, kGemmBM, sm_count);
  if (width != 128 && width != 192 && width != 256) return DISTIE_ERR_ARG;
  status = make_map(&map_b, w, N, K, K, width);
  if (status != 0) return status;
#define DISTIE_GEMM(BNV, STAGESV, STAGES32)                                                                              \
  return epi == GEMM_EPI_F32                                                                                            \
             ? launch_gemm<BNV, STAGES32, GEMM_EPI_F32>(map_a, map_b, out, ldo, M, N, K, 0, sm_count, error, stream) \
             : launch_gemm<BNV, STAGESV, GEMM_EPI_BF16>(map_a, map_b, out, ldo, M, N, K, 0, sm_count, error, stream)
  if (width == 256) { DISTIE_GEMM(256, 4, 4); }
  if (width == 192) { DISTIE_GEMM(192, 5, 4); }
  DISTIE_GEMM(128, 6, 6);
#undef DISTIE_GEMM
}

// The q/k/v projection of prompt portions with its epilogue fused in: x[M >= 128, K] w[N, K]^T + bias, q and k
// rotated, q to q_out[M, num_heads * head_dim] (row stride ldq) and k and v into the paged cache, all bfloat16.
// `trig` [M, head_dim] float32 and `cache_row` [M] int32 come from distie_rope_rows (once per step); `cache_row`
// null: nothing is written to the cache.  head_dim 64 or 128; N = (num_heads + 2 * num_kv_heads) * head_dim.
extern "C" int distie_gemm_tcgen05_qkv(const void* x, int ldx, const void* w, const float* bias, const float* trig,
                                       const int* cache_row, void* q_out, int ldq, void* k_cache, void* v_cache, int M,
                                       int N, int K, int num_heads, int num_kv_heads, int head_dim, int page_size,
                                       int sm_count, int* error, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (M < kGemmBM || N < 1 || K < 8 || (K & 7) || (ldx & 7) || (ldq & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) ||
      ((uintptr_t)q_out & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)bias & 15) ||
      ((uintptr_t)trig & 15) || trig == nullptr || (head_dim != 64 && head_dim != 128) ||
      N != (num_heads + 2 * num_kv_heads) * head_dim || (cache_row != nullptr && (k_cache == nullptr || v_cache == nullptr)))
    return DISTIE_ERR_UNSUPPORTED;
  if (sm_count < 1) sm_count = 148;
  QkvEpilogue qkv;
  qkv.bias = bias;
  qkv.trig = trig;
  qkv.cache_row = cache_row;
  qkv.k_cache = (__nv_bfloat16*)k_cache;
  qkv.v_cache = (__nv_bfloat16*)v_cache;
  qkv.num_heads = num_heads;
  qkv.num_kv_heads = num_kv_heads;
  qkv.head_dim = head_dim;
  qkv.page_size = page_size;
  CUtensorMap map_a, map_b;
  int status = make_map(&map_a, x, M, K, ldx, kGemmBM);
  if (status != 0) return status;
  if (M >= 2 * kGemmBM && sm_count >= 2) {
    if ((status = make_map(&map_b, w, N, K, K, 128)) != 0) return status;
    return launch_gemm_pair<256, 4, 1, GEMM_EPI_QKV>(map_a, map_b, q_out, ldq, M, N, K, 0, sm_count, error, stream, qkv);
  }
  if ((status = make_map(&map_b, w, N, K, K, 256)) != 0) return status;
  return launch_gemm<256, 3, GEMM_EPI_QKV>(map_a, map_b, q_out, ldq, M, N, K, 0, sm_count, error, stream, qkv);
}

// ---- few rows of x: the weight-streaming orientation ------------------------------------------------------------
namespace distie {

static int skinny_splits(int tiles, int K, int sm_count) {
  const int k_blocks = (K + kGemmBK - 1) / kGemmBK;
  int splits = sm_count / tiles;                 // one CTA per SM at most: a second wave would wait for the first
  splits = min(splits, max(1, k_blocks / 4));    // at least four K blocks per CTA: below that a CTA's start and end outweigh its copies
  return max(1, min(splits, 10));                // every slice is written once and read once more by the consumer
}

template <int BN, int STAGES, int EPI, typename OutT>
static int launch_skinny_tc(const CUtensorMap& map_w, const CUtensorMap& map_x, const float* bias, OutT* out, int ldo,
                            int M, int N, int K, int inter, int tiles, int splits, int* error, cudaStream_t stream) {
  const size_t shared = sizeof(SkinnyShared<BN, STAGES>) + 1024;
  static bool configured = false;
  if (!configured) {
    const cudaError_t err = cudaFuncSetAttribute(gemm_tcgen05_skinny_kernel<BN, STAGES, EPI, OutT>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  const cudaError_t err =
      launch_dependent_family(16, gemm_tcgen05_skinny_kernel<BN, STAGES, EPI, OutT>, dim3(tiles, splits),
                              dim3(kGemmThreads), shared, stream, map_w, map_x, bias, out, ldo, M, N, K, inter, error);
  return err == cudaSuccess ? 0 : (int)err;
}

template <int EPI, typename OutT>
static int dispatch_skinny_tc(const CUtensorMap& map_w, const void* x, int ldx, const float* bias, OutT* out, int ldo,
                              int M, int N, int K, int inter, int tiles, int splits, int* error, cudaStream_t stream) {
  CUtensorMap map_x;
  int status;
  // A CTA whose share of K is four blocks long or less asks for a ring of four stages: the shared
  // memory it leaves free lets the CTAs of the kernel after it (launched early) move in beside it.
  const int k_blocks = (K + kGemmBK - 1) / kGemmBK;
  const bool brief = EPI == SKINNY_EPI_SLICE && (k_blocks + splits - 1) / splits <= 4;
  if (M <= 16) {
    if ((status = make_map(&map_x, x, M, K, ldx, 16)) != 0) return status;
    if (brief)
      return launch_skinny_tc<16, 4, EPI, OutT>(map_w, map_x, bias, out, ldo, M, N, K, inter, tiles, splits, error, stream);
    // The product that hands slices to a consumer runs on eight stages, the others on ten (measured:
    // a decode step is 1.3 % shorter than with ten for all, and longer again with seven).
    if (EPI == SKINNY_EPI_SLICE)
      return launch_skinny_tc<16, 8, EPI, OutT>(map_w, map_x, bias, out, ldo, M, N, K, inter, tiles, splits, error, stream);
    return launch_skinny_tc<16, 10, EPI, OutT>(map_w, map_x, bias, out, ldo, M, N, K, inter, tiles, splits, error, stream);
  }
  if (M <= 32) {
    if ((status = make_map(&map_x, x, M, K, ldx, 32)) != 0) return status;
    if (brief)
      return launch_skinny_tc<32, 4, EPI, OutT>(map_w, map_x, bias, out, ldo, M, N, K, inter, tiles, splits, error, stream);
    return launch_skinny_tc<32, 9, EPI, OutT>(map_w, map_x, bias, out, ldo, M, N, K, inter, tiles, splits, error, stream);
  }
  if ((status = make_map(&map_x, x, M, K, ldx, 64)) != 0) return status;
  return launch_skinny_tc<64, 7, EPI, OutT>(map_w, map_x, bias, out, ldo, M, N, K, inter, tiles, splits, error, stream);
}

}  // namespace distie

// Slices the call below writes for these sizes (mode 0).
extern "C" int distie_gemm_tcgen05_skinny_splits(int N, int K, int sm_count) {
  return skinny_splits((N + kGemmBM - 1) / kGemmBM, K, sm_count < 1 ? 148 : sm_count);
}

// x[M <= 64, K] (bfloat16, row stride ldx) against w[N, K] (bfloat16, contiguous).
//   mode 0: out[splits, M, N] float32 slices (ldo = N); their sum is x w^T
//   mode 1: out[M, N] bfloat16 (out_dtype 1) or float32 (0) = x w^T + bias
//   mode 2: w is [2 * inter, K]; out[M, inter] bfloat16 = silu(x Wg^T) * (x Wu^T)
extern "C" int distie_gemm_tcgen05_skinny(const void* x, int ldx, const void* w, const float* bias, void* out, int ldo,
                                          int M, int N, int K, int mode, int out_dtype, int sm_count, int* error,
                                          cudaStream_t stream) {
  if (M <= 0) return 0;
  if (M > 64 || N < 1 || K < 8 || (K & 7) || (ldx & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
    return DISTIE_ERR_UNSUPPORTED;
  if (sm_count < 1) sm_count = 148;
  CUtensorMap map_w;
  int status;
  if (mode == 2) {
    if (N & 1) return DISTIE_ERR_ARG;
    const int inter = N / 2;
    if ((status = make_map(&map_w, w, N, K, K, 64)) != 0) return status;
    return dispatch_skinny_tc<SKINNY_EPI_SWIGLU, __nv_bfloat16>(map_w, x, ldx, nullptr, (__nv_bfloat16*)out, ldo, M, N, K,
                                                                 inter, (inter + 63) / 64, 1, error, stream);
  }
  if ((status = make_map(&map_w, w, N, K, K, kGemmBM)) != 0) return status;
  const int tiles = (N + kGemmBM - 1) / kGemmBM;
  if (mode == 0)
    return dispatch_skinny_tc<SKINNY_EPI_SLICE, float>(map_w, x, ldx, nullptr, (float*)out, N, M, N, K, 0, tiles,
                                                       skinny_splits(tiles, K, sm_count), error, stream);
  if (mode != 1) return DISTIE_ERR_ARG;
  if (out_dtype == DISTIE_F32)
    return dispatch_skinny_tc<SKINNY_EPI_STORE, float>(map_w, x, ldx, bias, (float*)out, ldo, M, N, K, 0, tiles, 1, error,
                                                       stream);
  return dispatch_skinny_tc<SKINNY_EPI_STORE, __nv_bfloat16>(map_w, x, ldx, bias, (__nv_bfloat16*)out, ldo, M, N, K, 0,
                                                             tiles, 1, error, stream);
}
