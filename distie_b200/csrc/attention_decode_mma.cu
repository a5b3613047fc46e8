// Split-KV attention for single tokens (decoding) on the tensor cores, bfloat16.
//
// Decoding reads every cached key and value of a request once per step.  The
// float32-math kernel in attention_decode.cu spends far more instructions per
// byte than the memory system needs time per byte (a dot product per key and
// head on the CUDA cores, reduced over lanes with shuffles); this one lets the
// tensor cores do the products so that the loads set the pace:
//
//   grid   (token, kv head * chunks of up to 16 query heads, split)
//   block  4 warps; a warp takes groups of 16 keys of the split in turn
//   S      the query heads of the group are the 16 rows of mma.m16n8k16, 8 keys
//          the columns, head_dim the reduction:  S[head, key] = q[head] . k[key]
//   P V    the same heads are the rows, 16 keys the reduction, head_dim the columns
//
// Operands come from global memory in 16-byte pieces that are already the lanes' mma
// fragments, so nothing is rearranged on the way: the reduction index of an mma may be enumerated in any order as long as
// both operands agree, and so may the columns of the output.  A lane therefore
// loads 8 consecutive elements of a key row and uses them as its share of two
// k-steps of S, and 2 * head_dim / 16 consecutive elements of 4 value rows, from
// which it assembles its B fragments of P V with byte permutes; output column
// (n-tile t, lane group g) stands for dimension g * head_dim / 8 + t.
//
// The pieces travel through a small ring in shared memory (cp.async, three groups of 16 keys per
// warp): the copies of the next two groups are in flight while a group is computed, which is what
// keeps enough bytes in the air with only eight warps per SM.  Each lane reads back exactly the
// pieces it copied, so the ring needs no layout beyond [stage][load][lane].
//
// Softmax state (max, sum) is float32 per lane; the four warps and, with several
// splits, the CTAs of a token are merged as in the other kernel (same scratch
// layout, same merge kernel).  head_dim 64 or 128.
#include "common.cuh"

namespace distie {

constexpr int kMmaDecodeWarps = 4;
constexpr int kMmaDecodeClusterSplits = 8;  // splits that one cluster can hold (portable cluster size)
constexpr int kMmaDecodePages = 1024;       // page ids of a split that are kept in shared memory

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

// Keys and values are read once and the newest row was written by the kernel just before this one,
// which may still have been running when this kernel started: through L2, past L1.
__device__ __forceinline__ uint4 load16(const void* p) { return load16_cg(p); }

__device__ __forceinline__ void mma_16816_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint32_t word_of(const uint4& v, int i) {
  return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// STAGES groups of 16 keys per warp are in flight or in use: 3 for few CTAs (deep prefetch), 2 for many
// (three CTAs fit an SM then, and twelve warps hide more latency than eight).
template <int D, int STAGES>
__global__ void __launch_bounds__(kMmaDecodeWarps * 32)
attention_decode_mma_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride, __nv_bfloat16* __restrict__ out,
                            int out_row_stride, float* __restrict__ scratch_o, float* __restrict__ scratch_ml,
                            const int* __restrict__ positions, const int* __restrict__ token_seq,
                            const int* __restrict__ seq_seat, const int* __restrict__ block_table, int table_width,
                            const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                            int num_heads, int group_size, int head_chunks, int num_kv_heads, int page_size,
                            int page_shift, int num_pages, int window, float scale_log2, int cluster_merge,
                            int* __restrict__ error) {
  constexpr int QC = D / 32;      // 16-byte pieces of a key row per lane (and of a query row)
  constexpr int NT = D / 8;       // output n-tiles
  constexpr int VW = D / 64;      // 16-byte pieces of a value row per lane
  constexpr int LOADS = 2 * QC + 4 * VW;  // 16-byte pieces per lane and group of 16 keys
  extern __shared__ __align__(16) unsigned char dyn[];
  // The ring of the main loop and the merge area of the tail share the dynamic shared memory.
  uint4* ring = reinterpret_cast<uint4*>(dyn);  // [warp][stage][load][lane]
  float(*sh_o)[16][D + 1] = reinterpret_cast<float(*)[16][D + 1]>(dyn);
  // This split's result, read by the other CTAs of a cluster: behind the merge area.
  float(*cl_o)[D] = reinterpret_cast<float(*)[D]>(dyn + kMmaDecodeWarps * 16 * (D + 1) * sizeof(float));
  __shared__ float sh_m[kMmaDecodeWarps][16], sh_l[kMmaDecodeWarps][16];
  __shared__ float cl_m[16], cl_l[16];
  __shared__ int sh_pages[kMmaDecodePages];           // the split's part of the block table

  grid_dependency_release();
  const int t = blockIdx.x;
  const int kv_head = blockIdx.y / head_chunks, chunk = blockIdx.y % head_chunks;
  const int split = blockIdx.z, num_splits = gridDim.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int head0 = kv_head * group_size + chunk * 16;
  const int heads_here = min(16, group_size - chunk * 16);

  const int pos = positions[t];
  const int seat = seq_seat[token_seq[t]];
  const int* table = block_table + (size_t)seat * table_width;
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int first_page = first / page_size;
  const int pages = pos / page_size - first_page + 1;
  const int pages_per_split = (pages + num_splits - 1) / num_splits;
  const int split_page = first_page + split * pages_per_split;
  const int lo = max(first, split_page * page_size);
  const int hi = min(pos, (split_page + pages_per_split) * page_size - 1);
  // The split's page ids come into shared memory in one round of loads (requested here, stored after
  // the first copies are on their way); a row of keys then costs no dependent global load before its
  // copy can be issued.  Until they are there (`staged_ready`), the table itself is read.
  constexpr int kStagedPerThread = kMmaDecodePages / (kMmaDecodeWarps * 32);
  int staged[kStagedPerThread];
#pragma unroll
  for (int u = 0; u < kStagedPerThread; ++u) {
    const int i = threadIdx.x + u * kMmaDecodeWarps * 32;
    staged[u] = (i < pages_per_split && split_page + i < table_width) ? table[split_page + i] : -1;
  }
  bool staged_ready = false;
  auto page_of = [&](int key) {
    const int column = page_shift >= 0 ? key >> page_shift : key / page_size;
    const int i = column - split_page;
    return (staged_ready && i < kMmaDecodePages) ? sh_pages[i] : table[column];
  };

  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int r = 0; r < 4; ++r) o[i][r] = 0.f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};

  const int lo16 = lo & ~15;
  const int groups = hi >= lo ? (hi - lo16) / 16 + 1 : 0;
  uint4* my_ring = ring + (size_t)warp * STAGES * LOADS * 32;
  // Issues the copies of one group of 16 keys into a stage of this warp's ring: 2 key rows (columns g
  // and g + 8 of S) and 4 value rows (reduction slots 2c, 2c+1, 2c+8, 2c+9 of P V) per lane.
  auto issue = [&](int grp, int stage) {
    const int base_key = lo16 + grp * 16;
    uint4* dst = my_ring + (size_t)stage * LOADS * 32 + lane;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int key = base_key + g + 8 * h;
      bool ok = grp < groups && key >= lo && key <= hi;
      size_t at = 0;
      if (ok) {
        // page_shift >= 0: the page size is a power of two, so no division per row.
        const int page = page_of(key);
        const int within = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
        if (page < 0 || page >= num_pages) {
          if (error) atomicExch(error, 4);
          ok = false;
        } else {
          at = (((size_t)page * num_kv_heads + kv_head) * page_size + within) * D + 8 * c;
        }
      }
#pragma unroll
      for (int j = 0; j < QC; ++j)
        cp_async16((uint32_t)__cvta_generic_to_shared(dst + (h * QC + j) * 32), k_cache + at + 32 * j, ok ? 16 : 0);
    }
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int key = base_key + 2 * c + (s & 1) + 8 * (s >> 1);
      bool ok = grp < groups && key >= lo && key <= hi;
      size_t at = 0;
      if (ok) {
        const int page = page_of(key);
        const int within = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
        if (page < 0 || page >= num_pages) {
          ok = false;
        } else {
          at = (((size_t)page * num_kv_heads + kv_head) * page_size + within) * D + g * (D / 8);
        }
      }
#pragma unroll
      for (int w = 0; w < VW; ++w)
        cp_async16((uint32_t)__cvta_generic_to_shared(dst + (2 * QC + s * VW + w) * 32), v_cache + at + 8 * w,
                   ok ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // Positions, seats and tables are inputs of the step.  Of the cache only the row of the newest
  // position comes from the kernel before this one (every other row was written in an earlier step),
  // so groups of keys that end before it are requested before the wait; q comes after it.
  const bool early0 = lo16 + warp * 16 + 15 < pos;
  const bool early1 = STAGES > 2 && early0 && lo16 + (warp + kMmaDecodeWarps) * 16 + 15 < pos;
  if (early0) issue(warp, 0);
  if (early1) issue(warp + kMmaDecodeWarps, 1);
  grid_dependency_wait();
  if (!early0) issue(warp, 0);
  if (STAGES > 2 && !early1) issue(warp + kMmaDecodeWarps, 1);
  // Query fragments: rows g and g + 8 of the head chunk, 8 consecutive dims per piece.
  uint4 qa[QC], qb[QC];
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int j = 0; j < QC; ++j) {
    const __nv_bfloat16* base = q + (size_t)t * q_row_stride + 32 * j + 8 * c;
    qa[j] = g < heads_here ? load16_cg(base + (size_t)(head0 + g) * D) : zero;
    qb[j] = g + 8 < heads_here ? load16_cg(base + (size_t)(head0 + g + 8) * D) : zero;
  }
#pragma unroll
  for (int u = 0; u < kStagedPerThread; ++u) sh_pages[threadIdx.x + u * kMmaDecodeWarps * 32] = staged[u];
  __syncthreads();
  staged_ready = true;
  int stage = 0;
  for (int grp = warp; grp < groups; grp += kMmaDecodeWarps) {
    const int base_key = lo16 + grp * 16;
    issue(grp + (STAGES - 1) * kMmaDecodeWarps, (stage + STAGES - 1) % STAGES);  // empty group past the end
    if (STAGES > 2) asm volatile("cp.async.wait_group 2;" ::: "memory");
    else asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncwarp();
    uint4 kr[2][QC], vr[4][VW];
    const uint4* src = my_ring + (size_t)stage * LOADS * 32 + lane;
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int j = 0; j < QC; ++j) kr[h][j] = src[(h * QC + j) * 32];
#pragma unroll
    for (int s = 0; s < 4; ++s)
#pragma unroll
      for (int w = 0; w < VW; ++w) vr[s][w] = src[(2 * QC + s * VW + w) * 32];
    stage = (stage + 1) % STAGES;

    // ---- S = Q K^T for keys base..base+7 (s1) and base+8..base+15 (s2) ---------------------------
    float s1[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < QC; ++j) {
      mma_16816_bf16(s1, qa[j].x, qb[j].x, qa[j].y, qb[j].y, kr[0][j].x, kr[0][j].y);
      mma_16816_bf16(s1, qa[j].z, qb[j].z, qa[j].w, qb[j].w, kr[0][j].z, kr[0][j].w);
      mma_16816_bf16(s2, qa[j].x, qb[j].x, qa[j].y, qb[j].y, kr[1][j].x, kr[1][j].y);
      mma_16816_bf16(s2, qa[j].z, qb[j].z, qa[j].w, qb[j].w, kr[1][j].z, kr[1][j].w);
    }

    // ---- mask and online softmax; rows: [0] head g, [1] head g + 8 ----------------------------------
    float p1[4], p2[4], corr[2];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int key1 = base_key + 2 * c + (r & 1), key2 = key1 + 8;
      p1[r] = (key1 >= lo && key1 <= hi) ? s1[r] * scale_log2 : -INFINITY;
      p2[r] = (key2 >= lo && key2 <= hi) ? s2[r] * scale_log2 : -INFINITY;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float m = fmaxf(fmaxf(p1[2 * h], p1[2 * h + 1]), fmaxf(p2[2 * h], p2[2 * h + 1]));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      const float m_new = fmaxf(row_max[h], m);
      corr[h] = m_new == -INFINITY ? 1.f : exp2f(row_max[h] - m_new);
      row_max[h] = m_new;
      const float shift = m_new == -INFINITY ? 0.f : m_new;
      float sum = 0.f;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        p1[2 * h + e] = exp2f(p1[2 * h + e] - shift);
        p2[2 * h + e] = exp2f(p2[2 * h + e] - shift);
        sum += p1[2 * h + e] + p2[2 * h + e];
      }
      row_sum[h] = row_sum[h] * corr[h] + sum;
    }
    const uint32_t a0 = pack2(p1[0], p1[1]), a1 = pack2(p1[2], p1[3]);
    const uint32_t a2 = pack2(p2[0], p2[1]), a3 = pack2(p2[2], p2[3]);

    // ---- O = O * corr + P V --------------------------------------------------------------------------
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      o[nt][0] *= corr[0]; o[nt][1] *= corr[0];
      o[nt][2] *= corr[1]; o[nt][3] *= corr[1];
      const int w = (nt >> 1) & 3, piece = nt >> 3;
      const uint32_t sel = (nt & 1) ? 0x7632u : 0x5410u;
      const uint32_t b0 = __byte_perm(word_of(vr[0][piece], w), word_of(vr[1][piece], w), sel);
      const uint32_t b1 = __byte_perm(word_of(vr[2][piece], w), word_of(vr[3][piece], w), sel);
      mma_16816_bf16(o[nt], a0, a1, a2, a3, b0, b1);
    }
  }

  // ---- merge the warps ---------------------------------------------------------------------------------
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();  // the ring is done with: its memory becomes the merge area
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float l = row_sum[h];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (c == 0) { sh_m[warp][g + 8 * h] = row_max[h]; sh_l[warp][g + 8 * h] = l; }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      sh_o[warp][g + 8 * h][(2 * c) * (D / 8) + nt] = o[nt][2 * h];
      sh_o[warp][g + 8 * h][(2 * c + 1) * (D / 8) + nt] = o[nt][2 * h + 1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < heads_here * D; idx += kMmaDecodeWarps * 32) {
    const int hd = idx / D, e = idx % D;
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMmaDecodeWarps; ++w) m_all = fmaxf(m_all, sh_m[w][hd]);
    float l_all = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kMmaDecodeWarps; ++w) {
      const float weight = sh_m[w][hd] == -INFINITY ? 0.f : exp2f(sh_m[w][hd] - m_all);
      l_all += sh_l[w][hd] * weight;
      acc += sh_o[w][hd][e] * weight;
    }
    const int head = head0 + hd;
    if (num_splits == 1) {
      out[(size_t)t * out_row_stride + (size_t)head * D + e] = __float2bfloat16_rn(l_all > 0.f ? acc / l_all : 0.f);
    } else if (cluster_merge) {
      cl_o[hd][e] = acc;
      if (e == 0) { cl_m[hd] = m_all; cl_l[hd] = l_all; }
    } else {
      const size_t row = ((size_t)t * num_heads + head) * num_splits + split;
      scratch_o[row * D + e] = acc;
      if (e == 0) {
        scratch_ml[row * 2] = m_all;  // in base-2 units, like everything in this file
        scratch_ml[row * 2 + 1] = l_all;
      }
    }
  }
  if (num_splits > 1 && cluster_merge) {
    // The splits of a (token, head chunk) are the CTAs of one cluster: each combines its share of the
    // output elements from every CTA's shared memory, splits in order, as the merge kernel would.
    cluster_barrier();
    const int total = heads_here * D;
    const int share = (total + num_splits - 1) / num_splits;
    const int end = min(total, (split + 1) * share);
    for (int idx = split * share + threadIdx.x; idx < end; idx += kMmaDecodeWarps * 32) {
      const int hd = idx / D, e = idx % D;
      float m_all = -INFINITY;
      for (int s = 0; s < num_splits; ++s) m_all = fmaxf(m_all, cluster_load(&cl_m[hd], s));
      float l_all = 0.f, acc = 0.f;
      for (int s = 0; s < num_splits; ++s) {
        const float ms = cluster_load(&cl_m[hd], s);
        const float weight = ms == -INFINITY ? 0.f : exp2f(ms - m_all);
        l_all += cluster_load(&cl_l[hd], s) * weight;
        acc += cluster_load(&cl_o[hd][e], s) * weight;
      }
      out[(size_t)t * out_row_stride + (size_t)(head0 + hd) * D + e] = __float2bfloat16_rn(l_all > 0.f ? acc / l_all : 0.f);
    }
    cluster_barrier();  // no CTA leaves while another may still read its shared memory
  }
}

// Combines the partial results of the splits of one (token, head): maxima are base-2 exponents.
__global__ void __launch_bounds__(128)
attention_decode_mma_merge_kernel(const float* __restrict__ scratch_o, const float* __restrict__ scratch_ml,
                                  __nv_bfloat16* __restrict__ out, int out_row_stride, int num_heads, int head_dim,
                                  int num_splits) {
  grid_dependency_release();
  grid_dependency_wait();
  const int t = blockIdx.x, head = blockIdx.y;
  const size_t row0 = ((size_t)t * num_heads + head) * num_splits;
  float m_all = -INFINITY;
  for (int s = 0; s < num_splits; ++s) m_all = fmaxf(m_all, __ldcg(scratch_ml + (row0 + s) * 2));
  for (int e = threadIdx.x; e < head_dim; e += blockDim.x) {
    float l_all = 0.f, acc = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float ms = __ldcg(scratch_ml + (row0 + s) * 2);
      const float weight = ms == -INFINITY ? 0.f : exp2f(ms - m_all);
      l_all += __ldcg(scratch_ml + (row0 + s) * 2 + 1) * weight;
      acc += __ldcg(scratch_o + (row0 + s) * head_dim + e) * weight;
    }
    out[(size_t)t * out_row_stride + (size_t)head * head_dim + e] =
        __float2bfloat16_rn(l_all > 0.f ? acc / l_all : 0.f);
  }
}

}  // namespace distie

using namespace distie;

// Stages of the key/value ring (and with them the CTAs that fit an SM: 2 with three stages, 3 with two)
// for `tokens` single tokens and `blocks_per_token` CTAs per token and split.
extern "C" int distie_attention_decode_mma_stages(int tokens, int blocks_per_token, int sm_count) {
  return (long long)tokens * blocks_per_token * 2 >= sm_count ? 2 : 3;
}

// Same arguments and scratch layout as distie_attention_decode (bfloat16 only).
extern "C" int distie_attention_decode_mma(const void* q, int q_row_stride, void* out, int out_row_stride,
                                           float* scratch, const int* positions, const int* token_seq,
                                           const int* seq_seat, const int* block_table, int table_width,
                                           const void* k_cache, const void* v_cache, int tokens, int num_heads,
                                           int num_kv_heads, int head_dim, int page_size, int num_pages, int window,
                                           float scale, int num_splits, int* error, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads != 0 || page_size < 1 || table_width < 1 ||
      num_splits < 1 || num_splits > 65535 || (num_splits > kMmaDecodeClusterSplits && scratch == nullptr) || (q_row_stride & 7))
    return DISTIE_ERR_ARG;
  if (head_dim != 64 && head_dim != 128) return DISTIE_ERR_UNSUPPORTED;
  const int group = num_heads / num_kv_heads;
  const int chunks = (group + 15) / 16;
  const dim3 grid(tokens, num_kv_heads * chunks, num_splits);
  float* scratch_o = scratch;
  float* scratch_ml = scratch ? scratch + (size_t)tokens * num_heads * num_splits * head_dim : nullptr;
  const float scale_log2 = scale * 1.4426950408889634f;
  int page_shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (page_shift = 0; (1 << page_shift) < page_size; ++page_shift) {
    }
  cudaError_t err;
  // Many CTAs: two stages, so that three CTAs fit an SM; few: three stages.
  static int sm_count = 0;
  if (sm_count == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sm_count < 1)
      sm_count = 148;
  }
  const int stages = distie_attention_decode_mma_stages(tokens, num_kv_heads * chunks, sm_count);
  // Dynamic shared memory: the larger of the ring (warps x stages x loads x 512 bytes) and the merge areas.
  const size_t loads = 2 * (head_dim / 32) + 4 * (head_dim / 64);
  const size_t ring_bytes = (size_t)kMmaDecodeWarps * stages * loads * 512;
  const size_t merge_bytes = (size_t)kMmaDecodeWarps * 16 * (head_dim + 1) * sizeof(float) + 16 * head_dim * sizeof(float);
  const size_t shared = ring_bytes > merge_bytes ? ring_bytes : merge_bytes;
  static bool configured = false;
  if (!configured) {
    err = cudaFuncSetAttribute(attention_decode_mma_kernel<64, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(attention_decode_mma_kernel<64, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(attention_decode_mma_kernel<128, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(attention_decode_mma_kernel<128, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  // Up to 8 splits (the portable cluster size) are merged inside the kernel, through the cluster's shared memory.
  const int cluster_merge = (num_splits > 1 && num_splits <= kMmaDecodeClusterSplits) ? 1 : 0;
  const dim3 cluster = cluster_merge ? dim3(1, 1, num_splits) : dim3(0, 0, 0);
#define DISTIE_MMA_DECODE(DV, SV)                                                                                  \
  err = launch_dependent_cluster(8, cluster, attention_decode_mma_kernel<DV, SV>, grid, dim3(kMmaDecodeWarps * 32), shared, \
                         stream, (const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, out_row_stride, scratch_o, \
                         scratch_ml, positions, token_seq, seq_seat, block_table, table_width,                     \
                         (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, num_heads, group, chunks,   \
                         num_kv_heads, page_size, page_shift, num_pages, window, scale_log2, cluster_merge, error)
  if (head_dim == 64) {
    if (stages == 2) DISTIE_MMA_DECODE(64, 2);
    else DISTIE_MMA_DECODE(64, 3);
  } else {
    if (stages == 2) DISTIE_MMA_DECODE(128, 2);
    else DISTIE_MMA_DECODE(128, 3);
  }
#undef DISTIE_MMA_DECODE
  if (err != cudaSuccess) return (int)err;
  if (num_splits > 1 && !cluster_merge) {
    const dim3 merge_grid(tokens, num_heads);
    err = launch_dependent_family(8, attention_decode_mma_merge_kernel, merge_grid, dim3(head_dim >= 128 ? 128 : 64), 0, stream,
                           (const float*)scratch_o, (const float*)scratch_ml, (__nv_bfloat16*)out, out_row_stride,
                           num_heads, head_dim, num_splits);
    if (err != cudaSuccess) return (int)err;
  }
  return 0;
}
