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
//   S^T    the 16 keys of a group are the rows of mma.m16n8k16, the (up to 8, or 2 x 8) query heads
//          that share the kv head are the columns, head_dim the reduction: S^T[key, head] = k[key] . q[head]
//   O^T    16 dims are the rows, the heads the columns, the 16 keys the reduction: O^T += V^T P^T
//
// With the heads as the narrow side, 16 keys cost head_dim / 16 MMAs for the scores and as many for
// the output, whatever the number of heads up to 8; the accumulators are head_dim / 4 registers.
// K and V rows travel by cp.async into a per-warp ring in shared memory whose 16-byte chunks are
// swizzled (chunk ^ (row & 7)), so that ldmatrix reads the A operands -- K as it lies, V transposed --
// without bank conflicts.  P^T becomes the B operand of the second product with two movmatrix
// transposes.  Column maxima and sums (per head, over keys) are reduced over the lanes that hold
// the same column.
//
// Softmax state (max, sum) is float32 per lane; the four warps and, with several splits, the CTAs of a
// token are merged as in the other kernel (same scratch layout, same merge kernel).  head_dim 64 or 128.
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

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// An 8 x 8 matrix of 16-bit values held as an mma C-style fragment (lane = row * 4 + column pair), transposed.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

// STAGES groups of 16 keys per warp are in flight or in use: 3 for few CTAs (deep prefetch), 2 for many
// (three CTAs fit an SM then, and twelve warps hide more latency than eight).
// NH: column tiles of 8 query heads (1 for up to 8 heads per kv head, 2 for up to 16).
// PAGE16: the page size is a power of two >= 16, so a group of 16 keys lies in one page.
// (The kernel runs for microseconds; its code is kept small -- one form of the copy loop per
// instantiation, few inlined copies of it -- because fetching instructions is part of that time.)
//
// FUSED: the kernel starts from the q/k/v projection itself instead of from a rotated q and a cache that
// already holds the token's key and value.  `proj` is the projection's float32 slices (see ProjectionInput).
// The threads of the CTA share out its query heads (and, in the split that holds the token's own position,
// the token's key and value of its kv head) in units of 4 dims and their partners half a head further on: a
// thread adds up the slices of its unit, all loads in flight together, adds the bias, rotates with cos and
// sin of the position (computed once per CTA before the dependency wait) and leaves the result as bfloat16
// in shared memory, from where the lanes take their MMA fragments as they would from a q in global memory.
// The token's key and value also go into their cache page, and the warp that owns the last group of keys
// puts them over that row of its tile.  The kernel that did all this for a decode step, one link of the
// chain of dependent kernels, is then not launched.
struct ProjectionInput {
  const float* slices;     // [splits, tokens, row_stride]: q heads, then k heads, then v heads, head_dim each
  int splits;
  long long split_stride;  // floats between slices
  int row_stride;          // floats per token
  const float* bias;       // [row_stride] or null
  const float* inv_freq;   // [head_dim / 2] or null (nothing is rotated)
  float trig_factor;
  int write_new;           // 0: the cache already holds the token's key and value (a layer that reads another's cache)
};

template <int D, int STAGES, int NH, bool PAGE16, bool FUSED>
__global__ void __launch_bounds__(kMmaDecodeWarps * 32)
attention_decode_mma_kernel(const ProjectionInput proj,
                            const __nv_bfloat16* __restrict__ q, int q_row_stride, __nv_bfloat16* __restrict__ out,
                            int out_row_stride, float* __restrict__ scratch_o, float* __restrict__ scratch_ml,
                            const int* __restrict__ positions, const int* __restrict__ token_seq,
                            const int* __restrict__ seq_seat, const int* __restrict__ block_table, int table_width,
                            const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                            int num_heads, int group_size, int head_chunks, int num_kv_heads, int page_size,
                            int page_shift, int num_pages, int window, float scale_log2, int cluster_merge,
                            int* __restrict__ error) {
  constexpr int CPR = D / 8;                 // 16-byte chunks per row of keys or values
  constexpr int ROW_BYTES = D * 2;
  constexpr int TILE_BYTES = 16 * ROW_BYTES;  // 16 keys (or values)
  constexpr int COPIES = 16 * CPR / 32;       // chunks a lane copies per tile
  constexpr int MT = D / 16;                  // 16-dim row tiles of O^T, and k-steps of S^T
  extern __shared__ __align__(128) unsigned char dyn[];
  // The ring of the main loop ([warp][stage][K tile | V tile]) and the merge area of the tail share the
  // dynamic shared memory.
  float(*sh_o)[16][D + 1] = reinterpret_cast<float(*)[16][D + 1]>(dyn);
  // This split's result, read by the other CTAs of a cluster: behind the merge area.
  float(*cl_o)[D] = reinterpret_cast<float(*)[D]>(dyn + kMmaDecodeWarps * 16 * (D + 1) * sizeof(float));
  __shared__ float sh_m[kMmaDecodeWarps][16], sh_l[kMmaDecodeWarps][16];
  __shared__ float cl_m[16], cl_l[16];
  __shared__ int sh_pages[kMmaDecodePages];           // the split's part of the block table
  // FUSED: q of this CTA's heads (rows 0 .. 8 NH - 1), then the token's key and value of this kv head, rotated,
  // as bfloat16 (rows 16 bytes longer than a head, against bank conflicts); and cos | sin of the position.
  constexpr int HALF = D / 2;
  constexpr int QROW = D + 8;
  __shared__ __align__(16) __nv_bfloat16 sh_q[FUSED ? (NH * 8 + 2) * QROW : 8];
  __shared__ __align__(16) float sh_trig[FUSED ? D : 4];

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
  if (FUSED && threadIdx.x < HALF) {  // the angles depend on the position alone, an input of the step
    float sn = 0.f, cs = 1.f;
    if (proj.inv_freq) {
      sincosf((float)pos * proj.inv_freq[threadIdx.x], &sn, &cs);
      cs *= proj.trig_factor;
      sn *= proj.trig_factor;
    }
    sh_trig[threadIdx.x] = cs;
    sh_trig[HALF + threadIdx.x] = sn;
  }
  if (FUSED) __syncthreads();  // (before the wait: it delays nothing)
  // The split that holds the token's own position puts the token's key and value in place itself.
  const bool owns_new = FUSED && proj.write_new && hi == pos && lo <= pos;
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
    if (staged_ready && i < kMmaDecodePages) return sh_pages[i];
    return column < table_width ? table[column] : -1;  // past the end of the table: reported as a missing page
  };

  float o[NH][MT][4];  // O^T: [dim 16 mt + g (+8)][head 8 nh + 2c (+1)]
#pragma unroll
  for (int nh = 0; nh < NH; ++nh)
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int r = 0; r < 4; ++r) o[nh][i][r] = 0.f;
  float col_max[NH][2], col_sum[NH][2];  // of heads 8 nh + 2c and + 1; the sums over this lane's keys only
#pragma unroll
  for (int nh = 0; nh < NH; ++nh) {
    col_max[nh][0] = col_max[nh][1] = -INFINITY;
    col_sum[nh][0] = col_sum[nh][1] = 0.f;
  }

  const int lo16 = lo & ~15;
  const int groups = hi >= lo ? (hi - lo16) / 16 + 1 : 0;
  const uint32_t my_ring = (uint32_t)__cvta_generic_to_shared(dyn) + (uint32_t)warp * STAGES * 2 * TILE_BYTES;
  // Issues the copies of one group of 16 keys into a stage of this warp's ring: chunk `id` of the tile
  // (row id / CPR, chunk id % CPR) goes to row * ROW_BYTES + ((chunk ^ (row & 7)) * 16), K and V alike.
  constexpr int RPI = 32 / CPR;  // rows of a tile that one copy instruction of the warp covers
  const int row0 = lane / CPR, ch = lane % CPR;  // this lane's row within those, and its chunk of the row
  auto issue = [&](int grp, int stage) {
    const int base_key = lo16 + grp * 16;
    const uint32_t k_dst = my_ring + (uint32_t)stage * 2 * TILE_BYTES, v_dst = k_dst + TILE_BYTES;
    const bool live = grp < groups;
    if (PAGE16) {
      // Pages of 16, 32, ... rows: the group lies in one page, whose id is looked up once; the rows
      // are then a fixed distance apart.  Groups inside [lo, hi] need no test per row.
      const int page = live ? page_of(base_key) : 0;
      const bool page_ok = live && page >= 0 && page < num_pages;
      if (live && !page_ok && error) atomicExch(error, 4);
      const size_t at = (((size_t)(page_ok ? page : 0) * num_kv_heads + kv_head) * page_size +
                         (base_key & (page_size - 1)) + row0) * D + ch * 8;
      const __nv_bfloat16* k_src = k_cache + at;
      const __nv_bfloat16* v_src = v_cache + at;
      const bool whole = page_ok && base_key >= lo && base_key + 15 <= hi;
#pragma unroll
      for (int i = 0; i < COPIES; ++i) {
        const int row = i * RPI + row0;
        const bool ok = whole || (page_ok && base_key + row >= lo && base_key + row <= hi);
        const uint32_t offset = (uint32_t)(row * ROW_BYTES + ((ch ^ (row & 7)) << 4));
        cp_async16(k_dst + offset, ok ? k_src + i * RPI * D : k_cache, ok ? 16 : 0);
        cp_async16(v_dst + offset, ok ? v_src + i * RPI * D : v_cache, ok ? 16 : 0);
      }
    } else {
#pragma unroll
      for (int i = 0; i < COPIES; ++i) {
        const int row = i * RPI + row0;
        const int key = base_key + row;
        bool ok = live && key >= lo && key <= hi;
        size_t at = 0;
        if (ok) {
          const int page = page_of(key);
          const int within = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
          if (page < 0 || page >= num_pages) {
            if (error) atomicExch(error, 4);
            ok = false;
          } else {
            at = (((size_t)page * num_kv_heads + kv_head) * page_size + within) * D + ch * 8;
          }
        }
        const uint32_t offset = (uint32_t)(row * ROW_BYTES + ((ch ^ (row & 7)) << 4));
        cp_async16(k_dst + offset, k_cache + at, ok ? 16 : 0);
        cp_async16(v_dst + offset, v_cache + at, ok ? 16 : 0);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // Positions, seats and tables are inputs of the step.  Of the cache only the row of the newest
  // position comes from the kernel before this one (every other row was written in an earlier step),
  // so groups of keys that end before it are requested before the wait; q comes after it.
  int issued = 0;
#pragma unroll 1
  for (; issued < STAGES - 1; ++issued) {
    if (lo16 + (warp + issued * kMmaDecodeWarps) * 16 + 15 >= pos) break;
    issue(warp + issued * kMmaDecodeWarps, issued);
  }
  grid_dependency_wait();
#pragma unroll 1
  for (; issued < STAGES - 1; ++issued) issue(warp + issued * kMmaDecodeWarps, issued);
  // B fragments of S^T = K Q^T: for k-step ks, dims 16 ks + 2c, + 1 and 16 ks + 2c + 8, + 9 of head g.
  uint32_t qb[NH][MT][2];
  if (!FUSED) {
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
      const int hd = nh * 8 + g;
      const __nv_bfloat16* row = q + (size_t)t * q_row_stride + (size_t)(head0 + hd) * D + 2 * c;
#pragma unroll
      for (int ks = 0; ks < MT; ++ks) {
        qb[nh][ks][0] = hd < heads_here ? __ldcg(reinterpret_cast<const unsigned int*>(row + 16 * ks)) : 0u;
        qb[nh][ks][1] = hd < heads_here ? __ldcg(reinterpret_cast<const unsigned int*>(row + 16 * ks + 8)) : 0u;
      }
    }
  } else {
    // Units of 4 dims j0 .. j0 + 3 and their partners HALF further on: this CTA's query heads, then (in the
    // split that owns the new position) the token's key and value of its kv head.
    constexpr int UPH = HALF / 4;  // units per head
    constexpr int ROUND = 8;       // slices in flight together
    const int units = (heads_here + (owns_new ? 2 : 0)) * UPH;
    const float* row = proj.slices + (size_t)t * proj.row_stride;
    __nv_bfloat16* new_k_row = nullptr;  // the token's row of the page, for the CTA that writes it
    __nv_bfloat16* new_v_row = nullptr;
    if (owns_new && chunk == 0) {  // (one CTA per kv head writes the page; every head chunk needs the row)
      const int page = page_of(pos);
      if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0 && error) atomicExch(error, 2);
      } else {
        const int within = page_shift >= 0 ? pos & (page_size - 1) : pos % page_size;
        const size_t at = (((size_t)page * num_kv_heads + kv_head) * page_size + within) * D;
        new_k_row = const_cast<__nv_bfloat16*>(k_cache) + at;
        new_v_row = const_cast<__nv_bfloat16*>(v_cache) + at;
      }
    }
    for (int unit = threadIdx.x; unit < units; unit += kMmaDecodeWarps * 32) {
      const int hd = unit / UPH, j0 = (unit % UPH) * 4;
      int column, slot;  // where the head starts in the projection's row, and its row of sh_q
      __nv_bfloat16* page_row = nullptr;
      if (hd < heads_here) { column = (head0 + hd) * D; slot = hd; }
      else if (hd == heads_here) { column = (num_heads + kv_head) * D; slot = NH * 8; page_row = new_k_row; }
      else { column = (num_heads + num_kv_heads + kv_head) * D; slot = NH * 8 + 1; page_row = new_v_row; }
      const float* first = row + column + j0;
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;  // slices in order, then the bias, as the separate kernel adds
      for (int s0 = 0; s0 < proj.splits; s0 += ROUND) {
        float4 da[ROUND], db[ROUND];
#pragma unroll
        for (int u = 0; u < ROUND; ++u) {
          if (s0 + u < proj.splits) {
            const float* slice = first + (size_t)(s0 + u) * proj.split_stride;
            da[u] = load4_cg(slice);
            db[u] = load4_cg(slice + HALF);
          } else {
            da[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            db[u] = da[u];
          }
        }
#pragma unroll
        for (int u = 0; u < ROUND; ++u) {
          a.x += da[u].x; a.y += da[u].y; a.z += da[u].z; a.w += da[u].w;
          b.x += db[u].x; b.y += db[u].y; b.z += db[u].z; b.w += db[u].w;
        }
      }
      if (proj.bias) {
        const float4 ba = load4(proj.bias + column + j0), bb = load4(proj.bias + column + HALF + j0);
        a.x += ba.x; a.y += ba.y; a.z += ba.z; a.w += ba.w;
        b.x += bb.x; b.y += bb.y; b.z += bb.z; b.w += bb.w;
      }
      float4 lo = a, hi = b;
      if (slot != NH * 8 + 1) {  // q and k are rotated, v is not
        const float4 cs = *reinterpret_cast<const float4*>(&sh_trig[j0]), sn = *reinterpret_cast<const float4*>(&sh_trig[HALF + j0]);
        lo = make_float4(a.x * cs.x - b.x * sn.x, a.y * cs.y - b.y * sn.y, a.z * cs.z - b.z * sn.z, a.w * cs.w - b.w * sn.w);
        hi = make_float4(b.x * cs.x + a.x * sn.x, b.y * cs.y + a.y * sn.y, b.z * cs.z + a.z * sn.z, b.w * cs.w + a.w * sn.w);
      }
      uint2 lo2, hi2;
      lo2.x = pack2(lo.x, lo.y); lo2.y = pack2(lo.z, lo.w);
      hi2.x = pack2(hi.x, hi.y); hi2.y = pack2(hi.z, hi.w);
      *reinterpret_cast<uint2*>(&sh_q[slot * QROW + j0]) = lo2;
      *reinterpret_cast<uint2*>(&sh_q[slot * QROW + HALF + j0]) = hi2;
      if (page_row) {
        *reinterpret_cast<uint2*>(page_row + j0) = lo2;
        *reinterpret_cast<uint2*>(page_row + HALF + j0) = hi2;
      }
    }
  }
#pragma unroll
  for (int u = 0; u < kStagedPerThread; ++u) sh_pages[threadIdx.x + u * kMmaDecodeWarps * 32] = staged[u];
  __syncthreads();
  staged_ready = true;
  const int last_group = groups - 1;
  const bool owner_warp = owns_new && groups > 0 && warp == last_group % kMmaDecodeWarps;
  if (FUSED) {
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
      const int hd = nh * 8 + g;
      const __nv_bfloat16* x = &sh_q[hd * QROW + 2 * c];
#pragma unroll
      for (int ks = 0; ks < MT; ++ks) {
        qb[nh][ks][0] = hd < heads_here ? *reinterpret_cast<const uint32_t*>(x + 16 * ks) : 0u;
        qb[nh][ks][1] = hd < heads_here ? *reinterpret_cast<const uint32_t*>(x + 16 * ks + 8) : 0u;
      }
    }
  }
  // ldmatrix addressing: lane = 8 * matrix + row of the matrix.
  const int lm_mat = lane >> 3, lm_row = lane & 7;
  int stage = 0;
  for (int grp = warp; grp < groups; grp += kMmaDecodeWarps) {
    const int base_key = lo16 + grp * 16;
    issue(grp + (STAGES - 1) * kMmaDecodeWarps, (stage + STAGES - 1) % STAGES);  // empty group past the end
    if (STAGES > 2) asm volatile("cp.async.wait_group 2;" ::: "memory");
    else asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncwarp();
    const uint32_t k_tile = my_ring + (uint32_t)stage * 2 * TILE_BYTES, v_tile = k_tile + TILE_BYTES;
    stage = (stage + 1) % STAGES;
    if (FUSED && owner_warp && grp == last_group) {
      // The copy brought whatever the page held in the token's own row: put the token's key and value there.
      const int r = pos - base_key;
#pragma unroll
      for (int i = 0; i < D / 64; ++i) {
        const int d = 2 * (lane + 32 * i);  // two dims to a lane and round
        const uint32_t offset = (uint32_t)(r * ROW_BYTES + (((d >> 3) ^ (r & 7)) << 4) + (d & 7) * 2);
        const uint32_t kk = *reinterpret_cast<const uint32_t*>(&sh_q[NH * 8 * QROW + d]);
        const uint32_t vv = *reinterpret_cast<const uint32_t*>(&sh_q[(NH * 8 + 1) * QROW + d]);
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(k_tile + offset), "r"(kk) : "memory");
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(v_tile + offset), "r"(vv) : "memory");
      }
      __syncwarp();
    }

    // ---- S^T = K Q^T: rows = keys g and g + 8 of the group, columns = heads 2c and 2c + 1 -------------
    float st[NH][4];
    {
      // Matrices of a k-step: (keys 0-7, chunk 2 ks), (keys 8-15, 2 ks), (keys 0-7, 2 ks + 1), (keys 8-15, 2 ks + 1).
      // Even and odd k-steps accumulate apart, which halves the chain of dependent MMAs.
      float half[NH][2][4];
#pragma unroll
      for (int nh = 0; nh < NH; ++nh)
#pragma unroll
        for (int r = 0; r < 4; ++r) half[nh][0][r] = half[nh][1][r] = 0.f;
      const int key = lm_row + 8 * (lm_mat & 1);
#pragma unroll
      for (int ks = 0; ks < MT; ++ks) {
        const int ch = 2 * ks + (lm_mat >> 1);
        uint32_t a[4];
        ldmatrix_x4(a, k_tile + (uint32_t)(key * ROW_BYTES + ((ch ^ (key & 7)) << 4)));
#pragma unroll
        for (int nh = 0; nh < NH; ++nh)
          mma_16816_bf16(half[nh][ks & 1], a[0], a[1], a[2], a[3], qb[nh][ks][0], qb[nh][ks][1]);
      }
#pragma unroll
      for (int nh = 0; nh < NH; ++nh)
#pragma unroll
        for (int r = 0; r < 4; ++r) st[nh][r] = half[nh][0][r] + half[nh][1][r];
    }

    // ---- mask (first and last group of a split), maxima and exponentials per head -------------------------
    const bool edge = base_key < lo || base_key + 15 > hi;
    const bool keep_lo = !edge || (base_key + g >= lo && base_key + g <= hi);
    const bool keep_hi = !edge || (base_key + g + 8 >= lo && base_key + g + 8 <= hi);
    uint32_t pb[NH][2];
    float corr[NH][2];
#pragma unroll
    for (int nh = 0; nh < NH; ++nh) {
      float x[4];
      x[0] = keep_lo ? st[nh][0] * scale_log2 : -INFINITY;
      x[1] = keep_lo ? st[nh][1] * scale_log2 : -INFINITY;
      x[2] = keep_hi ? st[nh][2] * scale_log2 : -INFINITY;
      x[3] = keep_hi ? st[nh][3] * scale_log2 : -INFINITY;
#pragma unroll
      for (int e = 0; e < 2; ++e) {  // column e of the lane: head 8 nh + 2c + e
        float m = fmaxf(x[e], x[e + 2]);
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
        const float m_new = fmaxf(col_max[nh][e], m);
        corr[nh][e] = m_new == -INFINITY ? 1.f : exp2f(col_max[nh][e] - m_new);
        col_max[nh][e] = m_new;
        const float shift = m_new == -INFINITY ? 0.f : m_new;
        x[e] = exp2f(x[e] - shift);
        x[e + 2] = exp2f(x[e + 2] - shift);
        col_sum[nh][e] = col_sum[nh][e] * corr[nh][e] + x[e] + x[e + 2];
      }
      // P^T as the B operand of the second product: keys become the reduction index.
      pb[nh][0] = movmatrix_trans(pack2(x[0], x[1]));
      pb[nh][1] = movmatrix_trans(pack2(x[2], x[3]));
    }

    // ---- O^T = O^T * corr + V^T P^T ------------------------------------------------------------------------
    {
      // Matrices of a row tile: (keys 0-7, chunk 2 mt), (keys 0-7, 2 mt + 1), (keys 8-15, 2 mt), (keys 8-15, 2 mt + 1),
      // each transposed on the way in.
      const int key = lm_row + 8 * (lm_mat >> 1);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int ch = 2 * mt + (lm_mat & 1);
        uint32_t a[4];
        ldmatrix_x4_trans(a, v_tile + (uint32_t)(key * ROW_BYTES + ((ch ^ (key & 7)) << 4)));
#pragma unroll
        for (int nh = 0; nh < NH; ++nh) {
          o[nh][mt][0] *= corr[nh][0]; o[nh][mt][1] *= corr[nh][1];
          o[nh][mt][2] *= corr[nh][0]; o[nh][mt][3] *= corr[nh][1];
          mma_16816_bf16(o[nh][mt], a[0], a[1], a[2], a[3], pb[nh][0], pb[nh][1]);
        }
      }
    }
  }

  // ---- merge the warps ---------------------------------------------------------------------------------
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();  // the ring is done with: its memory becomes the merge area
#pragma unroll
  for (int nh = 0; nh < NH; ++nh)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float l = col_sum[nh][e];  // add up the lanes that hold other keys of the same head
      l += __shfl_xor_sync(0xffffffffu, l, 4);
      l += __shfl_xor_sync(0xffffffffu, l, 8);
      l += __shfl_xor_sync(0xffffffffu, l, 16);
      const int hd = nh * 8 + 2 * c + e;
      if (g == 0) { sh_m[warp][hd] = col_max[nh][e]; sh_l[warp][hd] = l; }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        sh_o[warp][hd][16 * mt + g] = o[nh][mt][e];
        sh_o[warp][hd][16 * mt + g + 8] = o[nh][mt][e + 2];
      }
    }
  if (NH == 1 && lane < 8) { sh_m[warp][8 + lane] = -INFINITY; sh_l[warp][8 + lane] = 0.f; }
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
      // All loads from the other CTAs' shared memory are issued before the first is used: one trip through
      // the cluster's network instead of one per split.
      float ms[kMmaDecodeClusterSplits], ls[kMmaDecodeClusterSplits], os[kMmaDecodeClusterSplits];
#pragma unroll
      for (int s = 0; s < kMmaDecodeClusterSplits; ++s) {
        const bool there = s < num_splits;
        ms[s] = there ? cluster_load(&cl_m[hd], s) : -INFINITY;
        ls[s] = there ? cluster_load(&cl_l[hd], s) : 0.f;
        os[s] = there ? cluster_load(&cl_o[hd][e], s) : 0.f;
      }
      float m_all = -INFINITY;
#pragma unroll
      for (int s = 0; s < kMmaDecodeClusterSplits; ++s) m_all = fmaxf(m_all, ms[s]);
      float l_all = 0.f, acc = 0.f;
#pragma unroll
      for (int s = 0; s < kMmaDecodeClusterSplits; ++s) {
        const float weight = ms[s] == -INFINITY ? 0.f : exp2f(ms[s] - m_all);
        l_all += ls[s] * weight;
        acc += os[s] * weight;
      }
      out[(size_t)t * out_row_stride + (size_t)(head0 + hd) * D + e] = __float2bfloat16_rn(l_all > 0.f ? acc / l_all : 0.f);
    }
    cluster_barrier_exit();  // no CTA leaves while another may still read its shared memory
  }
}

// Combines the partial results of the splits of one (token, head): maxima are base-2 exponents.
// A row of head_dim floats takes head_dim / 4 threads (four floats each); the block's 256 threads
// hold 256 / (head_dim / 4) rows at a time, so that the loads of many splits are in flight together,
// and the rows meet in shared memory.  The order of the additions is fixed by the split count alone.
constexpr int kMergeThreads = 256;

__global__ void __launch_bounds__(kMergeThreads)
attention_decode_mma_merge_kernel(const float* __restrict__ scratch_o, const float* __restrict__ scratch_ml,
                                  __nv_bfloat16* __restrict__ out, int out_row_stride, int num_heads, int head_dim,
                                  int num_splits) {
  __shared__ float sh_max[kMergeThreads / 32];
  __shared__ float sh_l[kMergeThreads / 16];
  __shared__ float4 sh_acc[kMergeThreads];
  grid_dependency_release();
  grid_dependency_wait();
  const int t = blockIdx.x, head = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t row0 = ((size_t)t * num_heads + head) * num_splits;
  const int per_row = head_dim / 4;             // threads of one split's row (16 or 32)
  const int rows = kMergeThreads / per_row;     // splits in flight
  const int mine = threadIdx.x / per_row, piece = threadIdx.x % per_row;

  float m_all = -INFINITY;
  for (int s = threadIdx.x; s < num_splits; s += kMergeThreads) m_all = fmaxf(m_all, __ldcg(scratch_ml + (row0 + s) * 2));
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) m_all = fmaxf(m_all, __shfl_xor_sync(0xffffffffu, m_all, d));
  if (lane == 0) sh_max[warp] = m_all;
  __syncthreads();
#pragma unroll
  for (int w = 0; w < kMergeThreads / 32; ++w) m_all = fmaxf(m_all, sh_max[w]);

  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float l = 0.f;
#pragma unroll 4
  for (int s = mine; s < num_splits; s += rows) {
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(scratch_ml + (row0 + s) * 2));
    const float4 o = load4_cg(scratch_o + (row0 + s) * head_dim + piece * 4);
    const float weight = ml.x == -INFINITY ? 0.f : exp2f(ml.x - m_all);
    l += ml.y * weight;
    acc.x += o.x * weight; acc.y += o.y * weight; acc.z += o.z * weight; acc.w += o.w * weight;
  }
  sh_acc[threadIdx.x] = acc;
  if (piece == 0) sh_l[mine] = l;
  __syncthreads();
  if (threadIdx.x < per_row) {
    float l_all = 0.f;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < rows; ++r) {
      const float4 part = sh_acc[r * per_row + piece];
      sum.x += part.x; sum.y += part.y; sum.z += part.z; sum.w += part.w;
      l_all += sh_l[r];
    }
    const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
    __nv_bfloat162 lo = __floats2bfloat162_rn(sum.x * inv, sum.y * inv), hi = __floats2bfloat162_rn(sum.z * inv, sum.w * inv);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + (size_t)t * out_row_stride + (size_t)head * head_dim + piece * 4) = packed;
  }
}

}  // namespace distie

using namespace distie;

// Stages of the key/value ring (and with them the CTAs that fit an SM: 2 with three stages, 3 with two)
// for `tokens` single tokens, `blocks_per_token` CTAs per token and split, and `num_splits` splits.
// Three stages when the kernel amounts to about one CTA per SM, which then has to cover the latency of
// its copies alone; two otherwise (measured at batch 1 to 64 with 1,024-token contexts: a step at
// batch 16 or 24 is 11 % shorter with two, at batch 8 it is 2 % shorter with three).
extern "C" int distie_attention_decode_mma_stages(int tokens, int blocks_per_token, int num_splits, int sm_count) {
  const long long ctas = (long long)tokens * blocks_per_token * num_splits;
  return (2 * ctas > sm_count && ctas <= sm_count) ? 3 : 2;
}

// `proj` null: q is given, rotated, and the cache holds every key; else the kernel starts from the projection.
static int launch_decode_mma(const ProjectionInput* proj, const void* q, int q_row_stride, void* out, int out_row_stride,
                             float* scratch, const int* positions, const int* token_seq, const int* seq_seat,
                             const int* block_table, int table_width, const void* k_cache, const void* v_cache,
                             int tokens, int num_heads, int num_kv_heads, int head_dim, int page_size, int num_pages,
                             int window, float scale, int num_splits, int* error, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads != 0 || page_size < 1 || table_width < 1 ||
      num_splits < 1 || num_splits > 65535 || (num_splits > kMmaDecodeClusterSplits && scratch == nullptr) || (q_row_stride & 7) ||
      (out_row_stride & 3))
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
  // Two or three ring stages (see distie_attention_decode_mma_stages).
  static int sm_count = 0;
  if (sm_count == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sm_count < 1)
      sm_count = 148;
  }
  const int stages = distie_attention_decode_mma_stages(tokens, num_kv_heads * chunks, num_splits, sm_count);
  // Dynamic shared memory: the larger of the ring (warps x stages x loads x 512 bytes) and the merge areas.
  const size_t ring_bytes = (size_t)kMmaDecodeWarps * stages * 2 * 16 * head_dim * 2;  // K and V tiles of 16 rows
  const size_t merge_bytes = (size_t)kMmaDecodeWarps * 16 * (head_dim + 1) * sizeof(float) + 16 * head_dim * sizeof(float);
  const size_t shared = ring_bytes > merge_bytes ? ring_bytes : merge_bytes;
  const int column_tiles = group > 8 ? 2 : 1;  // (of a chunk of up to 16 heads)
  static bool configured = false;
  if (!configured) {
#define DISTIE_MMA_DECODE_SMEM(DV, SV, NV)                                                                        \
  if ((err = cudaFuncSetAttribute(attention_decode_mma_kernel<DV, SV, NV, true, false>,                             \
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024)) != cudaSuccess ||       \
      (err = cudaFuncSetAttribute(attention_decode_mma_kernel<DV, SV, NV, false, false>,                            \
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024)) != cudaSuccess ||       \
      (err = cudaFuncSetAttribute(attention_decode_mma_kernel<DV, SV, NV, true, true>,                              \
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024)) != cudaSuccess ||       \
      (err = cudaFuncSetAttribute(attention_decode_mma_kernel<DV, SV, NV, false, true>,                             \
                                  cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024)) != cudaSuccess)         \
    return (int)err
    DISTIE_MMA_DECODE_SMEM(64, 2, 1); DISTIE_MMA_DECODE_SMEM(64, 3, 1); DISTIE_MMA_DECODE_SMEM(128, 2, 1); DISTIE_MMA_DECODE_SMEM(128, 3, 1);
    DISTIE_MMA_DECODE_SMEM(64, 2, 2); DISTIE_MMA_DECODE_SMEM(64, 3, 2); DISTIE_MMA_DECODE_SMEM(128, 2, 2); DISTIE_MMA_DECODE_SMEM(128, 3, 2);
#undef DISTIE_MMA_DECODE_SMEM
    configured = true;
  }
  // Up to 8 splits (the portable cluster size) are merged inside the kernel, through the cluster's shared memory.
  const int cluster_merge = (num_splits > 1 && num_splits <= kMmaDecodeClusterSplits) ? 1 : 0;
  const dim3 cluster = cluster_merge ? dim3(1, 1, num_splits) : dim3(0, 0, 0);
  const ProjectionInput projection = proj ? *proj : ProjectionInput();
#define DISTIE_MMA_DECODE(DV, SV, NV)                                                                              \
  if (page_shift >= 4) { DISTIE_MMA_DECODE_FUSED(DV, SV, NV, true); }                                               \
  else { DISTIE_MMA_DECODE_FUSED(DV, SV, NV, false); }
#define DISTIE_MMA_DECODE_FUSED(DV, SV, NV, PV)                                                                    \
  if (proj) DISTIE_MMA_DECODE_PAGE(DV, SV, NV, PV, true);                                                           \
  else DISTIE_MMA_DECODE_PAGE(DV, SV, NV, PV, false)
#define DISTIE_MMA_DECODE_PAGE(DV, SV, NV, PV, FV)                                                                 \
  err = launch_dependent_cluster(8, cluster, attention_decode_mma_kernel<DV, SV, NV, PV, FV>, grid, dim3(kMmaDecodeWarps * 32), \
                         shared, stream, projection, (const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, out_row_stride, \
                         scratch_o, scratch_ml, positions, token_seq, seq_seat, block_table, table_width,          \
                         (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, num_heads, group, chunks,   \
                         num_kv_heads, page_size, page_shift, num_pages, window, scale_log2, cluster_merge, error)
#define DISTIE_MMA_DECODE_BY_STAGES(DV, NV)   \
  if (stages == 2) { DISTIE_MMA_DECODE(DV, 2, NV) } \
  else { DISTIE_MMA_DECODE(DV, 3, NV) }
  if (head_dim == 64) {
    if (column_tiles == 1) { DISTIE_MMA_DECODE_BY_STAGES(64, 1); } else { DISTIE_MMA_DECODE_BY_STAGES(64, 2); }
  } else {
    if (column_tiles == 1) { DISTIE_MMA_DECODE_BY_STAGES(128, 1); } else { DISTIE_MMA_DECODE_BY_STAGES(128, 2); }
  }
#undef DISTIE_MMA_DECODE_BY_STAGES
#undef DISTIE_MMA_DECODE_PAGE
#undef DISTIE_MMA_DECODE_FUSED
#undef DISTIE_MMA_DECODE
  if (err != cudaSuccess) return (int)err;
  if (num_splits > 1 && !cluster_merge) {
    const dim3 merge_grid(tokens, num_heads);
    err = launch_dependent_family(8, attention_decode_mma_merge_kernel, merge_grid, dim3(kMergeThreads), 0, stream,
                           (const float*)scratch_o, (const float*)scratch_ml, (__nv_bfloat16*)out, out_row_stride,
                           num_heads, head_dim, num_splits);
    if (err != cudaSuccess) return (int)err;
  }
  return 0;
}

// Same arguments and scratch layout as distie_attention_decode (bfloat16 only).
extern "C" int distie_attention_decode_mma(const void* q, int q_row_stride, void* out, int out_row_stride,
                                           float* scratch, const int* positions, const int* token_seq,
                                           const int* seq_seat, const int* block_table, int table_width,
                                           const void* k_cache, const void* v_cache, int tokens, int num_heads,
                                           int num_kv_heads, int head_dim, int page_size, int num_pages, int window,
                                           float scale, int num_splits, int* error, cudaStream_t stream) {
  return launch_decode_mma(nullptr, q, q_row_stride, out, out_row_stride, scratch, positions, token_seq, seq_seat,
                           block_table, table_width, k_cache, v_cache, tokens, num_heads, num_kv_heads, head_dim,
                           page_size, num_pages, window, scale, num_splits, error, stream);
}

// The same for a step of single tokens that starts from the q/k/v projection: `slices` [splits, tokens, row_stride]
// float32 (q heads, k heads, v heads), `bias` [row_stride] or null, `inv_freq` [head_dim / 2] or null (no rotation; the
// rotation is over the whole head, pairs (j, j + head_dim / 2)).  With `write_new` the token's key and value go into
// their cache page and are used; without it the cache must hold them already.
extern "C" int distie_attention_decode_mma_qkv(const float* slices, int splits, long long split_stride, int row_stride,
                                               const float* bias, const float* inv_freq, float trig_factor,
                                               int write_new, void* out, int out_row_stride, float* scratch,
                                               const int* positions, const int* token_seq, const int* seq_seat,
                                               const int* block_table, int table_width, void* k_cache, void* v_cache,
                                               int tokens, int num_heads, int num_kv_heads, int head_dim, int page_size,
                                               int num_pages, int window, float scale, int num_splits, int* error,
                                               cudaStream_t stream) {
  if (slices == nullptr || splits < 1 || row_stride < (num_heads + 2 * num_kv_heads) * head_dim) return DISTIE_ERR_ARG;
  if ((row_stride & 3) || (split_stride & 3) || ((uintptr_t)slices & 15) || ((uintptr_t)bias & 15)) return DISTIE_ERR_UNSUPPORTED;
  ProjectionInput proj;
  proj.slices = slices;
  proj.splits = splits;
  proj.split_stride = split_stride;
  proj.row_stride = row_stride;
  proj.bias = bias;
  proj.inv_freq = inv_freq;
  proj.trig_factor = trig_factor;
  proj.write_new = write_new;
  return launch_decode_mma(&proj, nullptr, 8, out, out_row_stride, scratch, positions, token_seq, seq_seat, block_table,
                           table_width, k_cache, v_cache, tokens, num_heads, num_kv_heads, head_dim, page_size,
                           num_pages, window, scale, num_splits, error, stream);
}
