// Products of a few rows with a large weight matrix (decoding): y[M, N] = x[M, K] W[N, K]^T.
//
// With M <= 16 every weight is used for at most 16 multiply-adds, so the product
// is bound by streaming W from HBM once.  The kernel is organised around that
// stream: each lane reads 16-byte pieces of weight rows straight from global
// memory into registers (no shared-memory staging, no reuse to exploit), many
// loads in flight, and feeds them to the tensor cores with the weights as the
// 16-row operand and the few rows of x as the 8-column operand
// (mma.sync.m16n8k16, bfloat16 in, float32 accumulate).
//
//   grid  = one CTA per 16 weight rows (per 8 gate rows + 8 up rows when fused with SwiGLU)
//   block = 8 warps; warp w takes the K blocks w, w + 8, ... (32 elements each), so that
//           neighbouring warps read neighbouring 64-byte pieces of the same rows
//   tail  = cross-warp sum through shared memory, then the epilogue in registers:
//           bias, cast to bfloat16 or float32, or silu(gate) * up
//   split = matrices with few rows (hidden x hidden, hidden x intermediate) would leave most SMs
//           idle and make each CTA walk K in many dependent round trips, so K is also split
//           over gridDim.y CTAs per row tile.  Each writes its float32 partial sums to a
//           workspace; the CTA that arrives last (a counter per tile) adds them up in a
//           fixed order and runs the epilogue, then resets the counter for the next launch.
//
// The order of the 16 k-values inside one mma does not matter as long as both
// operands use the same order; a lane therefore loads 8 consecutive elements
// (one 16-byte load) and uses them as its share of two mma steps.
#include "common.cuh"

namespace distie {

constexpr int kSkinnyWarps = 8;
constexpr int kSkinnyUnroll = 6;
constexpr int EPI_STORE = 0;
constexpr int EPI_SWIGLU = 1;
constexpr int EPI_PARTIAL = 2;  // every split stores its own float32 sums; a later kernel adds them up

__device__ __forceinline__ uint4 load_stream(const void* p) {  // read once: keep it out of L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// The few rows of x were written by the kernel before this one, which may still have been running
// when this kernel started: an ordinary coherent load (cached in L1, where the CTAs of an SM share
// it), never the non-coherent path, which returned stale rows in that situation.
__device__ __forceinline__ uint4 load_cached(const void* p) {
  uint4 v;
  asm volatile("ld.global.ca.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT, int EPI, typename OutT>
__global__ void __launch_bounds__(kSkinnyWarps * 32, 2)
skinny_gemm_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ w,
                   const float* __restrict__ bias, OutT* __restrict__ out, int ldo, int M, int N, int K, int inter,
                   float* __restrict__ partials, int* __restrict__ counters) {
  __shared__ float red[kSkinnyWarps][NT][4][32];
  __shared__ int ticket;
  grid_dependency_release();  // the next kernel may start its own weight loads
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int tile = blockIdx.x;
  int row_a, row_b, limit_a, limit_b;
  if (EPI == EPI_SWIGLU) {
    row_a = tile * 8 + g;   // gate row
    row_b = inter + row_a;  // up row
    limit_a = inter;
    limit_b = 2 * inter;
  } else {
    row_a = tile * 16 + g;
    row_b = row_a + 8;
    limit_a = limit_b = N;
  }
  const bool ok_a = row_a < limit_a, ok_b = row_b < limit_b && (EPI != EPI_SWIGLU || ok_a);
  const __nv_bfloat16* wa = w + (size_t)(ok_a ? row_a : 0) * K;
  const __nv_bfloat16* wb = w + (size_t)(ok_b ? row_b : 0) * K;
  const __nv_bfloat16* xr[NT];
  bool ok_x[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    ok_x[nt] = nt * 8 + g < M;
    xr[nt] = x + (size_t)(ok_x[nt] ? nt * 8 + g : 0) * ldx;
  }

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int r = 0; r < 4; ++r) acc[nt][r] = 0.f;

  const int splits = gridDim.y, split = blockIdx.y;
  const int k_blocks_all = (K + 31) >> 5;
  const int per_split = (k_blocks_all + splits - 1) / splits;
  const int k_blocks = min(k_blocks_all, (split + 1) * per_split);
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  // The weights are written by no kernel: their first loads are issued before the wait for the
  // kernel that produces x, so that they fly while that kernel is still running.
  bool waited = false;
  for (int kb0 = split * per_split + warp; kb0 < k_blocks; kb0 += kSkinnyWarps * kSkinnyUnroll) {
    uint4 a0[kSkinnyUnroll], a1[kSkinnyUnroll], xv[NT][kSkinnyUnroll];
#pragma unroll
    for (int u = 0; u < kSkinnyUnroll; ++u) {
      const int kb = kb0 + u * kSkinnyWarps;
      const int k0 = kb * 32 + c * 8;
      const bool in_k = kb < k_blocks && k0 + 8 <= K;  // K is a multiple of 8
      a0[u] = (in_k && ok_a) ? load_stream(wa + k0) : zero;
      a1[u] = (in_k && ok_b) ? load_stream(wb + k0) : zero;
    }
    if (!waited) {
      grid_dependency_wait();
      waited = true;
    }
#pragma unroll
    for (int u = 0; u < kSkinnyUnroll; ++u) {
      const int kb = kb0 + u * kSkinnyWarps;
      const int k0 = kb * 32 + c * 8;
      const bool in_k = kb < k_blocks && k0 + 8 <= K;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
        xv[nt][u] = (in_k && ok_x[nt]) ? load_cached(xr[nt] + k0) : zero;
    }
#pragma unroll
    for (int u = 0; u < kSkinnyUnroll; ++u) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        mma_bf16_16816(acc[nt], a0[u].x, a1[u].x, a0[u].y, a1[u].y, xv[nt][u].x, xv[nt][u].y);
        mma_bf16_16816(acc[nt], a0[u].z, a1[u].z, a0[u].w, a1[u].w, xv[nt][u].z, xv[nt][u].w);
      }
    }
  }

  if (!waited) grid_dependency_wait();  // nothing is written before the earlier kernels are done
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int r = 0; r < 4; ++r) red[warp][nt][r][lane] = acc[nt][r];
  __syncthreads();

  // acc[nt][0..1]: (row_a, m = nt*8 + 2c, +1); acc[nt][2..3]: (row_b, same m).
  // Thread idx < NT * 64 owns the two sums (row_a, row_b) of one (nt, pair, lane).
  const int idx = threadIdx.x;
  const bool owner = idx < NT * 64;
  const int nt = idx >> 6, pair = (idx >> 5) & 1, l = idx & 31;
  float sum_a = 0.f, sum_b = 0.f;
  if (owner) {
#pragma unroll
    for (int wi = 0; wi < kSkinnyWarps; ++wi) {
      sum_a += red[wi][nt][pair][l];
      sum_b += red[wi][nt][pair + 2][l];
    }
  }
  if (EPI == EPI_PARTIAL) {
    // out is [splits, M, N] float32 (ldo = N); no bias, no fix-up: the consumer sums the slices.
    if (!owner) return;
    const int lg = l >> 2, lc = l & 3;
    const int m = nt * 8 + 2 * lc + pair;
    if (m >= M) return;
    OutT* slice = out + (size_t)split * M * ldo;
    const int ra = tile * 16 + lg, rb = ra + 8;
    if (ra < N) slice[(size_t)m * ldo + ra] = from_float<OutT>(sum_a);
    if (rb < N) slice[(size_t)m * ldo + rb] = from_float<OutT>(sum_b);
    return;
  }
  if (splits > 1) {
    float* mine = partials + ((size_t)tile * splits + split) * (NT * 128);
    if (owner) {
      mine[idx] = sum_a;
      mine[NT * 64 + idx] = sum_b;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) ticket = atomicAdd(&counters[tile], 1);
    __syncthreads();
    if (ticket != splits - 1) return;  // another CTA of this tile finishes the job
    __threadfence();
    if (owner) {
      sum_a = 0.f;
      sum_b = 0.f;
      const float* all = partials + (size_t)tile * splits * (NT * 128);
      for (int sp = 0; sp < splits; ++sp) {  // fixed order: the result does not depend on who came last
        sum_a += __ldcg(all + sp * (NT * 128) + idx);
        sum_b += __ldcg(all + sp * (NT * 128) + NT * 64 + idx);
      }
    }
    if (threadIdx.x == 0) counters[tile] = 0;
  }
  if (!owner) return;
  const int lg = l >> 2, lc = l & 3;
  const int m = nt * 8 + 2 * lc + pair;
  if (m >= M) return;
  if (EPI == EPI_SWIGLU) {
    const int ra = tile * 8 + lg;
    if (ra < inter) out[(size_t)m * ldo + ra] = from_float<OutT>(sum_a / (1.f + __expf(-sum_a)) * sum_b);
  } else {
    const int ra = tile * 16 + lg, rb = ra + 8;
    if (ra < N) out[(size_t)m * ldo + ra] = from_float<OutT>(sum_a + (bias ? bias[ra] : 0.f));
    if (rb < N) out[(size_t)m * ldo + rb] = from_float<OutT>(sum_b + (bias ? bias[rb] : 0.f));
  }
}

// Splits of K for a product with `tiles` row tiles: about two CTAs per SM, at least one K block per warp.
static int plan_splits(int tiles, int K, int sm_count) {
  const int k_blocks = (K + 31) / 32;
  int splits = (2 * sm_count + tiles - 1) / tiles;
  splits = min(splits, k_blocks / kSkinnyWarps);
  return max(1, min(splits, 16));
}

template <int NT>
int launch_skinny(const void* x, int ldx, const void* w, const float* bias, void* out, int ldo, int M, int N, int K,
                  int out_dtype, int swiglu, float* workspace, long long workspace_floats, int sm_count,
                  cudaStream_t stream) {
  const auto* xp = (const __nv_bfloat16*)x;
  const auto* wp = (const __nv_bfloat16*)w;
  const int threads = kSkinnyWarps * 32;
  const int inter = N / 2;
  const int tiles = swiglu ? (inter + 7) / 8 : (N + 15) / 16;
  // Split K until about two CTAs per SM are busy, keeping at least one K block per warp and split.
  int splits = plan_splits(tiles, K, sm_count);
  // Workspace: one counter per tile (ints, zero between launches), then the partial sums.
  int* counters = (int*)workspace;
  float* partials = workspace + tiles;
  if (splits > 1 && (workspace == nullptr || (long long)tiles + (long long)tiles * splits * NT * 128 > workspace_floats))
    splits = 1;
  const dim3 grid(tiles, splits);
  cudaError_t err;
  if (swiglu) {
    err = launch_dependent_family(1, skinny_gemm_kernel<NT, EPI_SWIGLU, __nv_bfloat16>, grid, dim3(threads), 0, stream, xp, ldx,
                           wp, (const float*)nullptr, (__nv_bfloat16*)out, ldo, M, N, K, inter, partials, counters);
  } else if (out_dtype == DISTIE_F32) {
    err = launch_dependent_family(1, skinny_gemm_kernel<NT, EPI_STORE, float>, grid, dim3(threads), 0, stream, xp, ldx, wp, bias,
                           (float*)out, ldo, M, N, K, 0, partials, counters);
  } else {
    err = launch_dependent_family(1, skinny_gemm_kernel<NT, EPI_STORE, __nv_bfloat16>, grid, dim3(threads), 0, stream, xp, ldx,
                           wp, bias, (__nv_bfloat16*)out, ldo, M, N, K, 0, partials, counters);
  }
  return err == cudaSuccess ? 0 : (int)err;
}

}  // namespace distie

using namespace distie;

// The most rows of x the kernel takes.
extern "C" int distie_linear_skinny_max_rows(void) { return 16; }

// out[M, N] (bfloat16 or float32, row stride ldo) = x[M, K] (bfloat16, row stride ldx) W[N, K]^T (+ bias[N]).
// With swiglu != 0, W is [2 * inter, K] (gate rows, then up rows) and out[M, inter] = silu(x Wg^T) * (x Wu^T).
// `workspace` (workspace_floats floats, zeroed once by the caller, shared by launches on one stream) lets the
// kernel split K over several CTAs; without it every row tile is one CTA.
extern "C" int distie_linear_skinny(const void* x, int ldx, const void* w, const float* bias, void* out, int ldo,
                                    int M, int N, int K, int out_dtype, int swiglu, float* workspace,
                                    long long workspace_floats, int sm_count, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (N < 1 || K < 8 || (K & 7) || (ldx & 7) || M > 16 || (swiglu && (N & 1))) return DISTIE_ERR_UNSUPPORTED;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return DISTIE_ERR_UNSUPPORTED;
  if (out_dtype != DISTIE_F32 && out_dtype != DISTIE_BF16) return DISTIE_ERR_UNSUPPORTED;
  if (sm_count < 1) sm_count = 148;
  if (M <= 8)
    return launch_skinny<1>(x, ldx, w, bias, out, ldo, M, N, K, out_dtype, swiglu, workspace, workspace_floats,
                            sm_count, stream);
  return launch_skinny<2>(x, ldx, w, bias, out, ldo, M, N, K, out_dtype, swiglu, workspace, workspace_floats,
                          sm_count, stream);
}

// Number of float32 slices distie_linear_skinny_partial writes for these sizes.
extern "C" int distie_linear_skinny_splits(int M, int N, int K, int sm_count) {
  (void)M;
  return plan_splits((N + 15) / 16, K, sm_count < 1 ? 148 : sm_count);
}

// out[s, M, N] (float32, contiguous) for s < distie_linear_skinny_splits(...): slice s holds the part of
// x W^T that comes from its share of K; their sum is the product.  No bias.
extern "C" int distie_linear_skinny_partial(const void* x, int ldx, const void* w, float* out, int M, int N, int K,
                                            int sm_count, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (N < 1 || K < 8 || (K & 7) || (ldx & 7) || M > 16) return DISTIE_ERR_UNSUPPORTED;
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return DISTIE_ERR_UNSUPPORTED;
  if (sm_count < 1) sm_count = 148;
  const int tiles = (N + 15) / 16;
  const dim3 grid(tiles, plan_splits(tiles, K, sm_count));
  const int threads = kSkinnyWarps * 32;
  cudaError_t err;
  if (M <= 8)
    err = launch_dependent_family(1, skinny_gemm_kernel<1, EPI_PARTIAL, float>, grid, dim3(threads), 0, stream,
                           (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, (const float*)nullptr, out, N, M, N,
                           K, 0, (float*)nullptr, (int*)nullptr);
  else
    err = launch_dependent_family(1, skinny_gemm_kernel<2, EPI_PARTIAL, float>, grid, dim3(threads), 0, stream,
                           (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, (const float*)nullptr, out, N, M, N,
                           K, 0, (float*)nullptr, (int*)nullptr);
  return err == cudaSuccess ? 0 : (int)err;
}
