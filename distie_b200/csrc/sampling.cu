// Token selection on the device: greedy argmax and temperature sampling.
//
// A row of float32 logits is shared out over a cluster of up to 8 CTAs of 1024 threads (a CTA can
// pull only so many bytes a microsecond, and a row of a large vocabulary is 600 KB); their partial
// results meet through distributed shared memory.  A row with temperature <= 0 takes the arg-max
// (ties: the lowest index, like an arg-max on the host).  Any other row draws from
// softmax(logits / temperature) by inverting the cumulative distribution, taken in index order, at
// the uniform number the host passes for that row: token = the first index whose cumulative
// probability exceeds u.  The host derives u from (seed, request, output index), so a request's
// stream of tokens does not depend on the batch it was sampled in.  Only the token ids (int32)
// leave the device.
#include "common.cuh"

namespace distie {

constexpr int kSampleThreads = 1024;
constexpr int kSampleWarps = kSampleThreads / 32;
constexpr int kSampleCluster = 8;

__device__ __forceinline__ void better(float& best, int& at, float v, int i) {
  if (v > best || (v == best && i < at)) { best = v; at = i; }
}

__device__ __forceinline__ int cluster_load_int(const int* local, uint32_t rank) {
  return __float_as_int(cluster_load(reinterpret_cast<const float*>(local), rank));
}

// gridDim.x = rows * ctas (ctas = CTAs per row = cluster size, 1 when launched without clusters).
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
              const float* __restrict__ temperatures, const float* __restrict__ uniforms,
              int* __restrict__ tokens, int ctas) {
  __shared__ float sh_val[kSampleWarps];
  __shared__ int sh_idx[kSampleWarps];
  __shared__ float sh_sum[kSampleWarps];
  __shared__ float cl_best, cl_total;  // this CTA's share, read by the others of the cluster
  __shared__ int cl_at, cl_pick;
  grid_dependency_release();
  const int row = blockIdx.x / ctas;
  const uint32_t rank = blockIdx.x % ctas;
  const float* z = logits + (size_t)row * row_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float temperature = temperatures ? temperatures[row] : 0.f;
  // This CTA's share of the vocabulary, a multiple of 4 entries long.
  const int span = (((vocab + ctas - 1) / ctas) + 3) & ~3;
  const int first = min(vocab, (int)rank * span), last = min(vocab, first + span);
  grid_dependency_wait();  // the logits come from the kernel before this one

  // Arg-max (also the softmax shift and the fallback pick): pieces of four where the row allows it.
  float best = -INFINITY;
  int at = 0x7fffffff;
  if (((row_stride | first) & 3) == 0 && ((uintptr_t)logits & 15) == 0) {
    const int pieces = (last - first) >> 2;
    for (int p = threadIdx.x; p < pieces; p += kSampleThreads) {
      const int i = first + 4 * p;
      const float4 v = load4_cg(z + i);
      better(best, at, v.x, i); better(best, at, v.y, i + 1); better(best, at, v.z, i + 2); better(best, at, v.w, i + 3);
    }
    for (int i = first + 4 * pieces + threadIdx.x; i < last; i += kSampleThreads) better(best, at, __ldcg(z + i), i);
  } else {
    for (int i = first + threadIdx.x; i < last; i += kSampleThreads) better(best, at, __ldcg(z + i), i);
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, offset);
    const int oi = __shfl_xor_sync(0xffffffffu, at, offset);
    better(best, at, ov, oi);
  }
  if (lane == 0) { sh_val[warp] = best; sh_idx[warp] = at; }
  __syncthreads();
  best = sh_val[0];
  at = sh_idx[0];
  for (int w = 1; w < kSampleWarps; ++w) better(best, at, sh_val[w], sh_idx[w]);
  if (ctas > 1) {
    if (threadIdx.x == 0) { cl_best = best; cl_at = at; cl_pick = -1; }
    cluster_barrier();
    best = -INFINITY;
    at = 0x7fffffff;
    // (all loads from the other CTAs are issued before the first is used: one trip, not one per CTA)
    float their_best[kSampleCluster];
    int their_at[kSampleCluster];
#pragma unroll
    for (int r = 0; r < kSampleCluster; ++r) {
      their_best[r] = r < ctas ? cluster_load(&cl_best, r) : -INFINITY;
      their_at[r] = r < ctas ? cluster_load_int(&cl_at, r) : 0x7fffffff;
    }
#pragma unroll
    for (int r = 0; r < kSampleCluster; ++r)
      if (r < ctas) better(best, at, their_best[r], their_at[r]);
  } else if (threadIdx.x == 0) {
    cl_pick = -1;
  }
  if (at == 0x7fffffff) at = 0;  // a row of NaNs: still a valid token id
  if (!(temperature > 0.f)) {
    if (threadIdx.x == 0 && rank == 0) tokens[row] = at;
    if (ctas > 1) cluster_barrier_exit();  // nobody leaves while its shared memory may still be read
    return;
  }

  // Each warp owns a contiguous chunk of the CTA's share, so that cumulative sums run in index
  // order; lanes stride inside the chunk for coalesced reads.
  const float inv_t = 1.f / temperature;
  const float shift = best * inv_t;
  const int chunk = (last - first + kSampleWarps - 1) / kSampleWarps;
  const int begin = min(last, first + warp * chunk);
  const int end = min(last, begin + chunk);
  float sum = 0.f;
  for (int i = begin + lane; i < end; i += 32) sum += expf(__ldcg(z + i) * inv_t - shift);
  sum = warp_sum(sum);
  if (lane == 0) sh_sum[warp] = sum;
  __syncthreads();
  float total = 0.f, before = 0.f;
  for (int w = 0; w < kSampleWarps; ++w) {
    if (w == warp) before = total;
    total += sh_sum[w];
  }
  if (ctas > 1) {
    if (threadIdx.x == 0) cl_total = total;
    cluster_barrier();
    float all = 0.f, ahead = 0.f;
    float their_total[kSampleCluster];
#pragma unroll
    for (int r = 0; r < kSampleCluster; ++r) their_total[r] = r < ctas ? cluster_load(&cl_total, r) : 0.f;
#pragma unroll
    for (int r = 0; r < kSampleCluster; ++r) {
      if ((uint32_t)r == rank) ahead = all;
      if (r < ctas) all += their_total[r];
    }
    before += ahead;
    total = all;
  }
  const float target = uniforms[row] * total;
  // The warp whose chunk holds the target walks it, 32 entries at a time.
  if (target >= before && target < before + sh_sum[warp]) {
    float running = before;
    for (int start = begin; start < end; start += 32) {
      const int i = start + lane;
      const float p = i < end ? expf(__ldcg(z + i) * inv_t - shift) : 0.f;
      float scan = p;
#pragma unroll
      for (int offset = 1; offset < 32; offset <<= 1) {
        const float other = __shfl_up_sync(0xffffffffu, scan, offset);
        if (lane >= offset) scan += other;
      }
      const unsigned hit = __ballot_sync(0xffffffffu, i < end && running + scan > target);
      if (hit) {
        if (lane == 0) cl_pick = start + __ffs(hit) - 1;
        break;
      }
      running += __shfl_sync(0xffffffffu, scan, 31);
    }
  }
  __syncthreads();
  if (ctas > 1) {
    cluster_barrier();
    if (rank == 0 && threadIdx.x == 0) {
      int pick = -1;  // the first CTA that found the target; rounding may have pushed it past every chunk
      for (uint32_t r = 0; r < (uint32_t)ctas && pick < 0; ++r) pick = cluster_load_int(&cl_pick, r);
      tokens[row] = pick >= 0 ? pick : at;
    }
    cluster_barrier_exit();
  } else if (threadIdx.x == 0) {
    tokens[row] = cl_pick >= 0 ? cl_pick : at;
  }
}

}  // namespace distie

using namespace distie;

extern "C" int distie_sample(const float* logits, long long row_stride, int rows, int vocab,
                             const float* temperatures, const float* uniforms, int* tokens, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab < 1 || row_stride < vocab) return DISTIE_ERR_ARG;
  // A cluster per row for large vocabularies and few rows; one CTA per row otherwise.
  const int ctas = (vocab >= 32768 && rows <= 64) ? kSampleCluster : 1;
  const dim3 cluster = ctas > 1 ? dim3(ctas, 1, 1) : dim3(0, 0, 0);
  const cudaError_t err = launch_dependent_cluster(0xff, cluster, sample_kernel, dim3(rows * ctas), dim3(kSampleThreads), 0,
                                                   stream, logits, row_stride, vocab, temperatures, uniforms, tokens, ctas);
  return err == cudaSuccess ? 0 : (int)err;
}
