// Token selection on the device: greedy argmax and temperature sampling.
//
// One block of 1024 threads per row of float32 logits.  A row with temperature
// <= 0 takes the arg-max (ties: the lowest index, like an arg-max on the host).
// Any other row draws from softmax(logits / temperature) by inverting the
// cumulative distribution, taken in index order, at the uniform number the host
// passes for that row: token = the first index whose cumulative probability
// exceeds u.  The host derives u from (seed, request, output index), so a
// request's stream of tokens does not depend on the batch it was sampled in.
// Only the token ids (int32) leave the device.
#include "common.cuh"

namespace distie {

constexpr int kSampleThreads = 1024;
constexpr int kSampleWarps = kSampleThreads / 32;

__device__ __forceinline__ void better(float& best, int& at, float v, int i) {
  if (v > best || (v == best && i < at)) { best = v; at = i; }
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
              const float* __restrict__ temperatures, const float* __restrict__ uniforms,
              int* __restrict__ tokens) {
  __shared__ float sh_val[kSampleWarps];
  __shared__ int sh_idx[kSampleWarps];
  __shared__ float sh_sum[kSampleWarps];
  __shared__ int sh_pick;
  const int row = blockIdx.x;
  const float* z = logits + (size_t)row * row_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float temperature = temperatures ? temperatures[row] : 0.f;

  // Arg-max (also the softmax shift and the fallback pick).
  float best = -INFINITY;
  int at = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += kSampleThreads) better(best, at, z[i], i);
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
  if (at == 0x7fffffff) at = 0;  // a row of NaNs: still a valid token id
  if (!(temperature > 0.f)) {
    if (threadIdx.x == 0) tokens[row] = at;
    return;
  }

  // Each warp owns a contiguous chunk of the vocabulary, so that cumulative sums
  // run in index order; lanes stride inside the chunk for coalesced reads.
  const float inv_t = 1.f / temperature;
  const float shift = best * inv_t;
  const int chunk = (vocab + kSampleWarps - 1) / kSampleWarps;
  const int begin = warp * chunk;
  const int end = min(vocab, begin + chunk);
  float sum = 0.f;
  for (int i = begin + lane; i < end; i += 32) sum += expf(z[i] * inv_t - shift);
  sum = warp_sum(sum);
  if (threadIdx.x == 0) sh_pick = -1;
  if (lane == 0) sh_sum[warp] = sum;
  __syncthreads();
  float total = 0.f, before = 0.f;
  for (int w = 0; w < kSampleWarps; ++w) {
    if (w == warp) before = total;
    total += sh_sum[w];
  }
  const float target = uniforms[row] * total;
  // The warp whose chunk holds the target walks it, 32 entries at a time.
  if (target >= before && target < before + sh_sum[warp]) {
    float running = before;
    for (int start = begin; start < end; start += 32) {
      const int i = start + lane;
      const float p = i < end ? expf(z[i] * inv_t - shift) : 0.f;
      float scan = p;
#pragma unroll
      for (int offset = 1; offset < 32; offset <<= 1) {
        const float other = __shfl_up_sync(0xffffffffu, scan, offset);
        if (lane >= offset) scan += other;
      }
      const unsigned hit = __ballot_sync(0xffffffffu, i < end && running + scan > target);
      if (hit) {
        if (lane == 0) sh_pick = start + __ffs(hit) - 1;
        break;
      }
      running += __shfl_sync(0xffffffffu, scan, 31);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) tokens[row] = sh_pick >= 0 ? sh_pick : at;  // rounding pushed the target past the end
}

}  // namespace distie

using namespace distie;

extern "C" int distie_sample(const float* logits, long long row_stride, int rows, int vocab,
                             const float* temperatures, const float* uniforms, int* tokens, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab < 1 || row_stride < vocab) return DISTIE_ERR_ARG;
  sample_kernel<<<rows, kSampleThreads, 0, stream>>>(logits, row_stride, vocab, temperatures, uniforms, tokens);
  DISTIE_LAUNCH_CHECK();
  return 0;
}
