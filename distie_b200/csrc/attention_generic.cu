// Attention over the paged cache for any batch of tokens: the size-agnostic kernel.
//
// One block per (token, query head).  The token at position `pos` of its request
// sees the keys `max(0, pos - window + 1) .. pos` of that request (window <= 0:
// all of them), which by then are all in the cache: earlier steps stored the older
// ones and this step's write kernel ran before.  Nothing but the token's position,
// its request's seat and the block table decides what is read, so the result does
// not depend on how a prompt was cut into steps or on what else is in the batch.
//
// Arithmetic is float32 throughout (scores, online softmax, the mix); T only
// selects the storage type.  Any even head_dim up to 256, any head counts, any
// page size.  This is the float32 engine's attention and the fallback of the
// bfloat16 engine for head sizes its faster kernels do not take.
#include "common.cuh"

namespace distie {

constexpr int kGenericWarps = 4;
constexpr int kMaxHeadDim = 256;

template <typename T>
__global__ void __launch_bounds__(kGenericWarps * 32)
attention_generic_kernel(const T* __restrict__ q, int q_row_stride, T* __restrict__ out, int out_row_stride,
                         const int* __restrict__ positions, const int* __restrict__ token_seq,
                         const int* __restrict__ seq_seat, const int* __restrict__ block_table, int table_width,
                         const T* __restrict__ k_cache, const T* __restrict__ v_cache, int group_size,
                         int num_kv_heads, int head_dim, int page_size, int num_pages, int window, float scale,
                         int* __restrict__ error) {
  __shared__ float sh_m[kGenericWarps], sh_l[kGenericWarps];
  __shared__ float sh_acc[kGenericWarps][kMaxHeadDim];
  const int t = blockIdx.x, head = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int kv_head = head / group_size;
  const int pos = positions[t];
  const int seat = seq_seat[token_seq[t]];
  const int* table = block_table + (size_t)seat * table_width;
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  constexpr int R = kMaxHeadDim / 32;

  float qv[R], acc[R];
  const T* q_row = q + (size_t)t * q_row_stride + (size_t)head * head_dim;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int e = lane + 32 * i;
    qv[i] = e < head_dim ? to_float(q_row[e]) : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  for (int key = first + warp; key <= pos; key += kGenericWarps) {
    const int column = key / page_size;
    const int page = column < table_width ? table[column] : -1;
    if (page < 0 || page >= num_pages) {  // a table that does not cover the keys: report, skip
      if (lane == 0 && error) atomicExch(error, 3);
      continue;
    }
    const size_t base = (((size_t)page * num_kv_heads + kv_head) * page_size + key % page_size) * head_dim;
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int e = lane + 32 * i;
      if (e < head_dim) dot += qv[i] * to_float(k_cache[base + e]);
    }
    const float s = warp_sum(dot) * scale;  // scaled after the product, as the reference does
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);
    const float p = expf(s - m_new);
    l = l * corr + p;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int e = lane + 32 * i;
      if (e < head_dim) acc[i] = acc[i] * corr + p * to_float(v_cache[base + e]);
    }
    m = m_new;
  }
  if (lane == 0) { sh_m[warp] = m; sh_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int e = lane + 32 * i;
    if (e < head_dim) sh_acc[warp][e] = acc[i];
  }
  __syncthreads();
  float m_all = -INFINITY;
#pragma unroll
  for (int w = 0; w < kGenericWarps; ++w) m_all = fmaxf(m_all, sh_m[w]);
  float l_all = 0.f;
  float weight[kGenericWarps];
#pragma unroll
  for (int w = 0; w < kGenericWarps; ++w) {
    weight[w] = sh_m[w] == -INFINITY ? 0.f : expf(sh_m[w] - m_all);
    l_all += sh_l[w] * weight[w];
  }
  const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
  T* out_row = out + (size_t)t * out_row_stride + (size_t)head * head_dim;
  for (int e = threadIdx.x; e < head_dim; e += blockDim.x) {
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kGenericWarps; ++w) total += sh_acc[w][e] * weight[w];
    out_row[e] = from_float<T>(total * inv);
  }
}

}  // namespace distie

using namespace distie;

extern "C" int distie_attention_generic(const void* q, int q_row_stride, void* out, int out_row_stride,
                                        const int* positions, const int* token_seq, const int* seq_seat,
                                        const int* block_table, int table_width, const void* k_cache,
                                        const void* v_cache, int tokens, int num_heads, int num_kv_heads,
                                        int head_dim, int page_size, int num_pages, int window, float scale,
                                        int dtype, int* error, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads != 0 || head_dim < 1 ||
      head_dim > kMaxHeadDim || page_size < 1 || table_width < 1 || num_heads > 65535)
    return DISTIE_ERR_ARG;
  const dim3 grid(tokens, num_heads);
  const int threads = kGenericWarps * 32;
  const int group = num_heads / num_kv_heads;
  if (dtype == DISTIE_BF16)
    attention_generic_kernel<<<grid, threads, 0, stream>>>(
        (const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, out_row_stride, positions, token_seq, seq_seat,
        block_table, table_width, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, group, num_kv_heads,
        head_dim, page_size, num_pages, window, scale, error);
  else if (dtype == DISTIE_F32)
    attention_generic_kernel<<<grid, threads, 0, stream>>>(
        (const float*)q, q_row_stride, (float*)out, out_row_stride, positions, token_seq, seq_seat, block_table,
        table_width, (const float*)k_cache, (const float*)v_cache, group, num_kv_heads, head_dim, page_size,
        num_pages, window, scale, error);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}
