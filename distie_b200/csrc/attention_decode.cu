// Split-KV attention for single tokens (decoding) over block tables.
//
// Decoding reads every cached key and value of a request once per step, so the
// kernel is bound by memory traffic; it is organised around 16-byte (bfloat16) or
// 32-byte (float) loads of cache rows and keeps everything else in registers.
//
//   grid  = (tokens, kv_heads * head_chunks, splits)
//   block = 128 threads.  A cache row of head_dim elements is read by DL =
//           head_dim / 8 neighbouring lanes (8 elements each), so a warp reads
//           32 / DL rows per load and the block 4 * 32 / DL.  The GC query heads
//           of the chunk that share this kv head reuse each loaded row.
//
// Each split covers a page-aligned part of the keys `first .. pos` of its token and
// writes an un-normalised partial result (float32: max, sum, mix) to `scratch`;
// `attention_decode_merge_kernel` combines the splits.  With one split the first
// kernel writes the final result itself and the scratch is not touched.
//
//   scratch_o  [tokens, heads, splits, head_dim]   float32
//   scratch_ml [tokens, heads, splits, 2]          float32 (max, sum)
//
// The key range of a token depends only on its position and the window, so the
// result is the same whatever else the batch holds.  head_dim must be 16, 32, 64,
// 128 or 256 here; the launcher refuses other sizes and the caller then uses the
// size-agnostic kernel.
#include "common.cuh"

namespace distie {

constexpr int kDecodeThreads = 128;
constexpr int kDecodeUnroll = 4;

// The float32 engine uses the accurate exponential; bfloat16 serving the fast one.
template <typename T>
__device__ __forceinline__ float softmax_exp(float x);
template <>
__device__ __forceinline__ float softmax_exp<float>(float x) { return expf(x); }
template <>
__device__ __forceinline__ float softmax_exp<__nv_bfloat16>(float x) { return __expf(x); }

template <typename T, int DL, int GC>
__global__ void __launch_bounds__(kDecodeThreads)
attention_decode_kernel(const T* __restrict__ q, int q_row_stride, T* __restrict__ out, int out_row_stride,
                        float* __restrict__ scratch_o, float* __restrict__ scratch_ml,
                        const int* __restrict__ positions, const int* __restrict__ token_seq,
                        const int* __restrict__ seq_seat, const int* __restrict__ block_table, int table_width,
                        const T* __restrict__ k_cache, const T* __restrict__ v_cache, int num_heads, int group_size,
                        int head_chunks, int num_kv_heads, int page_size, int num_pages, int window, float scale,
                        int* __restrict__ error) {
  constexpr int HEAD_DIM = DL * 8;
  constexpr int ROWS_PER_WARP = 32 / DL;
  constexpr int GROUPS = (kDecodeThreads / 32) * ROWS_PER_WARP;  // independent row streams in the block
  __shared__ float sh_m[GROUPS][GC], sh_l[GROUPS][GC];
  __shared__ float sh_acc[GROUPS][GC][HEAD_DIM];

  const int t = blockIdx.x;
  const int kv_head = blockIdx.y / head_chunks;
  const int chunk = blockIdx.y % head_chunks;
  const int split = blockIdx.z, num_splits = gridDim.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % DL;               // which 8 elements of the row
  const int group = warp * ROWS_PER_WARP + lane / DL;
  const int head0 = kv_head * group_size + chunk * GC;  // first query head of this block
  const int heads_here = min(GC, group_size - chunk * GC);

  const int pos = positions[t];
  const int seat = seq_seat[token_seq[t]];
  const int* table = block_table + (size_t)seat * table_width;
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  // Page-aligned share of [first, pos] for this split.
  const int first_page = first / page_size;
  const int pages = pos / page_size - first_page + 1;
  const int pages_per_split = (pages + num_splits - 1) / num_splits;
  const int lo = max(first, (first_page + split * pages_per_split) * page_size);
  const int hi = min(pos, (first_page + (split + 1) * pages_per_split) * page_size - 1);

  float qv[GC][8], acc[GC][8], m[GC], l[GC];
#pragma unroll
  for (int g = 0; g < GC; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
    if (g < heads_here) {
      load8(q + (size_t)t * q_row_stride + (size_t)(head0 + g) * HEAD_DIM + sub * 8, qv[g]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) qv[g][i] = 0.f;
    }
  }

  // The trip count is the same for every thread of the block: the shuffles below need whole warps.
  const int iterations = hi >= lo ? (hi - lo + GROUPS * kDecodeUnroll) / (GROUPS * kDecodeUnroll) : 0;
  for (int it = 0; it < iterations; ++it) {
    const int base_key = lo + (it * GROUPS + group) * kDecodeUnroll;
    float kf[kDecodeUnroll][8], vf[kDecodeUnroll][8];
    bool live[kDecodeUnroll];
#pragma unroll
    for (int u = 0; u < kDecodeUnroll; ++u) {
      const int key = base_key + u;
      live[u] = key <= hi;
      int page = 0;
      if (live[u]) {  // a position past the end of the table is reported like a page that is missing
        const int column = key / page_size;
        page = column < table_width ? table[column] : -1;
      }
      if (page < 0 || page >= num_pages) {
        if (error) atomicExch(error, 4);
        live[u] = false;
        page = 0;
      }
      if (live[u]) {
        const size_t at = (((size_t)page * num_kv_heads + kv_head) * page_size + key % page_size) * HEAD_DIM + sub * 8;
        load8(k_cache + at, kf[u]);
        load8(v_cache + at, vf[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < kDecodeUnroll; ++u) {
      // `live` is uniform over the DL lanes of a row, so the shuffles below stay converged per row.
      float s[GC];
#pragma unroll
      for (int g = 0; g < GC; ++g) {
        float dot = 0.f;
        if (live[u]) {
#pragma unroll
          for (int i = 0; i < 8; ++i) dot += qv[g][i] * kf[u][i];
        }
#pragma unroll
        for (int offset = DL / 2; offset > 0; offset >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, offset);
        s[g] = dot * scale;
      }
      if (live[u]) {
#pragma unroll
        for (int g = 0; g < GC; ++g) {
          const float m_new = fmaxf(m[g], s[g]);
          const float corr = softmax_exp<T>(m[g] - m_new);
          const float p = softmax_exp<T>(s[g] - m_new);
          l[g] = l[g] * corr + p;
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[g][i] = acc[g][i] * corr + p * vf[u][i];
          m[g] = m_new;
        }
      }
    }
  }

#pragma unroll
  for (int g = 0; g < GC; ++g) {
    if (sub == 0) { sh_m[group][g] = m[g]; sh_l[group][g] = l[g]; }
#pragma unroll
    for (int i = 0; i < 8; ++i) sh_acc[group][g][sub * 8 + i] = acc[g][i];
  }
  __syncthreads();

  for (int idx = threadIdx.x; idx < heads_here * HEAD_DIM; idx += kDecodeThreads) {
    const int g = idx / HEAD_DIM, e = idx % HEAD_DIM;
    float m_all = -INFINITY;
#pragma unroll
    for (int r = 0; r < GROUPS; ++r) m_all = fmaxf(m_all, sh_m[r][g]);
    float l_all = 0.f, o = 0.f;
#pragma unroll
    for (int r = 0; r < GROUPS; ++r) {
      const float w = sh_m[r][g] == -INFINITY ? 0.f : softmax_exp<T>(sh_m[r][g] - m_all);
      l_all += sh_l[r][g] * w;
      o += sh_acc[r][g][e] * w;
    }
    const int head = head0 + g;
    if (num_splits == 1) {
      out[(size_t)t * out_row_stride + (size_t)head * HEAD_DIM + e] = from_float<T>(l_all > 0.f ? o / l_all : 0.f);
    } else {
      const size_t row = ((size_t)t * num_heads + head) * num_splits + split;
      scratch_o[row * HEAD_DIM + e] = o;
      if (e == 0) {
        scratch_ml[row * 2] = m_all;
        scratch_ml[row * 2 + 1] = l_all;
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
attention_decode_merge_kernel(const float* __restrict__ scratch_o,
                                              const float* __restrict__ scratch_ml, T* __restrict__ out,
                                              int out_row_stride, int num_heads, int head_dim, int num_splits) {
  const int t = blockIdx.x, head = blockIdx.y;
  const size_t row0 = ((size_t)t * num_heads + head) * num_splits;
  float m_all = -INFINITY;
  for (int s = 0; s < num_splits; ++s) m_all = fmaxf(m_all, scratch_ml[(row0 + s) * 2]);
  for (int e = threadIdx.x; e < head_dim; e += blockDim.x) {
    float l_all = 0.f, o = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float ms = scratch_ml[(row0 + s) * 2];
      const float w = ms == -INFINITY ? 0.f : softmax_exp<T>(ms - m_all);
      l_all += scratch_ml[(row0 + s) * 2 + 1] * w;
      o += scratch_o[(row0 + s) * head_dim + e] * w;
    }
    out[(size_t)t * out_row_stride + (size_t)head * head_dim + e] = from_float<T>(l_all > 0.f ? o / l_all : 0.f);
  }
}

template <typename T, int DL>
int launch_decode(const void* q, int q_row_stride, void* out, int out_row_stride, float* scratch_o,
                  float* scratch_ml, const int* positions, const int* token_seq, const int* seq_seat,
                  const int* block_table, int table_width, const void* k_cache, const void* v_cache, int tokens,
                  int num_heads, int num_kv_heads, int page_size, int num_pages, int window, float scale,
                  int num_splits, int* error, cudaStream_t stream) {
  const int group = num_heads / num_kv_heads;
  // Heads of one kv head are handled GC at a time; pick the chunk that wastes least.
  int gc = 8;
  if (group == 1) gc = 1;
  else if (group == 2) gc = 2;
  else if (group <= 4) gc = 4;
  else if (group % 6 == 0 && group % 8 != 0) gc = 6;
  const int chunks = (group + gc - 1) / gc;
  const dim3 grid(tokens, num_kv_heads * chunks, num_splits);
#define DISTIE_DECODE_CASE(GCV)                                                                                  \
  attention_decode_kernel<T, DL, GCV><<<grid, kDecodeThreads, 0, stream>>>(                                      \
      (const T*)q, q_row_stride, (T*)out, out_row_stride, scratch_o, scratch_ml, positions, token_seq, seq_seat, \
      block_table, table_width, (const T*)k_cache, (const T*)v_cache, num_heads, group, chunks, num_kv_heads,    \
      page_size, num_pages, window, scale, error)
  switch (gc) {
    case 1: DISTIE_DECODE_CASE(1); break;
    case 2: DISTIE_DECODE_CASE(2); break;
    case 4: DISTIE_DECODE_CASE(4); break;
    case 6: DISTIE_DECODE_CASE(6); break;
    default: DISTIE_DECODE_CASE(8); break;
  }
#undef DISTIE_DECODE_CASE
  DISTIE_LAUNCH_CHECK();
  if (num_splits > 1) {
    const dim3 merge_grid(tokens, num_heads);
    attention_decode_merge_kernel<T><<<merge_grid, DL * 8 >= 128 ? 128 : 64, 0, stream>>>(
        scratch_o, scratch_ml, (T*)out, out_row_stride, num_heads, DL * 8, num_splits);
    DISTIE_LAUNCH_CHECK();
  }
  return 0;
}

template <typename T>
int dispatch_decode(int head_dim, const void* q, int q_row_stride, void* out, int out_row_stride,
                    float* scratch_o, float* scratch_ml, const int* positions, const int* token_seq,
                    const int* seq_seat, const int* block_table, int table_width, const void* k_cache,
                    const void* v_cache, int tokens, int num_heads, int num_kv_heads, int page_size, int num_pages,
                    int window, float scale, int num_splits, int* error, cudaStream_t stream) {
#define DISTIE_DECODE_DIM(DLV)                                                                                   \
  return launch_decode<T, DLV>(q, q_row_stride, out, out_row_stride, scratch_o, scratch_ml, positions, token_seq, \
                               seq_seat, block_table, table_width, k_cache, v_cache, tokens, num_heads,          \
                               num_kv_heads, page_size, num_pages, window, scale, num_splits, error, stream)
  switch (head_dim) {
    case 16: DISTIE_DECODE_DIM(2);
    case 32: DISTIE_DECODE_DIM(4);
    case 64: DISTIE_DECODE_DIM(8);
    case 128: DISTIE_DECODE_DIM(16);
    case 256: DISTIE_DECODE_DIM(32);
    default: return DISTIE_ERR_UNSUPPORTED;
  }
#undef DISTIE_DECODE_DIM
}

}  // namespace distie

using namespace distie;

// Floats of scratch the call needs: tokens * heads * splits * (head_dim + 2); none with one split.
extern "C" long long distie_attention_decode_scratch_floats(int tokens, int num_heads, int head_dim, int num_splits) {
  if (num_splits <= 1) return 0;
  return (long long)tokens * num_heads * num_splits * (head_dim + 2);
}

extern "C" int distie_attention_decode(const void* q, int q_row_stride, void* out, int out_row_stride,
                                       float* scratch, const int* positions, const int* token_seq,
                                       const int* seq_seat, const int* block_table, int table_width,
                                       const void* k_cache, const void* v_cache, int tokens, int num_heads,
                                       int num_kv_heads, int head_dim, int page_size, int num_pages, int window,
                                       float scale, int num_splits, int dtype, int* error, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads != 0 || page_size < 1 || table_width < 1 ||
      num_splits < 1 || num_splits > 65535 || (num_splits > 1 && scratch == nullptr))
    return DISTIE_ERR_ARG;
  float* scratch_o = scratch;
  float* scratch_ml = scratch ? scratch + (size_t)tokens * num_heads * num_splits * head_dim : nullptr;
  if (dtype == DISTIE_BF16)
    return dispatch_decode<__nv_bfloat16>(head_dim, q, q_row_stride, out, out_row_stride, scratch_o, scratch_ml,
                                          positions, token_seq, seq_seat, block_table, table_width, k_cache, v_cache,
                                          tokens, num_heads, num_kv_heads, page_size, num_pages, window, scale,
                                          num_splits, error, stream);
  if (dtype == DISTIE_F32)
    return dispatch_decode<float>(head_dim, q, q_row_stride, out, out_row_stride, scratch_o, scratch_ml, positions,
                                  token_seq, seq_seat, block_table, table_width, k_cache, v_cache, tokens, num_heads,
                                  num_kv_heads, page_size, num_pages, window, scale, num_splits, error, stream);
  return DISTIE_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------
// distie_attention_decode_static: the same split-KV attention for callers that
// cannot allocate.  Declared and explained in no_alloc.h.
// ---------------------------------------------------------------------------
#include "no_alloc.h"

namespace distie {

// Room for the partial results of one call, held by every GPU that loads this library until the
// process exits.  Host code must not pass this name to a kernel: on the host it is only a handle
// for cudaGetSymbolAddress; the device address is looked up once per device below.
static __device__ __align__(256) float g_static_scratch[DISTIE_STATIC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
static float* g_static_scratch_address[kMaxDevices] = {};

// Device address of the array on the current device; looked up on the first call on that device.
static int static_scratch_address(float** out) {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return (int)err;
  if (device < 0 || device >= kMaxDevices) return DISTIE_ERR_ARG;
  if (g_static_scratch_address[device] == nullptr) {
    void* address = nullptr;
    err = cudaGetSymbolAddress(&address, g_static_scratch);
    if (err != cudaSuccess) return (int)err;
    g_static_scratch_address[device] = static_cast<float*>(address);
  }
  *out = g_static_scratch_address[device];
  return 0;
}

}  // namespace distie

extern "C" long long distie_attention_decode_static_capacity(void) { return DISTIE_STATIC_SCRATCH_FLOATS; }

extern "C" const char* distie_no_alloc_error(int code) {
  switch (code) {
    case 0: return "ok";
    case DISTIE_ERR_ARG: return "invalid argument";
    case DISTIE_ERR_UNSUPPORTED: return "head size or element type not supported by this kernel";
    case DISTIE_ERR_SCRATCH_TOO_SMALL:
      return "tokens * heads * splits * (head_dim + 2) exceeds the built-in scratch of "
             "DISTIE_STATIC_SCRATCH_FLOATS floats: use fewer splits or tokens, or the allocating entry point";
    default: return "CUDA error (the code is a cudaError_t)";
  }
}

extern "C" int distie_attention_decode_static(const void* q, int q_row_stride, void* out, int out_row_stride,
                                              const int* positions, const int* token_seq, const int* seq_seat,
                                              const int* block_table, int table_width, const void* k_cache,
                                              const void* v_cache, int tokens, int num_heads, int num_kv_heads,
                                              int head_dim, int page_size, int num_pages, int window, float scale,
                                              int num_splits, int dtype, int* error, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (num_heads < 1 || head_dim < 1 || num_splits < 1) return DISTIE_ERR_ARG;
  const long long needed = distie_attention_decode_scratch_floats(tokens, num_heads, head_dim, num_splits);
  if (needed > (long long)DISTIE_STATIC_SCRATCH_FLOATS) return DISTIE_ERR_SCRATCH_TOO_SMALL;
  float* scratch = nullptr;
  const int status = static_scratch_address(&scratch);
  if (status != 0) return status;
  // Nothing in the array has to start at zero: the first kernel writes every partial
  // (max, sum, mix) of every (token, head, split) before the merge kernel reads it.
  return distie_attention_decode(q, q_row_stride, out, out_row_stride, scratch, positions, token_seq, seq_seat,
                                 block_table, table_width, k_cache, v_cache, tokens, num_heads, num_kv_heads, head_dim,
                                 page_size, num_pages, window, scale, num_splits, dtype, error, stream);
}
