// Row-wise kernels of the decoder: embedding gather, residual sum + RMSNorm,
// position rotation fused with the paged key/value write, and SiLU(gate)*up.
//
// Conventions: the residual stream is float32 in both engines (the residual sum
// is a 32-bit sum); activations between kernels are T (bfloat16 or float);
// norm weights, biases and rotation frequencies are float32.
#include "common.cuh"

namespace distie {

// ---------------------------------------------------------------------------
// Embedding: residual[t, :] = table[ids[t], :] as float32.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                             float* __restrict__ residual, int hidden, int vocab, int* __restrict__ error) {
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0 && error) atomicExch(error, 1);
    id = 0;  // never read outside the table
  }
  const T* row = table + (size_t)id * hidden;
  float* out = residual + (size_t)t * hidden;
  if ((hidden & 7) == 0) {
    for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
      float v[8];
      load8(row + i, v);
      store8(out + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = to_float(row[i]);
  }
}

// ---------------------------------------------------------------------------
// residual += delta (float32 sum, written back), then
//   out = weight * cast_T(residual * rsqrt(mean(residual^2) + eps))
// The normalised value is rounded to T before the weight multiplies it, as the
// reference does.  With `rows_index` the kernel normalises only the listed rows
// (used before the output head) and leaves the residual untouched.
// One block per output row.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void add_rmsnorm_kernel(const T* __restrict__ delta, float* __restrict__ residual,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows_index, int hidden, float eps) {
  __shared__ float scratch[32];
  const int out_row = blockIdx.x;
  const int row = rows_index ? rows_index[out_row] : out_row;
  float* res = residual + (size_t)row * hidden;
  const T* del = delta ? delta + (size_t)row * hidden : nullptr;
  T* dst = out + (size_t)out_row * hidden;
  const bool write_back = (delta != nullptr) && (rows_index == nullptr);

  float sumsq = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = res[i];
    if (del) v += to_float(del[i]);
    if (write_back) res[i] = v;
    sumsq += v * v;
  }
  const float total = block_sum(sumsq, scratch);
  const float rstd = rsqrtf(total / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = res[i];
    if (del && !write_back) v += to_float(del[i]);
    const float normed = to_float(from_float<T>(v * rstd));
    dst[i] = from_float<T>(weight[i] * normed);
  }
}

// The same for rows whose width is a multiple of 4 and at most 16 * blockDim.x (blocks of up to 512): every thread
// loads all its elements before it computes anything (one round trip to memory instead of one
// per loop iteration) and keeps the summed residual in registers for the second pass.
// `delta` may also be the float32 partial sums of a product whose K was split over several CTAs:
// `splits` slices, `split_stride` elements apart, which are added up here in a fixed order.
template <typename T, typename DT, int VPT>
__global__ void __launch_bounds__(512) add_rmsnorm_vec_kernel(const DT* __restrict__ delta, int splits, size_t split_stride,
                                       float* __restrict__ residual, const float* __restrict__ weight,
                                       T* __restrict__ out, const int* __restrict__ rows_index, int hidden,
                                       float eps) {
  constexpr int ROUND = 16 / VPT;  // slices whose loads are in flight together
  __shared__ float scratch[32];
  const int out_row = blockIdx.x;
  const int row = rows_index ? rows_index[out_row] : out_row;
  float* res = residual + (size_t)row * hidden;
  const DT* del = delta ? delta + (size_t)row * hidden : nullptr;
  T* dst = out + (size_t)out_row * hidden;
  const bool write_back = (delta != nullptr) && (rows_index == nullptr);
  const int chunks = hidden >> 2;
  float4 v[VPT], wv[VPT];
  grid_dependency_release();
#pragma unroll
  for (int i = 0; i < VPT; ++i) {  // the norm's weight is written by no kernel: load it before the wait
    const int ch = threadIdx.x + i * blockDim.x;
    wv[i] = ch < chunks ? load4(weight + 4 * ch) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  grid_dependency_wait();
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int ch = threadIdx.x + i * blockDim.x;
    v[i] = ch < chunks ? load4(res + 4 * ch) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (del) {
    // ROUND slices per round, all their loads issued before any sum: one round trip for a whole round.
    for (int sp0 = 0; sp0 < splits; sp0 += ROUND) {
      float4 d[ROUND][VPT];
#pragma unroll
      for (int u = 0; u < ROUND; ++u)
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int ch = threadIdx.x + i * blockDim.x;
          d[u][i] = (sp0 + u < splits && ch < chunks) ? load4_cg(del + (sp0 + u) * split_stride + 4 * ch)
                                                      : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
      for (int u = 0; u < ROUND; ++u)  // fixed order: slice 0 first
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          v[i].x += d[u][i].x; v[i].y += d[u][i].y; v[i].z += d[u][i].z; v[i].w += d[u][i].w;
        }
    }
  }
  float sumsq = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int ch = threadIdx.x + i * blockDim.x;
    if (write_back && ch < chunks) store4(res + 4 * ch, v[i]);
    sumsq += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  }
  const float total = block_sum(sumsq, scratch);
  const float rstd = rsqrtf(total / (float)hidden + eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int ch = threadIdx.x + i * blockDim.x;
    if (ch >= chunks) continue;
    float4 y;
    y.x = wv[i].x * to_float(from_float<T>(v[i].x * rstd));
    y.y = wv[i].y * to_float(from_float<T>(v[i].y * rstd));
    y.z = wv[i].z * to_float(from_float<T>(v[i].z * rstd));
    y.w = wv[i].w * to_float(from_float<T>(v[i].w * rstd));
    store4(dst + 4 * ch, y);
  }
}

// Threads and elements per thread for a row of `hidden` (a multiple of 4, at most 8192).  A CTA per row in
// every case.  Many rows (prompt portions) want small CTAs, at most 256 threads with four or eight pieces of
// 4 per thread: many CTAs fit an SM and each thread has eight or sixteen loads in flight (2,048 rows of
// 3,584: 11.3 us against 18.6 us with two pieces and against 20.2 us with a warp per row and the row in
// registers, a form that was removed; the same bytes take a plain copy 8.5 us).  Few rows (decoding) want
// as many threads per row as 512 allow: alone, the kernel is as fast with four pieces per thread there too,
// but a decode step of 8 rows was 15 % longer with them (1.42 against 1.23 ms), so the rule for few rows
// stays as the whole step measured it.
template <typename T, typename DT>
static cudaError_t launch_add_rmsnorm_vec(const DT* delta, int splits, size_t split_stride, float* residual,
                                          const float* weight, T* out, const int* rows_index, int rows, int hidden,
                                          float eps, cudaStream_t stream) {
  const int chunks = hidden >> 2;
  int vpt;
  if (rows >= 256) vpt = chunks <= 1024 ? 4 : 8;
  else vpt = chunks <= 512 ? 1 : (chunks <= 1024 ? 2 : 4);
  const int threads = (((chunks + vpt - 1) / vpt) + 31) & ~31;
  if (vpt == 1)
    return launch_dependent_family(2, add_rmsnorm_vec_kernel<T, DT, 1>, dim3(rows), dim3(threads), 0, stream, delta, splits,
                                   split_stride, residual, weight, out, rows_index, hidden, eps);
  if (vpt == 2)
    return launch_dependent_family(2, add_rmsnorm_vec_kernel<T, DT, 2>, dim3(rows), dim3(threads), 0, stream, delta, splits,
                                   split_stride, residual, weight, out, rows_index, hidden, eps);
  if (vpt == 8)
    return launch_dependent_family(2, add_rmsnorm_vec_kernel<T, DT, 8>, dim3(rows), dim3(threads), 0, stream, delta, splits,
                                   split_stride, residual, weight, out, rows_index, hidden, eps);
  return launch_dependent_family(2, add_rmsnorm_vec_kernel<T, DT, 4>, dim3(rows), dim3(threads), 0, stream, delta, splits,
                                 split_stride, residual, weight, out, rows_index, hidden, eps);
}

// ---------------------------------------------------------------------------
// Rotation of q and k (rotate-half or interleaved pairs, over the first
// `rotary_dim` dims of each head) in float32, fused with the write of the new
// key and value rows into their pages.
//
//   qkv      [T, row_stride]: q heads, then k heads, then v heads, each head_dim wide
//   k_cache  [pages, kv_heads, page_size, head_dim] of this layer's slot (v likewise)
//   slot of token t = block_table[seat(t), pos / page_size], row pos % page_size
//
// q is rotated in place; k (rotated) and v go straight to the cache; nothing else
// is written.  Without `inv_freq` nothing is rotated; with `write_cache == 0`
// only q is handled.  One block per token.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ token_seq, const int* __restrict__ seq_seat,
                                     const int* __restrict__ block_table, int table_width,
                                     const float* __restrict__ inv_freq, float trig_factor, T* __restrict__ k_cache,
                                     T* __restrict__ v_cache, int row_stride, int num_heads, int num_kv_heads,
                                     int head_dim, int rotary_dim, int interleaved, int page_size, int num_pages,
                                     int write_cache, int* __restrict__ error) {
  extern __shared__ float trig[];  // cos[rotary_dim/2], sin[rotary_dim/2]
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = rotary_dim >> 1;
  if (inv_freq) {
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      float s, c;
      sincosf((float)pos * inv_freq[j], &s, &c);
      trig[j] = c * trig_factor;  // the factor scales cos and sin alike (1 for the plain rotation)
      trig[half + j] = s * trig_factor;
    }
  }
  __syncthreads();

  T* row = qkv + (size_t)t * row_stride;
  T* k_dst = nullptr;
  T* v_dst = nullptr;
  if (write_cache) {
    const int seat = seq_seat[token_seq[t]];
    const int column = pos / page_size;
    const int page = (pos >= 0 && column < table_width) ? block_table[(size_t)seat * table_width + column] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0 && error) atomicExch(error, 2);
      write_cache = 0;  // never write outside the slab
    } else {
      const size_t base = ((size_t)page * num_kv_heads * page_size + (pos % page_size)) * head_dim;
      k_dst = k_cache + base;
      v_dst = v_cache + base;
    }
  }
  const size_t cache_head_stride = (size_t)page_size * head_dim;

  // q and k heads: pairs (j, j + half) or (2j, 2j + 1) inside the rotary dims.
  const int rot_heads = num_heads + num_kv_heads;
  const int pairs_per_head = head_dim >> 1;
  for (int idx = threadIdx.x; idx < rot_heads * pairs_per_head; idx += blockDim.x) {
    const int head = idx / pairs_per_head;
    const int j = idx % pairs_per_head;
    const bool is_k = head >= num_heads;
    if (is_k && !write_cache) continue;
    T* src = row + (size_t)head * head_dim;
    int i0, i1;
    float c = 1.f, s = 0.f;
    if (j < half) {
      if (interleaved) { i0 = 2 * j; i1 = 2 * j + 1; } else { i0 = j; i1 = j + half; }
      if (inv_freq) { c = trig[j]; s = trig[half + j]; }
    } else {  // dims beyond rotary_dim pass through, two at a time
      i0 = rotary_dim + 2 * (j - half);
      i1 = i0 + 1;
    }
    const float x0 = to_float(src[i0]), x1 = to_float(src[i1]);
    const float y0 = x0 * c - x1 * s;
    const float y1 = x1 * c + x0 * s;
    if (is_k) {
      T* dst = k_dst + (size_t)(head - num_heads) * cache_head_stride;
      dst[i0] = from_float<T>(y0);
      dst[i1] = from_float<T>(y1);
    } else {
      src[i0] = from_float<T>(y0);
      src[i1] = from_float<T>(y1);
    }
  }
  if (write_cache) {
    const T* v_src = row + (size_t)(num_heads + num_kv_heads) * head_dim;
    for (int idx = threadIdx.x; idx < num_kv_heads * head_dim; idx += blockDim.x) {
      const int head = idx / head_dim, i = idx % head_dim;
      v_dst[(size_t)head * cache_head_stride + i] = v_src[idx];
    }
  }
}

// The common case (rotate-half over the whole head, head_dim a multiple of 16, rows aligned to
// 16 bytes) in pieces of 4 elements: a thread loads the 4 low and the 4 matching high elements of
// one head, rotates them and stores them (q in place, k to its page); the values are copied in
// pieces of 8.  All loads of a thread come before its stores.
// The input may be the product itself (QT = T; q is then rotated in place when q_out is the input)
// or the float32 partial sums of a product whose K was split (`splits` slices, `split_stride`
// elements apart), to which the bias is added here: the projection's epilogue, the rotation and
// the cache write are then one kernel and q goes to its own buffer.
template <typename T, typename QT>
__global__ void rope_kv_write_vec_kernel(const QT* in, int splits, size_t split_stride, int row_stride,
                                         const float* __restrict__ bias, T* q_out, int q_out_stride,
                                         const int* __restrict__ positions, const int* __restrict__ token_seq,
                                         const int* __restrict__ seq_seat, const int* __restrict__ block_table,
                                         int table_width, const float* __restrict__ inv_freq, float trig_factor, T* __restrict__ k_cache,
                                         T* __restrict__ v_cache, int num_heads, int num_kv_heads, int head_dim,
                                         int page_size, int num_pages, int write_cache, int* __restrict__ error) {
  extern __shared__ float trig[];  // cos[head_dim/2], sin[head_dim/2]
  // Positions, block tables and frequencies are inputs of the step, written by no kernel: the
  // angles and the page are worked out before the wait for the projection.
  grid_dependency_release();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = head_dim >> 1;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float s = 0.f, c = 1.f;
    if (inv_freq) {
      sincosf((float)pos * inv_freq[j], &s, &c);
      c *= trig_factor;  // the factor scales cos and sin alike (1 for the plain rotation)
      s *= trig_factor;
    }
    trig[j] = c;
    trig[half + j] = s;
  }
  const QT* row = in + (size_t)t * row_stride;
  T* k_dst = nullptr;
  T* v_dst = nullptr;
  if (write_cache) {
    const int seat = seq_seat[token_seq[t]];
    const int column = pos / page_size;
    const int page = (pos >= 0 && column < table_width) ? block_table[(size_t)seat * table_width + column] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0 && error) atomicExch(error, 2);
      write_cache = 0;
    } else {
      const size_t base = ((size_t)page * num_kv_heads * page_size + (pos % page_size)) * head_dim;
      k_dst = k_cache + base;
      v_dst = v_cache + base;
    }
  }
  __syncthreads();
  grid_dependency_wait();
  const size_t cache_head_stride = (size_t)page_size * head_dim;
  const int pieces = half >> 2;  // pieces of 4 pairs per head
  const int rot_units = (num_heads + (write_cache ? num_kv_heads : 0)) * pieces;
  const int v_units = write_cache ? num_kv_heads * (head_dim >> 3) : 0;
  // Two pieces of 4 elements of the input row, each summed over the splits in slice order, plus the
  // bias.  The loads of up to eight slices are issued before any sum: one round trip for all of them.
  constexpr int ROUND = 8;
  auto gather = [&](int first, int second, float4& a, float4& b) {
    a = make_float4(0.f, 0.f, 0.f, 0.f);
    b = a;
    if (splits == 1) {  // the product of a prompt portion: one slice, no rounds
      a = load4_cg(row + first);
      b = load4_cg(row + second);
    }
    for (int sp0 = 0; splits > 1 && sp0 < splits; sp0 += ROUND) {
      float4 da[ROUND], db[ROUND];
#pragma unroll
      for (int u = 0; u < ROUND; ++u) {
        if (sp0 + u < splits) {
          const QT* slice = row + (sp0 + u) * split_stride;
          da[u] = load4_cg(slice + first);
          db[u] = load4_cg(slice + second);
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
    if (bias) {
      const float4 ba = load4(bias + first), bb = load4(bias + second);
      a.x += ba.x; a.y += ba.y; a.z += ba.z; a.w += ba.w;
      b.x += bb.x; b.y += bb.y; b.z += bb.z; b.w += bb.w;
    }
  };
  for (int unit = threadIdx.x; unit < rot_units + v_units; unit += blockDim.x) {
    if (unit < rot_units) {
      const int head = unit / pieces, j0 = (unit % pieces) * 4;
      float4 lo, hi;
      gather(head * head_dim + j0, head * head_dim + half + j0, lo, hi);
      const float4 c = *reinterpret_cast<const float4*>(trig + j0), sn = *reinterpret_cast<const float4*>(trig + half + j0);
      const float4 out_lo = make_float4(lo.x * c.x - hi.x * sn.x, lo.y * c.y - hi.y * sn.y, lo.z * c.z - hi.z * sn.z,
                                        lo.w * c.w - hi.w * sn.w);
      const float4 out_hi = make_float4(hi.x * c.x + lo.x * sn.x, hi.y * c.y + lo.y * sn.y, hi.z * c.z + lo.z * sn.z,
                                        hi.w * c.w + lo.w * sn.w);
      T* dst = head < num_heads ? q_out + (size_t)t * q_out_stride + (size_t)head * head_dim
                                : k_dst + (size_t)(head - num_heads) * cache_head_stride;
      store4(dst + j0, out_lo);
      store4(dst + half + j0, out_hi);
    } else {
      const int piece = unit - rot_units;
      const int head = piece / (head_dim >> 3), j0 = (piece % (head_dim >> 3)) * 8;
      float4 first, second;
      const int offset = (num_heads + num_kv_heads + head) * head_dim + j0;
      gather(offset, offset + 4, first, second);
      store4(v_dst + (size_t)head * cache_head_stride + j0, first);
      store4(v_dst + (size_t)head * cache_head_stride + j0 + 4, second);
    }
  }
}

// ---------------------------------------------------------------------------
// out[t, i] = silu(gate_up[t, i]) * gate_up[t, inter + i], computed in float32.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total) {
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter;
    const int i = (int)(idx % inter);
    const float g = to_float(gate_up[t * 2 * inter + i]);
    const float u = to_float(gate_up[t * 2 * inter + inter + i]);
    out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
  }
}

// The same in pieces of 8 elements (inter a multiple of 8): blockIdx.y is the row, so no division per element.
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter) {
  const size_t t = blockIdx.y;
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= inter) return;
  float g[8], u[8], y[8];
  load8(gate_up + t * 2 * inter + i, g);
  load8(gate_up + t * 2 * inter + inter + i, u);
#pragma unroll
  for (int e = 0; e < 8; ++e) y[e] = g[e] / (1.f + expf(-g[e])) * u[e];
  store8(out + t * inter + i, y);
}

// out (T) [rows, cols] = cast(in (float32) + bias[col]): the epilogue of a product whose
// float32 result gets its bias added before the one rounding to T.
template <typename T>
__global__ void bias_cast_kernel(const float* __restrict__ in, const float* __restrict__ bias, T* __restrict__ out,
                                 int cols, size_t total) {
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    float v = in[idx];
    if (bias) v += bias[idx % cols];
    out[idx] = from_float<T>(v);
  }
}

}  // namespace distie

using namespace distie;

extern "C" int distie_embed(const int* ids, const void* table, float* residual, int tokens, int hidden, int vocab,
                            int table_dtype, int* error, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (hidden < 1 || vocab < 1) return DISTIE_ERR_ARG;
  const int threads = hidden >= 2048 ? 256 : 128;
  if (table_dtype == DISTIE_BF16)
    embed_kernel<<<tokens, threads, 0, stream>>>(ids, (const __nv_bfloat16*)table, residual, hidden, vocab, error);
  else if (table_dtype == DISTIE_F32)
    embed_kernel<<<tokens, threads, 0, stream>>>(ids, (const float*)table, residual, hidden, vocab, error);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}

extern "C" int distie_add_rmsnorm(const void* delta, float* residual, const float* weight, void* out,
                                  const int* rows_index, int rows, int hidden, float eps, int dtype,
                                  cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden < 1) return DISTIE_ERR_ARG;
  if (dtype != DISTIE_BF16 && dtype != DISTIE_F32) return DISTIE_ERR_UNSUPPORTED;
  const bool aligned = (((uintptr_t)delta | (uintptr_t)residual | (uintptr_t)weight | (uintptr_t)out) & 15) == 0;
  if ((hidden & 3) == 0 && hidden <= 16 * 512 && aligned) {
    cudaError_t err;
    if (dtype == DISTIE_BF16)
      err = launch_add_rmsnorm_vec((const __nv_bfloat16*)delta, 1, (size_t)0, residual, weight, (__nv_bfloat16*)out,
                                   rows_index, rows, hidden, eps, stream);
    else
      err = launch_add_rmsnorm_vec((const float*)delta, 1, (size_t)0, residual, weight, (float*)out, rows_index, rows,
                                   hidden, eps, stream);
    return err == cudaSuccess ? 0 : (int)err;
  }
  const int threads = hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128);
  if (dtype == DISTIE_BF16)
    add_rmsnorm_kernel<<<rows, threads, 0, stream>>>((const __nv_bfloat16*)delta, residual, weight,
                                                     (__nv_bfloat16*)out, rows_index, hidden, eps);
  else
    add_rmsnorm_kernel<<<rows, threads, 0, stream>>>((const float*)delta, residual, weight, (float*)out,
                                                     rows_index, hidden, eps);
  DISTIE_LAUNCH_CHECK();
  return 0;
}

extern "C" int distie_rope_kv_write(void* qkv, const int* positions, const int* token_seq, const int* seq_seat,
                                    const int* block_table, int table_width, const float* inv_freq, float trig_factor, void* k_cache,
                                    void* v_cache, int tokens, int row_stride, int num_heads, int num_kv_heads,
                                    int head_dim, int rotary_dim, int interleaved, int page_size, int num_pages,
                                    int write_cache, int dtype, int* error, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (head_dim < 2 || (head_dim & 1) || rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1) ||
      num_heads < 1 || num_kv_heads < 1 || page_size < 1 || table_width < 1)
    return DISTIE_ERR_ARG;
  if (dtype != DISTIE_BF16 && dtype != DISTIE_F32) return DISTIE_ERR_UNSUPPORTED;
  const bool aligned = (((uintptr_t)qkv | (uintptr_t)k_cache | (uintptr_t)v_cache) & 31) == 0;
  if ((inv_freq == nullptr || rotary_dim == head_dim) && !interleaved && (head_dim & 15) == 0 &&
      (row_stride & 7) == 0 && aligned) {
    const int units = (num_heads + num_kv_heads) * (head_dim >> 3) + num_kv_heads * (head_dim >> 3);
    const int threads = units >= 512 ? 512 : ((units + 31) & ~31);
    const size_t bytes = (size_t)head_dim * sizeof(float);
    if (dtype == DISTIE_BF16)
      rope_kv_write_vec_kernel<<<tokens, threads, bytes, stream>>>(
          (const __nv_bfloat16*)qkv, 1, (size_t)0, row_stride, (const float*)nullptr, (__nv_bfloat16*)qkv, row_stride,
          positions, token_seq, seq_seat, block_table, table_width, inv_freq, trig_factor, (__nv_bfloat16*)k_cache,
          (__nv_bfloat16*)v_cache, num_heads, num_kv_heads, head_dim, page_size, num_pages, write_cache, error);
    else
      rope_kv_write_vec_kernel<<<tokens, threads, bytes, stream>>>(
          (const float*)qkv, 1, (size_t)0, row_stride, (const float*)nullptr, (float*)qkv, row_stride, positions,
          token_seq, seq_seat, block_table, table_width, inv_freq, trig_factor, (float*)k_cache, (float*)v_cache, num_heads,
          num_kv_heads, head_dim, page_size, num_pages, write_cache, error);
    DISTIE_LAUNCH_CHECK();
    return 0;
  }
  const int threads = 128;
  const size_t shared = (size_t)rotary_dim * sizeof(float);
  if (dtype == DISTIE_BF16)
    rope_kv_write_kernel<<<tokens, threads, shared, stream>>>(
        (__nv_bfloat16*)qkv, positions, token_seq, seq_seat, block_table, table_width, inv_freq, trig_factor,
        (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, row_stride, num_heads, num_kv_heads, head_dim, rotary_dim,
        interleaved, page_size, num_pages, write_cache, error);
  else if (dtype == DISTIE_F32)
    rope_kv_write_kernel<<<tokens, threads, shared, stream>>>(
        (float*)qkv, positions, token_seq, seq_seat, block_table, table_width, inv_freq, trig_factor, (float*)k_cache,
        (float*)v_cache, row_stride, num_heads, num_kv_heads, head_dim, rotary_dim, interleaved, page_size, num_pages,
        write_cache, error);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}

// What the q/k/v product's fused epilogue reads per token, made once per step and shared by the layers of a
// cache group: trig[t] = (cos of the token's angles | sin of them) * factor, [head_dim] float32 (1 | 0 without
// a table of frequencies), and cache_row[t] = page * kv_heads * page_size + pos % page_size, the row of the
// token's slot for kv head 0 in a cache of [pages, kv_heads, page_size, head_dim], or -1 (with the error flag
// set) where the block table has no page for it.
__global__ void rope_rows_kernel(const int* __restrict__ positions, const int* __restrict__ token_seq,
                                 const int* __restrict__ seq_seat, const int* __restrict__ block_table, int table_width,
                                 const float* __restrict__ inv_freq, float trig_factor, int tokens, int head_dim,
                                 int num_kv_heads, int page_size, int num_pages, float* __restrict__ trig,
                                 int* __restrict__ cache_row, int* __restrict__ error) {
  const int t = blockIdx.x;
  if (t >= tokens) return;
  const int pos = positions[t];
  const int half = head_dim >> 1;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float s = 0.f, c = 1.f;
    if (inv_freq) {
      sincosf((float)pos * inv_freq[j], &s, &c);
      c *= trig_factor;
      s *= trig_factor;
    }
    trig[(size_t)t * head_dim + j] = c;
    trig[(size_t)t * head_dim + half + j] = s;
  }
  if (threadIdx.x == 0 && cache_row != nullptr) {
    const int seat = seq_seat[token_seq[t]];
    const int column = pos / page_size;
    const int page = (pos >= 0 && column < table_width) ? block_table[(size_t)seat * table_width + column] : -1;
    if (page < 0 || page >= num_pages) {
      if (error) atomicExch(error, 2);
      cache_row[t] = -1;
    } else {
      cache_row[t] = page * num_kv_heads * page_size + (pos % page_size);
    }
  }
}

extern "C" int distie_rope_rows(const int* positions, const int* token_seq, const int* seq_seat, const int* block_table,
                                int table_width, const float* inv_freq, float trig_factor, int tokens, int head_dim,
                                int num_kv_heads, int page_size, int num_pages, float* trig, int* cache_row, int* error,
                                cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (head_dim < 2 || (head_dim & 1) || trig == nullptr || positions == nullptr) return DISTIE_ERR_ARG;
  if (cache_row != nullptr) {
    if (num_kv_heads < 1 || page_size < 1 || table_width < 1 || num_pages < 1 || block_table == nullptr) return DISTIE_ERR_ARG;
    if ((long long)num_pages * num_kv_heads * page_size > 0x7fffffffLL) return DISTIE_ERR_UNSUPPORTED;  // rows are int32
  }
  rope_rows_kernel<<<tokens, 64, 0, stream>>>(positions, token_seq, seq_seat, block_table, table_width, inv_freq,
                                              trig_factor, tokens, head_dim, num_kv_heads, page_size, num_pages, trig,
                                              cache_row, error);
  DISTIE_LAUNCH_CHECK();
  return 0;
}

// The same two kernels fed with the float32 partial sums of a product whose K was split
// (`splits` slices of [rows, width], `split_stride` elements apart).  They exist only in the
// vectorised form: other shapes return DISTIE_ERR_UNSUPPORTED and the caller adds the slices up itself.
extern "C" int distie_add_rmsnorm_split(const float* partials, int splits, long long split_stride, float* residual,
                                        const float* weight, void* out, const int* rows_index, int rows, int hidden,
                                        float eps, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden < 1 || splits < 1 || partials == nullptr) return DISTIE_ERR_ARG;
  if (dtype != DISTIE_BF16 && dtype != DISTIE_F32) return DISTIE_ERR_UNSUPPORTED;
  const bool aligned = (((uintptr_t)partials | (uintptr_t)residual | (uintptr_t)weight | (uintptr_t)out) & 15) == 0;
  if ((hidden & 3) || hidden > 16 * 512 || !aligned || (split_stride & 3)) return DISTIE_ERR_UNSUPPORTED;
  cudaError_t err;
  if (dtype == DISTIE_BF16)
    err = launch_add_rmsnorm_vec(partials, splits, (size_t)split_stride, residual, weight, (__nv_bfloat16*)out, rows_index,
                                 rows, hidden, eps, stream);
  else
    err = launch_add_rmsnorm_vec(partials, splits, (size_t)split_stride, residual, weight, (float*)out, rows_index, rows,
                                 hidden, eps, stream);
  return err == cudaSuccess ? 0 : (int)err;
}

extern "C" int distie_rope_kv_write_split(const float* partials, int splits, long long split_stride, int row_stride,
                                          const float* bias, void* q_out, int q_out_stride, const int* positions,
                                          const int* token_seq, const int* seq_seat, const int* block_table,
                                          int table_width, const float* inv_freq, float trig_factor, void* k_cache, void* v_cache,
                                          int tokens, int num_heads, int num_kv_heads, int head_dim, int rotary_dim,
                                          int interleaved, int page_size, int num_pages, int write_cache, int dtype,
                                          int* error, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (head_dim < 2 || num_heads < 1 || num_kv_heads < 1 || page_size < 1 || table_width < 1 || splits < 1 ||
      partials == nullptr || q_out == nullptr)
    return DISTIE_ERR_ARG;
  if (dtype != DISTIE_BF16 && dtype != DISTIE_F32) return DISTIE_ERR_UNSUPPORTED;
  const bool aligned =
      (((uintptr_t)partials | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)bias) & 31) == 0;
  if (!((inv_freq == nullptr || rotary_dim == head_dim) && !interleaved && (head_dim & 15) == 0 &&
        (row_stride & 7) == 0 && (q_out_stride & 7) == 0 && (split_stride & 7) == 0 && aligned))
    return DISTIE_ERR_UNSUPPORTED;
  const int units = (num_heads + num_kv_heads) * (head_dim >> 3) + num_kv_heads * (head_dim >> 3);
  const int threads = units >= 512 ? 512 : ((units + 31) & ~31);
  const size_t bytes = (size_t)head_dim * sizeof(float);
  cudaError_t err;
  if (dtype == DISTIE_BF16)
    err = launch_dependent_family(4, rope_kv_write_vec_kernel<__nv_bfloat16, float>, dim3(tokens), dim3(threads), bytes, stream,
                           partials, splits, (size_t)split_stride, row_stride, bias, (__nv_bfloat16*)q_out, q_out_stride,
                           positions, token_seq, seq_seat, block_table, table_width, inv_freq, trig_factor, (__nv_bfloat16*)k_cache,
                           (__nv_bfloat16*)v_cache, num_heads, num_kv_heads, head_dim, page_size, num_pages, write_cache,
                           error);
  else
    err = launch_dependent_family(4, rope_kv_write_vec_kernel<float, float>, dim3(tokens), dim3(threads), bytes, stream, partials,
                           splits, (size_t)split_stride, row_stride, bias, (float*)q_out, q_out_stride, positions,
                           token_seq, seq_seat, block_table, table_width, inv_freq, trig_factor, (float*)k_cache, (float*)v_cache,
                           num_heads, num_kv_heads, head_dim, page_size, num_pages, write_cache, error);
  return err == cudaSuccess ? 0 : (int)err;
}

extern "C" int distie_swiglu(const void* gate_up, void* out, int tokens, int inter, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (inter < 1) return DISTIE_ERR_ARG;
  const size_t total = (size_t)tokens * inter;
  const int threads = 256;
  if ((inter & 7) == 0 && tokens <= 65535 && (((uintptr_t)gate_up | (uintptr_t)out) & 31) == 0 &&
      (dtype == DISTIE_BF16 || dtype == DISTIE_F32)) {
    const dim3 grid((inter / 8 + 127) / 128, tokens);
    if (dtype == DISTIE_BF16)
      swiglu_vec_kernel<<<grid, 128, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter);
    else
      swiglu_vec_kernel<<<grid, 128, 0, stream>>>((const float*)gate_up, (float*)out, inter);
    DISTIE_LAUNCH_CHECK();
    return 0;
  }
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == DISTIE_BF16)
    swiglu_kernel<<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total);
  else if (dtype == DISTIE_F32)
    swiglu_kernel<<<blocks, threads, 0, stream>>>((const float*)gate_up, (float*)out, inter, total);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}

extern "C" int distie_bias_cast(const float* in, const float* bias, void* out, long long rows, int cols, int dtype,
                                cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (cols < 1) return DISTIE_ERR_ARG;
  const size_t total = (size_t)rows * cols;
  const int threads = 256;
  const size_t want = (total + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == DISTIE_BF16)
    bias_cast_kernel<<<blocks, threads, 0, stream>>>(in, bias, (__nv_bfloat16*)out, cols, total);
  else if (dtype == DISTIE_F32)
    bias_cast_kernel<<<blocks, threads, 0, stream>>>(in, bias, (float*)out, cols, total);
  else
    return DISTIE_ERR_UNSUPPORTED;
  DISTIE_LAUNCH_CHECK();
  return 0;
}
