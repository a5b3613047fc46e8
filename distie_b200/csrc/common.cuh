// Shared helpers of the sm_100a kernels: element types, loads that convert to
// float, warp and block reductions, and the launcher conventions.
//
// Every launcher is `extern "C"`, takes raw device pointers plus a stream, starts
// no allocation and no synchronisation, and returns 0 or a cudaError_t (negative
// values are argument errors found on the host).  Element types are selected by
// the integer codes below so that one shared library serves the bfloat16 and the
// float32 engine.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define DISTIE_F32 0
#define DISTIE_BF16 1

#define DISTIE_ERR_ARG (-1)
#define DISTIE_ERR_UNSUPPORTED (-2)

#define DISTIE_LAUNCH_CHECK()                 \
  do {                                        \
    cudaError_t err__ = cudaGetLastError();   \
    if (err__ != cudaSuccess) return (int)err__; \
  } while (0)

namespace distie {

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats of shared memory.
// Every thread gets the result.  Safe to call repeatedly with the same scratch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int warps = (blockDim.x + 31) >> 5;
  float total = (lane < warps) ? scratch[lane] : 0.f;
  total = warp_sum(total);
  return total;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int warps = (blockDim.x + 31) >> 5;
  float total = (lane < warps) ? scratch[lane] : -INFINITY;
  total = warp_max(total);
  return total;
}

// Eight consecutive elements as floats.  `p` must be aligned to 8 elements
// (16 bytes for bfloat16, 32 for float).
__device__ __forceinline__ void load8(const float* p, float (&out)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
  out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&out)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162 t;
  t = __floats2bfloat162_rn(v[0], v[1]); raw.x = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(v[2], v[3]); raw.y = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(v[4], v[5]); raw.z = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(v[6], v[7]); raw.w = *reinterpret_cast<uint32_t*>(&t);
  *reinterpret_cast<uint4*>(p) = raw;
}

// Programmatic dependent launch.  A kernel launched with `launch_dependent` may start while the
// kernel before it in the stream is still running; it may read data that no kernel of the step
// writes (weights, the step's index arrays, block tables) at once, and must call
// `grid_dependency_wait()` before it reads anything an earlier kernel produced and before it
// writes global memory (a buffer it writes may still be read by an earlier kernel).  The wait
// returns when all earlier kernels have finished and their writes are visible.  Calling
// `grid_dependency_release()` early lets the next kernel start its own independent part in turn.
// Launched the ordinary way, both calls do nothing.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Loads of data that the kernel before this one produced, for kernels that start early (see
// launch_dependent below): through L2 (.cg), never through the non-coherent path or a line that L1
// may still hold from before the producer ran.
__device__ __forceinline__ uint4 load16_cg(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void load8_cg(const float* p, float (&out)[8]) {
  const uint4 a = load16_cg(p), b = load16_cg(p + 4);
  out[0] = __uint_as_float(a.x); out[1] = __uint_as_float(a.y); out[2] = __uint_as_float(a.z); out[3] = __uint_as_float(a.w);
  out[4] = __uint_as_float(b.x); out[5] = __uint_as_float(b.y); out[6] = __uint_as_float(b.z); out[7] = __uint_as_float(b.w);
}
__device__ __forceinline__ void load8_cg(const __nv_bfloat16* p, float (&out)[8]) {
  const uint4 raw = load16_cg(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ float4 load4_cg(const float* p) {
  const uint4 a = load16_cg(p);
  return make_float4(__uint_as_float(a.x), __uint_as_float(a.y), __uint_as_float(a.z), __uint_as_float(a.w));
}
__device__ __forceinline__ float4 load4_cg(const __nv_bfloat16* p) {
  uint2 raw;
  asm volatile("ld.global.cg.v2.u32 {%0,%1}, [%2];" : "=r"(raw.x), "=r"(raw.y) : "l"(p) : "memory");
  return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                     __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
}

// Four consecutive elements as floats (16-byte aligned for float, 8-byte for bfloat16).
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                     __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  uint2 raw;
  __nv_bfloat162 t;
  t = __floats2bfloat162_rn(v.x, v.y); raw.x = *reinterpret_cast<uint32_t*>(&t);
  t = __floats2bfloat162_rn(v.z, v.w); raw.y = *reinterpret_cast<uint32_t*>(&t);
  *reinterpret_cast<uint2*>(p) = raw;
}

// ---- thread-block clusters: barrier and reads of another CTA's shared memory -----------------------------------
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The barrier at the end of a kernel whose only purpose is that no CTA of the cluster leaves while another may still
// read its shared memory: it orders execution, not memory.  (With release semantics a thread would first wait until
// its own stores to global memory have been acknowledged, about a microsecond that the end of the grid waits for anyway.)
__device__ __forceinline__ void cluster_barrier_exit() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
}
// The float at `local` (an address in this CTA's shared memory) as CTA `rank` of the cluster holds it.
__device__ __forceinline__ float cluster_load(const float* local, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// A launch that may start before the kernel ahead of it in the stream has finished (the kernel calls
// grid_dependency_wait() before it touches what that kernel writes), optionally as thread-block
// clusters of `cluster` CTAs (cluster.x == 0: no clusters).
template <typename... Params, typename... Args>
inline cudaError_t launch_dependent_cluster(int family, dim3 cluster, void (*kernel)(Params...), dim3 grid, dim3 block,
                                            size_t shared, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared;
  config.stream = stream;
  (void)family;  // names the kind of kernel at the call site; every kind starts early
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  if (cluster.x > 0) {
    attribute[1].id = cudaLaunchAttributeClusterDimension;
    attribute[1].val.clusterDim.x = cluster.x;
    attribute[1].val.clusterDim.y = cluster.y;
    attribute[1].val.clusterDim.z = cluster.z;
    config.numAttrs = 2;
  }
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

template <typename... Params, typename... Args>
inline cudaError_t launch_dependent_family(int family, void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared,
                                           cudaStream_t stream, Args... args) {
  return launch_dependent_cluster(family, dim3(0, 0, 0), kernel, grid, block, shared, stream, args...);
}

template <typename... Params, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared,
                                    cudaStream_t stream, Args... args) {
  return launch_dependent_family(0xff, kernel, grid, block, shared, stream, args...);
}

}  // namespace distie
