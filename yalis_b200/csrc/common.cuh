// Shared device helpers for every kernel of the library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define YALIS_API extern "C" __attribute__((visibility("default")))

// dtype codes used across the C boundary
enum : int { YALIS_F32 = 0, YALIS_BF16 = 1 };

// Error codes returned by launchers (0 = launched).
enum : int {
  YALIS_OK = 0,
  YALIS_ERR_DTYPE = -1,      // dtype code not handled by this kernel
  YALIS_ERR_SHAPE = -2,      // a size this kernel refuses
  YALIS_ERR_LAUNCH = -3,     // cudaGetLastError() after the launch was not cudaSuccess
  YALIS_ERR_ALIGN = -4,      // a pointer or stride not aligned as the kernel needs
};

// Bits of the device error word (one int32 per engine).  Kernels never trap: what they cannot do they skip,
// raise a bit here with atomicOr and return; the host reads the word where it synchronises anyway.
enum : int {
  YALIS_FLAG_BAD_ID = 1,          // a token id outside the vocabulary (its embedding row was zeroed)
  YALIS_FLAG_BAD_PAGE = 2,        // a block-table entry outside the pool (the token was skipped)
  YALIS_FLAG_WAIT_ATTENTION = 4,  // a bounded wait of an attention kernel ran out (its block gave up)
  YALIS_FLAG_WAIT_PRODUCT = 8,    // a bounded wait of the weight-streaming product ran out
};

inline int yalis_launch_status() {
  return cudaGetLastError() == cudaSuccess ? YALIS_OK : YALIS_ERR_LAUNCH;
}

// Streaming multiprocessors of the current device (asked of the driver once per device).
inline int yalis_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// ---- programmatic dependent launch ---------------------------------------------------
// Every kernel of the library is launched with the "programmatic stream serialization"
// attribute: the next kernel in the stream may be scheduled while this one still runs, do
// work that does not depend on it (set-up, prefetch of weights) and then block in
// pdl_wait() until this one has completed and its writes are visible.  Rules kept by every
// kernel here: (1) pdl_wait() is executed by every thread before any early return and before the
// first read of an activation or write of an output, so completion of a kernel implies completion
// of all kernels before it; (2) only constant inputs (weights) are touched before pdl_wait() - and,
// where the caller of a kernel says so explicitly, data that was complete before the preceding
// kernel began (the cache entries of earlier steps and a step's index arrays: the decode attention's
// early fetch); (3) pdl_launch_dependents() is called at the top of short kernels, but by the
// bandwidth-bound ones (weight-streaming product, decode attention) only when a block has requested
// its last tile: blocks of the next kernels that start earlier fill their rings with bandwidth that
// this kernel's own tiles still wait for, and hold registers and shared memory that its later
// blocks need (measured: 9 % of a batch-64 decode step).
bool yalis_pdl_enabled();   // defined in elementwise.cu; switched by yalis_set_pdl()

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline int yalis_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                        Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = yalis_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...) == cudaSuccess ? YALIS_OK : YALIS_ERR_LAUNCH;
}

// The same with the grid divided into thread-block clusters of `cluster` blocks (each a divisor of the grid).
template <typename... KArgs, typename... Args>
inline int yalis_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, dim3 cluster, size_t smem,
                                cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster.x;
  attr[0].val.clusterDim.y = cluster.y;
  attr[0].val.clusterDim.z = cluster.z;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = yalis_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...) == cudaSuccess ? YALIS_OK : YALIS_ERR_LAUNCH;
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Sum of the n partial values p[s * stride], added in index order but loaded eight at a time
// (a load per addition would cost a trip to the L2 for each).
template <typename TS>
__device__ __forceinline__ float sum_parts(const TS* __restrict__ p, int n, size_t stride) {
  float acc = 0.f;
  for (int s0 = 0; s0 < n; s0 += 8) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = s0 + j < n ? to_f32<TS>(p[(size_t)(s0 + j) * stride]) : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += v[j];
  }
  return acc;
}

// silu(g) = g / (1 + exp(-g)).  The float32 path uses the accurate functions; on the bfloat16 path the result is
// rounded to 8 bits of mantissa at once, so the fast exponential and division (relative error about 1e-6) do not
// show, and they make the activation kernel memory-bound instead of arithmetic-bound (34 -> ~10 instructions an
// element).  One function for every bfloat16 place (activation kernels, the product's fused epilogue), so that
// they agree to the bit.
__device__ __forceinline__ float silu_exact(float g) { return g / (1.0f + expf(-g)); }
__device__ __forceinline__ float silu_bf16_path(float g) { return __fdividef(g, 1.0f + __expf(-g)); }
template <typename T>
__device__ __forceinline__ float silu_for(float g);
template <>
__device__ __forceinline__ float silu_for<float>(float g) { return silu_exact(g); }
template <>
__device__ __forceinline__ float silu_for<__nv_bfloat16>(float g) { return silu_bf16_path(g); }

// (x1, x2) turned by the angle with cosine cs and sine sn.  One pinned instruction sequence, so that every
// kernel that rotates (the rotary kernels, the decode attention that rotates its own queries) agrees to the bit.
__device__ __forceinline__ void rotate_pair(float x1, float x2, float cs, float sn, float& o1, float& o2) {
  o1 = __fmaf_rn(x1, cs, -__fmul_rn(x2, sn));
  o2 = __fmaf_rn(x2, cs, __fmul_rn(x1, sn));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` is 32 floats of shared memory; safe to call repeatedly.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? scratch[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

// Dispatch on a dtype code to a templated callable.
#define YALIS_DISPATCH_DTYPE(code, T, ...)                 \
  do {                                                     \
    if ((code) == YALIS_F32) {                             \
      using T = float;                                     \
      __VA_ARGS__;                                         \
    } else if ((code) == YALIS_BF16) {                     \
      using T = __nv_bfloat16;                             \
      __VA_ARGS__;                                         \
    } else {                                               \
      return YALIS_ERR_DTYPE;                              \
    }                                                      \
  } while (0)
