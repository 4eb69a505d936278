// Memory-bound kernels of the forward path: embedding gather, RMSNorm fused
// with the residual add, rotary encoding fused with the write of K and V into
// cache pages, and SiLU(gate)*up.  All arithmetic is float32; only loads and
// stores are in the storage type T (float or bfloat16).
#include "common.cuh"

namespace {
bool g_pdl_enabled = true;
}
bool yalis_pdl_enabled() { return g_pdl_enabled; }
// Switches programmatic dependent launch for every kernel of the library (on by default).
YALIS_API void yalis_set_pdl(int enabled) { g_pdl_enabled = enabled != 0; }

// --------------------------------------------------------------------------
// Embedding: out[t, :] = float(table[ids[t], :])      (yalis/external/model.py:137)
// The residual stream is float32 whatever the weight type.
// A token id outside [0, vocab) yields a row of zeros and raises YALIS_FLAG_BAD_ID in *bad_id.
// `scale` multiplies every value in float32 (1 for models that do not scale their embeddings).
// With `from_slot`, a token whose entry there is not negative takes its id from chosen[from_slot[t]] instead of
// ids[t]: the token that an earlier step chose for that request and left on the device.
// --------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int32_t* __restrict__ ids,
                                 const int32_t* __restrict__ from_slot, const int32_t* __restrict__ chosen,
                                 float* __restrict__ out, int width, int vocab, float scale, int32_t* bad_id) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (from_slot != nullptr) {
    const int s = from_slot[t];
    if (s >= 0) id = chosen[s];
  }
  float* o = out + (size_t)t * width;
  if (id < 0 || id >= vocab) {
    for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = 0.f;
    if (threadIdx.x == 0 && bad_id) atomicOr(bad_id, YALIS_FLAG_BAD_ID);
    return;
  }
  const T* row = table + (size_t)id * width;
  if (scale == 1.0f) {
    for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = to_f32<T>(row[c]);
  } else {
    for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = to_f32<T>(row[c]) * scale;
  }
}

YALIS_API int yalis_embedding(const void* table, int dtype, const int32_t* ids, const int32_t* from_slot,
                              const int32_t* chosen, float* out, int n_tokens, int width, int vocab, float scale,
                              int32_t* bad_id, cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if ((from_slot == nullptr) != (chosen == nullptr)) return YALIS_ERR_SHAPE;
  YALIS_DISPATCH_DTYPE(dtype, T,
                       return yalis_launch(embedding_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (const T*)table,
                                           ids, from_slot, chosen, out, width, vocab, scale, bad_id));
  return YALIS_OK;
}

// --------------------------------------------------------------------------
// Soft cap of float32 logits in place: v <- cap * tanh(v / cap).
// --------------------------------------------------------------------------
__global__ void softcap_kernel(float* __restrict__ v, size_t n, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  const float inv = 1.0f / cap;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    v[i] = cap * tanhf(v[i] * inv);
}

YALIS_API int yalis_softcap_f32(float* v, long long n, float cap, cudaStream_t stream) {
  if (n <= 0) return YALIS_OK;
  if (!(cap > 0.f)) return YALIS_ERR_SHAPE;
  const int blocks = (int)((n + 1023) / 1024 < 2048 ? (n + 1023) / 1024 : 2048);
  return yalis_launch(softcap_kernel, dim3(blocks), dim3(256), 0, stream, v, (size_t)n, cap);
}

// --------------------------------------------------------------------------
// RMSNorm with the residual add in front of it.
//   h = x[r] + sum_s delta[s][r]      (float32; the residual stream x is float32)
//   x[r] = h                          (only when write_back)
//   y[i] = (h * rsqrt(mean(h^2) + eps)) * w      rounded once to T
// (yalis/external/model.py:979-986 for the norm, :437-438 for the adds.)
// r = rows ? rows[i] : i, so the final norm can run on the few rows whose logits
// are wanted.  delta may be null; it may also consist of `n_delta` partial sums
// [n_delta, n_rows_total, width] (split-K GEMM partials) added in index order.
// One block per output row; the mean is a fixed-order block reduction, so a
// row's result does not depend on which other rows are in the launch.
// --------------------------------------------------------------------------
// MAXV: values a thread keeps in registers (the row is read once); 0 = re-read variant for wide rows.
template <typename T, typename TD, int MAXV>
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, int n_delta,
                                   size_t delta_stride, const float* __restrict__ w, T* __restrict__ y,
                                   const int32_t* __restrict__ rows, int width, float eps, int write_back) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  if (r < 0) return;  // padded row
  float* xr = x + (size_t)r * width;
  const TD* dr = delta ? delta + (size_t)r * width : nullptr;
  T* yr = y + (size_t)i * width;
  float ss = 0.f;
  if constexpr (MAXV > 0) {
    float h[MAXV];
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int c = threadIdx.x + v * blockDim.x;
      h[v] = c < width ? xr[c] : 0.f;
    }
    if (dr) {
      // Partial sums are added in index order, but loaded a batch at a time: one load per
      // addition would cost a trip to the L2 for every partial.
      constexpr int SB = 32 / MAXV;
      for (int s0 = 0; s0 < n_delta; s0 += SB) {
        float t[SB][MAXV];
#pragma unroll
        for (int j = 0; j < SB; ++j) {
#pragma unroll
          for (int v = 0; v < MAXV; ++v) {
            const int c = threadIdx.x + v * blockDim.x;
            t[j][v] = (s0 + j < n_delta && c < width) ? to_f32<TD>(dr[(size_t)(s0 + j) * delta_stride + c]) : 0.f;
          }
        }
#pragma unroll
        for (int j = 0; j < SB; ++j) {
#pragma unroll
          for (int v = 0; v < MAXV; ++v) h[v] += t[j][v];
        }
      }
      if (write_back) {
#pragma unroll
        for (int v = 0; v < MAXV; ++v) {
          const int c = threadIdx.x + v * blockDim.x;
          if (c < width) xr[c] = h[v];
        }
      }
    }
#pragma unroll
    for (int v = 0; v < MAXV; ++v) ss += h[v] * h[v];
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)width + eps);
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int c = threadIdx.x + v * blockDim.x;
      if (c < width) yr[c] = from_f32<T>((h[v] * inv) * w[c]);
    }
  } else {
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      float h = xr[c];
      if (dr) {
        for (int s = 0; s < n_delta; ++s) h += to_f32<TD>(dr[(size_t)s * delta_stride + c]);
        if (write_back) xr[c] = h;
      }
      ss += h * h;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
      float h = xr[c];
      if (dr && !write_back)
        for (int s = 0; s < n_delta; ++s) h += to_f32<TD>(dr[(size_t)s * delta_stride + c]);
      yr[c] = from_f32<T>((h * inv) * w[c]);
    }
  }
}

// Four consecutive values as float32 (16-byte load for float32 data, 8-byte for bfloat16).
__device__ __forceinline__ float4 load4_f32(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4_f32(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<unsigned*>(&a);
  u.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// The same norm for rows whose width is a multiple of four and whose pointers are 16-byte aligned:
// every thread keeps NV groups of four columns, all loads of a row are in flight at once, and the
// norm's weight is fetched before the wait for the preceding kernel.
template <typename T, typename TD, int NV>
__global__ void __launch_bounds__(1024) add_rmsnorm_vec_kernel(float* __restrict__ x, const TD* __restrict__ delta,
                                                               int n_delta, size_t delta_stride,
                                                               const float* __restrict__ w, T* __restrict__ y,
                                                               const int32_t* __restrict__ rows, int width, float eps,
                                                               int write_back) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  const int n4 = width >> 2;
  float4 wv[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int c = threadIdx.x + v * blockDim.x;
    wv[v] = c < n4 ? load4_f32(w + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  if (r < 0) return;  // padded row
  float* xr = x + (size_t)r * width;
  const TD* dr = delta ? delta + (size_t)r * width : nullptr;
  T* yr = y + (size_t)i * width;
  float4 h[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int c = threadIdx.x + v * blockDim.x;
    h[v] = c < n4 ? load4_f32(xr + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (dr) {
    constexpr int SB = 8 / NV;       // partial sums loaded per batch; they are added in index order
    for (int s0 = 0; s0 < n_delta; s0 += SB) {
      float4 t[SB][NV];
#pragma unroll
      for (int j = 0; j < SB; ++j) {
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          const int c = threadIdx.x + v * blockDim.x;
          t[j][v] = (s0 + j < n_delta && c < n4) ? load4_f32(dr + (size_t)(s0 + j) * delta_stride + 4 * c)
                                                   : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
#pragma unroll
      for (int j = 0; j < SB; ++j) {
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          h[v].x += t[j][v].x; h[v].y += t[j][v].y; h[v].z += t[j][v].z; h[v].w += t[j][v].w;
        }
      }
    }
    if (write_back) {
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const int c = threadIdx.x + v * blockDim.x;
        if (c < n4) store4(xr + 4 * c, h[v]);
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) ss += (h[v].x * h[v].x + h[v].y * h[v].y) + (h[v].z * h[v].z + h[v].w * h[v].w);
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)width + eps);
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int c = threadIdx.x + v * blockDim.x;
    if (c < n4)
      store4(yr + 4 * c, make_float4((h[v].x * inv) * wv[v].x, (h[v].y * inv) * wv[v].y, (h[v].z * inv) * wv[v].z,
                                     (h[v].w * inv) * wv[v].w));
  }
}

template <typename T, typename TD>
int launch_add_rmsnorm(float* x, const void* delta, int n_delta, size_t delta_stride, const float* w, void* y,
                        const int32_t* rows, int n_out_rows, int width, float eps, int write_back,
                        cudaStream_t stream) {
  const uintptr_t ptrs = (uintptr_t)x | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)y;
  if (width % 4 == 0 && width <= 16384 && (ptrs & 15) == 0 && delta_stride % 4 == 0) {
    const int n4 = width / 4;
    // Few rows (decode): as many threads per row as it has groups of four, every load in flight at once.
    // Many rows (prefill): 256 threads per row, so that eight rows are in flight per SM instead of two.
    const int cap = n_out_rows >= 256 ? 256 : 1024;
    const int vthreads = n4 >= cap ? cap : (n4 + 31) / 32 * 32;
    const int nv = (n4 + vthreads - 1) / vthreads;
#define YALIS_NORM_VEC(V)                                                                                          \
  return yalis_launch(add_rmsnorm_vec_kernel<T, TD, V>, dim3(n_out_rows), dim3(vthreads), 0, stream, x,            \
                      (const TD*)delta, n_delta, delta_stride, w, (T*)y, rows, width, eps, write_back)
    if (nv == 1) YALIS_NORM_VEC(1);
    else if (nv == 2) YALIS_NORM_VEC(2);
    else YALIS_NORM_VEC(4);
#undef YALIS_NORM_VEC
  }
  const int threads = width >= 4096 ? 1024 : width >= 1024 ? 512 : 256;
  const int per_thread = (width + threads - 1) / threads;
#define YALIS_NORM_LAUNCH(V)                                                                                  \
  return yalis_launch(add_rmsnorm_kernel<T, TD, V>, dim3(n_out_rows), dim3(threads), 0, stream, x, (const TD*)delta, \
                      n_delta, delta_stride, w, (T*)y, rows, width, eps, write_back)
  if (per_thread <= 4) YALIS_NORM_LAUNCH(4);
  else if (per_thread <= 8) YALIS_NORM_LAUNCH(8);
  else if (per_thread <= 16) YALIS_NORM_LAUNCH(16);
  else YALIS_NORM_LAUNCH(0);
#undef YALIS_NORM_LAUNCH
}

// delta_dtype: type of delta (YALIS_F32 for split-K partials, else the model type).
YALIS_API int yalis_add_rmsnorm(float* x, const void* delta, int delta_dtype, int n_delta, long long delta_stride,
                                const float* w, void* y, int out_dtype, const int32_t* rows, int n_out_rows,
                                int width, float eps, int write_back, cudaStream_t stream) {
  if (n_out_rows <= 0) return YALIS_OK;
  YALIS_DISPATCH_DTYPE(
      out_dtype, T,
      if (delta_dtype == YALIS_F32) {
        return launch_add_rmsnorm<T, float>(x, delta, n_delta, (size_t)delta_stride, w, y, rows, n_out_rows, width,
                                            eps, write_back, stream);
      } else if (delta_dtype == YALIS_BF16) {
        return launch_add_rmsnorm<T, __nv_bfloat16>(x, delta, n_delta, (size_t)delta_stride, w, y, rows, n_out_rows,
                                                    width, eps, write_back, stream);
      } else { return YALIS_ERR_DTYPE; });
  return YALIS_OK;
}

// Plain residual add without a norm: x[r] += sum_s delta[s][r]. Used to flush a
// pending delta when a caller wants the residual stream itself.
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ x, const TD* __restrict__ delta, int n_delta,
                                    size_t delta_stride, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float h = x[i];
  for (int s = 0; s < n_delta; ++s) h += to_f32<TD>(delta[(size_t)s * delta_stride + i]);
  x[i] = h;
}

YALIS_API int yalis_residual_add(float* x, const void* delta, int delta_dtype, int n_delta, long long delta_stride,
                                 long long n, cudaStream_t stream) {
  if (n <= 0) return YALIS_OK;
  const int threads = 256;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  if (delta_dtype == YALIS_F32)
    return yalis_launch(residual_add_kernel<float>, dim3(blocks), dim3(threads), 0, stream, x, (const float*)delta,
                        n_delta, (size_t)delta_stride, (size_t)n);
  if (delta_dtype == YALIS_BF16)
    return yalis_launch(residual_add_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, x,
                        (const __nv_bfloat16*)delta, n_delta, (size_t)delta_stride, (size_t)n);
  return YALIS_ERR_DTYPE;
}

// --------------------------------------------------------------------------
// Rotary encoding of Q and K and the write of K, V into cache pages.
//   angle = float(pos) * inv_freq[i]         (float32, as torch.outer of the
//   reference's table, yalis/external/model.py:810-820)
//   out[i]        = x[i]*cos - x[i+hs/2]*sin
//   out[i+hs/2]   = x[i+hs/2]*cos + x[i]*sin  (half-split, model.py:894-909)
// The source is the fused qkv row [Q heads | K heads | V heads] of each token,
// either in the model type or as `n_parts` float32 partial sums of a split-K
// product (added in order).  Rotated Q goes to q_out [N, nh*hs]; K (rotated)
// and V go to
//   pool[page][kv_head][pos % page_size][:], page = block_table[req][pos / page_size]
// (the reference's paged scatter: yalis/attention/utils/flash_utils.py:33-43).
// inv_freq == null means "no rotation" (K and V are still stored); k_pool == null
// means "store nothing" (Q is still rotated).
// A token whose request index is negative is padding and is skipped; a token
// whose page is unmapped raises *bad_page and is not stored.
// One block per (token, head of the fused row).
// --------------------------------------------------------------------------
template <typename T, typename TS>
__global__ void rope_kv_write_kernel(const TS* __restrict__ src, int src_stride, int n_parts, size_t part_stride,
                                     T* __restrict__ q_out, const int32_t* __restrict__ positions,
                                     const int32_t* __restrict__ req_of_token, const float* __restrict__ inv_freq,
                                     T* __restrict__ k_pool, T* __restrict__ v_pool,
                                     const int32_t* __restrict__ block_table, int table_width, int page_size,
                                     int num_pages, int nh, int g, int hs, int32_t* bad_page) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, head = blockIdx.y;   // head: [0, nh) Q, [nh, nh+g) K, [nh+g, nh+2g) V
  const int req = req_of_token[t];
  if (req < 0) return;
  const int pos = positions[t];
  const int half = hs >> 1;
  const bool is_q = head < nh, is_v = head >= nh + g;
  T* dst;
  if (is_q) {
    dst = q_out + ((size_t)t * nh + head) * hs;
  } else {
    if (k_pool == nullptr) return;               // a layer that reads another layer's cache stores nothing
    const int page_idx = pos / page_size;
    const int page = (page_idx < table_width) ? block_table[(size_t)req * table_width + page_idx] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0 && bad_page) atomicOr(bad_page, YALIS_FLAG_BAD_PAGE);
      return;
    }
    const int kvh = is_v ? head - nh - g : head - nh;
    dst = (is_v ? v_pool : k_pool) + (((size_t)page * g + kvh) * page_size + (pos - page_idx * page_size)) * hs;
  }
  const TS* row = src + (size_t)t * src_stride + (size_t)head * hs;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float x1 = sum_parts<TS>(row + i, n_parts, part_stride);
    const float x2 = sum_parts<TS>(row + i + half, n_parts, part_stride);
    float o1 = x1, o2 = x2;
    if (!is_v && inv_freq) {
      float sn, cs;
      sincosf((float)pos * inv_freq[i], &sn, &cs);
      rotate_pair(x1, x2, cs, sn, o1, o2);
    }
    dst[i] = from_f32<T>(o1);
    dst[i + half] = from_f32<T>(o2);
  }
}

// The same for steps with many tokens: one block per token walks all heads, with the token's
// cosines and sines computed once in shared memory.
template <typename T, typename TS>
__global__ void rope_kv_write_token_kernel(const TS* __restrict__ src, int src_stride, int n_parts, size_t part_stride,
                                           T* __restrict__ q_out, const int32_t* __restrict__ positions,
                                           const int32_t* __restrict__ req_of_token,
                                           const float* __restrict__ inv_freq, T* __restrict__ k_pool,
                                           T* __restrict__ v_pool, const int32_t* __restrict__ block_table,
                                           int table_width, int page_size, int num_pages, int nh, int g, int hs,
                                           int32_t* bad_page) {
  extern __shared__ float cs[];   // cos[hs/2], sin[hs/2]
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int req = req_of_token[t];
  if (req < 0) return;
  const int pos = positions[t];
  const int half = hs >> 1;
  if (inv_freq) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      float sn, c;
      sincosf((float)pos * inv_freq[i], &sn, &c);
      cs[i] = c;
      cs[half + i] = sn;
    }
  }
  int page = -1, off = 0;
  if (k_pool != nullptr) {
    const int page_idx = pos / page_size;
    off = pos - page_idx * page_size;
    page = (page_idx < table_width) ? block_table[(size_t)req * table_width + page_idx] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0 && bad_page) atomicOr(bad_page, YALIS_FLAG_BAD_PAGE);
      page = -1;
    }
  }
  __syncthreads();
  const TS* row = src + (size_t)t * src_stride;
  const int n_heads = nh + 2 * g;
  for (int e = threadIdx.x; e < n_heads * half; e += blockDim.x) {
    const int head = e / half, i = e - head * half;
    const bool is_q = head < nh, is_v = head >= nh + g;
    T* dst;
    if (is_q) {
      dst = q_out + ((size_t)t * nh + head) * hs;
    } else {
      if (page < 0) continue;
      const int kvh = is_v ? head - nh - g : head - nh;
      dst = (is_v ? v_pool : k_pool) + (((size_t)page * g + kvh) * page_size + off) * hs;
    }
    const TS* h = row + (size_t)head * hs;
    const float x1 = sum_parts<TS>(h + i, n_parts, part_stride);
    const float x2 = sum_parts<TS>(h + i + half, n_parts, part_stride);
    float o1 = x1, o2 = x2;
    if (!is_v && inv_freq) {
      const float c = cs[i], sn = cs[half + i];
      rotate_pair(x1, x2, c, sn, o1, o2);
    }
    dst[i] = from_f32<T>(o1);
    dst[i + half] = from_f32<T>(o2);
  }
}

// The per-token kernel for head sizes that are multiples of 8 and 16-byte aligned rows: a thread
// rotates four pairs at once (8- or 16-byte loads and stores).
template <typename T, typename TS>
__global__ void rope_kv_write_token_vec_kernel(const TS* __restrict__ src, int src_stride, int n_parts, size_t part_stride,
                                               T* __restrict__ q_out, const int32_t* __restrict__ positions,
                                               const int32_t* __restrict__ req_of_token,
                                               const float* __restrict__ inv_freq, T* __restrict__ k_pool,
                                               T* __restrict__ v_pool, const int32_t* __restrict__ block_table,
                                               int table_width, int page_size, int num_pages, int nh, int g, int hs,
                                               int32_t* bad_page) {
  extern __shared__ __align__(16) float cs[];   // cos[hs/2], sin[hs/2]
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int req = req_of_token[t];
  if (req < 0) return;
  const int pos = positions[t];
  const int half = hs >> 1;
  if (inv_freq) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      float sn, c;
      sincosf((float)pos * inv_freq[i], &sn, &c);
      cs[i] = c;
      cs[half + i] = sn;
    }
  }
  int page = -1, off = 0;
  if (k_pool != nullptr) {
    const int page_idx = pos / page_size;
    off = pos - page_idx * page_size;
    page = (page_idx < table_width) ? block_table[(size_t)req * table_width + page_idx] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0 && bad_page) atomicOr(bad_page, YALIS_FLAG_BAD_PAGE);
      page = -1;
    }
  }
  __syncthreads();
  const TS* row = src + (size_t)t * src_stride;
  const int n_heads = nh + 2 * g;
  const int quads = half >> 2;
  for (int e = threadIdx.x; e < n_heads * quads; e += blockDim.x) {
    const int head = e / quads, i = (e - head * quads) * 4;
    const bool is_q = head < nh, is_v = head >= nh + g;
    T* dst;
    if (is_q) {
      dst = q_out + ((size_t)t * nh + head) * hs;
    } else {
      if (page < 0) continue;
      const int kvh = is_v ? head - nh - g : head - nh;
      dst = (is_v ? v_pool : k_pool) + (((size_t)page * g + kvh) * page_size + off) * hs;
    }
    const TS* h = row + (size_t)head * hs;
    float4 x1 = load4_f32(h + i), x2 = load4_f32(h + i + half);
    for (int s = 1; s < n_parts; ++s) {     // partial sums in index order
      const float4 a = load4_f32(h + s * part_stride + i), b = load4_f32(h + s * part_stride + i + half);
      x1.x += a.x; x1.y += a.y; x1.z += a.z; x1.w += a.w;
      x2.x += b.x; x2.y += b.y; x2.z += b.z; x2.w += b.w;
    }
    float4 o1 = x1, o2 = x2;
    if (!is_v && inv_freq) {
      const float4 c = *reinterpret_cast<const float4*>(cs + i), sn = *reinterpret_cast<const float4*>(cs + half + i);
      rotate_pair(x1.x, x2.x, c.x, sn.x, o1.x, o2.x);
      rotate_pair(x1.y, x2.y, c.y, sn.y, o1.y, o2.y);
      rotate_pair(x1.z, x2.z, c.z, sn.z, o1.z, o2.z);
      rotate_pair(x1.w, x2.w, c.w, sn.w, o1.w, o2.w);
    }
    store4(dst + i, o1);
    store4(dst + i + half, o2);
  }
}

// src_dtype: the model type (n_parts must be 1) or YALIS_F32 partial sums [n_parts, N, src_stride].
YALIS_API int yalis_rope_kv_write(const void* src, int src_dtype, int src_stride, int n_parts, long long part_stride,
                                  void* q_out, int dtype, const int32_t* positions, const int32_t* req_of_token,
                                  const float* inv_freq, void* k_pool, void* v_pool, const int32_t* block_table,
                                  int table_width, int page_size, int num_pages, int nh, int g, int hs, int n_tokens,
                                  int32_t* bad_page, cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (hs <= 0 || (hs & 1) || n_parts < 1) return YALIS_ERR_SHAPE;
  if (nh + 2 * g > 65535) return YALIS_ERR_SHAPE;
  const bool per_token = n_tokens >= 128;      // enough tokens to fill the GPU with one block each
  dim3 grid(n_tokens, per_token ? 1 : nh + 2 * g);
  const int threads = per_token ? 256 : (hs / 2 + 31) / 32 * 32;
  const size_t smem = per_token ? (size_t)hs * sizeof(float) : 0;
  if (smem > 48 * 1024) return YALIS_ERR_SHAPE;
  const uintptr_t ptrs = (uintptr_t)src | (uintptr_t)q_out | (uintptr_t)k_pool | (uintptr_t)v_pool;
  const bool vec_ok = hs % 8 == 0 && src_stride % 4 == 0 && part_stride % 4 == 0 && (ptrs & 15) == 0;
#define YALIS_ROPE_ARGS(TS_)                                                                                         \
  (const TS_*)src, src_stride, n_parts, (size_t)part_stride, (T*)q_out, positions, req_of_token, inv_freq, (T*)k_pool, \
      (T*)v_pool, block_table, table_width, page_size, num_pages, nh, g, hs, bad_page
  YALIS_DISPATCH_DTYPE(
      dtype, T,
      if (per_token && vec_ok) {
        if (src_dtype == dtype && n_parts == 1)
          return yalis_launch(rope_kv_write_token_vec_kernel<T, T>, grid, dim3(threads), smem, stream, YALIS_ROPE_ARGS(T));
        if (src_dtype == YALIS_F32)
          return yalis_launch(rope_kv_write_token_vec_kernel<T, float>, grid, dim3(threads), smem, stream,
                              YALIS_ROPE_ARGS(float));
        return YALIS_ERR_DTYPE;
      }
      if (src_dtype == dtype && n_parts == 1) {
        return per_token ? yalis_launch(rope_kv_write_token_kernel<T, T>, grid, dim3(threads), smem, stream,
                                        YALIS_ROPE_ARGS(T))
                         : yalis_launch(rope_kv_write_kernel<T, T>, grid, dim3(threads), smem, stream,
                                        YALIS_ROPE_ARGS(T));
      } else if (src_dtype == YALIS_F32) {
        return per_token ? yalis_launch(rope_kv_write_token_kernel<T, float>, grid, dim3(threads), smem, stream,
                                        YALIS_ROPE_ARGS(float))
                         : yalis_launch(rope_kv_write_kernel<T, float>, grid, dim3(threads), smem, stream,
                                        YALIS_ROPE_ARGS(float));
      } else { return YALIS_ERR_DTYPE; });
#undef YALIS_ROPE_ARGS
  return YALIS_OK;
}

// --------------------------------------------------------------------------
// SwiGLU activation: out[t, i] = silu(gate[t, i]) * up[t, i], silu(z) = z / (1 + exp(-z))
// (yalis/external/model.py:741-743; float32 math as the reference's CUDA twin,
// yalis/external/csrc/vllm/activation_kernels.cu:34-37).
// Input row = [gate (inter) | up (inter)] when interleaved == 0, or
// gate0, up0, gate1, up1, ... when interleaved == 1 (the reference's layout).
// --------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ in, T* __restrict__ out, int inter, int interleaved,
                                size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / inter;
  const int i = (int)(idx - t * inter);
  const T* row = in + t * 2 * (size_t)inter;
  const float gate = to_f32<T>(interleaved ? row[2 * i] : row[i]);
  const float up = to_f32<T>(interleaved ? row[2 * i + 1] : row[inter + i]);
  const float act = silu_for<T>(gate);
  out[idx] = from_f32<T>(act * up);
}

// bfloat16, halves layout, inter % 8 == 0: eight elements per 16-byte access, two such groups per thread
// (both pairs of loads are issued before the first use).  The inputs are read once and the output is read
// by another kernel: streaming loads and stores keep them from pushing the weights out of the L2.
__device__ __forceinline__ uint4 silu_mul_8(const uint4 g4, const uint4 u4) {
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
  uint4 o4;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
    o2[k] = __floats2bfloat162_rn(silu_bf16_path(g.x) * u.x, silu_bf16_path(g.y) * u.y);
  }
  return o4;
}

__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                       int inter, size_t total_vec) {
  pdl_launch_dependents();
  pdl_wait();
  const int vec_per_row = inter >> 3;
  const size_t v0 = ((size_t)blockIdx.x * blockDim.x) * 2 + threadIdx.x, v1 = v0 + blockDim.x;
  uint4 g[2], u[2];
  size_t at[2];
  bool live[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const size_t v = j == 0 ? v0 : v1;
    live[j] = v < total_vec;
    if (live[j]) {
      const size_t t = v / vec_per_row;
      const int i = (int)(v - t * vec_per_row) << 3;
      const __nv_bfloat16* row = in + t * 2 * (size_t)inter;
      g[j] = __ldcs(reinterpret_cast<const uint4*>(row + i));
      u[j] = __ldcs(reinterpret_cast<const uint4*>(row + inter + i));
      at[j] = t * (size_t)inter + i;
    }
  }
#pragma unroll
  for (int j = 0; j < 2; ++j)
    if (live[j]) *reinterpret_cast<uint4*>(out + at[j]) = silu_mul_8(g[j], u[j]);
}

YALIS_API int yalis_silu_mul(const void* in, void* out, int dtype, int n_tokens, int inter, int interleaved,
                             cudaStream_t stream) {
  const size_t total = (size_t)n_tokens * inter;
  if (total == 0) return YALIS_OK;
  const int threads = 256;
  if (dtype == YALIS_BF16 && !interleaved && inter % 8 == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
    const size_t total_vec = total >> 3;
    return yalis_launch(silu_mul_bf16x8_kernel, dim3((unsigned)((total_vec + 2 * threads - 1) / (2 * threads))), dim3(threads), 0,
                        stream, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, inter, total_vec);
  }
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  YALIS_DISPATCH_DTYPE(dtype, T,
                       return yalis_launch(silu_mul_kernel<T>, dim3(blocks), dim3(threads), 0, stream, (const T*)in,
                                           (T*)out, inter, interleaved, total));
  return YALIS_OK;
}

// Gather rows of a float32 matrix: out[i, :] = x[rows[i], :].
__global__ void gather_rows_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows,
                                   float* __restrict__ out, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = rows[blockIdx.x];
  if (r < 0) return;
  for (int c = threadIdx.x; c < width; c += blockDim.x) out[(size_t)blockIdx.x * width + c] = x[(size_t)r * width + c];
}

YALIS_API int yalis_gather_rows_f32(const float* x, const int32_t* rows, float* out, int n_rows, int width,
                                    cudaStream_t stream) {
  if (n_rows <= 0) return YALIS_OK;
  return yalis_launch(gather_rows_kernel, dim3(n_rows), dim3(256), 0, stream, x, rows, out, width);
}

// --------------------------------------------------------------------------
// rows x width_bytes from pinned host memory to the device, both with a row pitch: the columns in use of a
// block table whose rows are wider (one strided copy instead of one per row).
// --------------------------------------------------------------------------
YALIS_API int yalis_copy_rows_h2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                                  size_t rows, cudaStream_t stream) {
  if (rows == 0 || width_bytes == 0) return YALIS_OK;
  if (width_bytes > dst_pitch || width_bytes > src_pitch) return YALIS_ERR_SHAPE;
  return cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyHostToDevice, stream) == cudaSuccess
             ? YALIS_OK
             : YALIS_ERR_LAUNCH;
}
