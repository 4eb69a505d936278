// Memory-bound kernels of the forward path: embedding gather, RMSNorm fused
// with the residual add, rotary encoding fused with the write of K and V into
// cache pages, and SiLU(gate)*up.  All arithmetic is float32; only loads and
// stores are in the storage type T (float or bfloat16).
#include "common.cuh"

// --------------------------------------------------------------------------
// Embedding: out[t, :] = float(table[ids[t], :])      (yalis/external/model.py:137)
// The residual stream is float32 whatever the weight type.
// A token id outside [0, vocab) yields a row of zeros and raises *bad_id.
// --------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int32_t* __restrict__ ids,
                                 float* __restrict__ out, int width, int vocab, int32_t* bad_id) {
  const int t = blockIdx.x;
  const int id = ids[t];
  float* o = out + (size_t)t * width;
  if (id < 0 || id >= vocab) {
    for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = 0.f;
    if (threadIdx.x == 0 && bad_id) atomicExch(bad_id, 1);
    return;
  }
  const T* row = table + (size_t)id * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) o[c] = to_f32<T>(row[c]);
}

YALIS_API int yalis_embedding(const void* table, int dtype, const int32_t* ids, float* out, int n_tokens,
                              int width, int vocab, int32_t* bad_id, cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  YALIS_DISPATCH_DTYPE(dtype, T,
                       embedding_kernel<T><<<n_tokens, 256, 0, stream>>>((const T*)table, ids, out, width, vocab,
                                                                         bad_id));
  return yalis_launch_status();
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
template <typename T, typename TD>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta, int n_delta,
                                   size_t delta_stride, const float* __restrict__ w, T* __restrict__ y,
                                   const int32_t* __restrict__ rows, int width, float eps, int write_back) {
  __shared__ float scratch[32];
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  if (r < 0) return;  // padded row
  float* xr = x + (size_t)r * width;
  const TD* dr = delta ? delta + (size_t)r * width : nullptr;
  float ss = 0.f;
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
  T* yr = y + (size_t)i * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float h = xr[c];
    if (dr && !write_back)
      for (int s = 0; s < n_delta; ++s) h += to_f32<TD>(dr[(size_t)s * delta_stride + c]);
    yr[c] = from_f32<T>((h * inv) * w[c]);
  }
}

// delta_dtype: type of delta (YALIS_F32 for split-K partials, else the model type).
YALIS_API int yalis_add_rmsnorm(float* x, const void* delta, int delta_dtype, int n_delta, long long delta_stride,
                                const float* w, void* y, int out_dtype, const int32_t* rows, int n_out_rows,
                                int width, float eps, int write_back, cudaStream_t stream) {
  if (n_out_rows <= 0) return YALIS_OK;
  const int threads = width >= 2048 ? 512 : 256;
  YALIS_DISPATCH_DTYPE(
      out_dtype, T,
      if (delta_dtype == YALIS_F32) {
        add_rmsnorm_kernel<T, float><<<n_out_rows, threads, 0, stream>>>(
            x, (const float*)delta, n_delta, (size_t)delta_stride, w, (T*)y, rows, width, eps, write_back);
      } else if (delta_dtype == YALIS_BF16) {
        add_rmsnorm_kernel<T, __nv_bfloat16><<<n_out_rows, threads, 0, stream>>>(
            x, (const __nv_bfloat16*)delta, n_delta, (size_t)delta_stride, w, (T*)y, rows, width, eps, write_back);
      } else { return YALIS_ERR_DTYPE; });
  return yalis_launch_status();
}

// Plain residual add without a norm: x[r] += sum_s delta[s][r]. Used to flush a
// pending delta when a caller wants the residual stream itself.
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ x, const TD* __restrict__ delta, int n_delta,
                                    size_t delta_stride, size_t n) {
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
    residual_add_kernel<float><<<blocks, threads, 0, stream>>>(x, (const float*)delta, n_delta, (size_t)delta_stride,
                                                              (size_t)n);
  else if (delta_dtype == YALIS_BF16)
    residual_add_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(x, (const __nv_bfloat16*)delta, n_delta,
                                                                      (size_t)delta_stride, (size_t)n);
  else
    return YALIS_ERR_DTYPE;
  return yalis_launch_status();
}

// --------------------------------------------------------------------------
// Rotary encoding of Q and K and the write of K, V into cache pages.
//   angle = float(pos) * inv_freq[i]         (float32, as torch.outer of the
//   reference's table, yalis/external/model.py:810-820)
//   out[i]        = x[i]*cos - x[i+hs/2]*sin
//   out[i+hs/2]   = x[i+hs/2]*cos + x[i]*sin  (half-split, model.py:894-909)
// Q is rotated in place inside the fused qkv row; K (rotated) and V go to
//   pool[page][kv_head][pos % page_size][:], page = block_table[req][pos / page_size]
// (the reference's paged scatter: yalis/attention/utils/flash_utils.py:33-43).
// inv_freq == null means "no rotation" (K and V are still stored); k_pool == null
// means "store nothing" (Q is still rotated).
// A token whose request index is negative is padding and is skipped; a token
// whose page is unmapped raises *bad_page and is not stored.
// One block per token.
// --------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int qkv_stride, const int32_t* __restrict__ positions,
                                     const int32_t* __restrict__ req_of_token, const float* __restrict__ inv_freq,
                                     T* __restrict__ k_pool, T* __restrict__ v_pool,
                                     const int32_t* __restrict__ block_table, int table_width, int page_size,
                                     int num_pages, int nh, int g, int hs, int32_t* bad_page) {
  extern __shared__ float cs[];  // cos[hs/2], sin[hs/2]
  const int t = blockIdx.x;
  const int req = req_of_token[t];
  if (req < 0) return;
  const int pos = positions[t];
  const int half = hs >> 1;
  if (inv_freq) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float angle = (float)pos * inv_freq[i];
      float s, c;
      sincosf(angle, &s, &c);
      cs[i] = c;
      cs[half + i] = s;
    }
  }
  __syncthreads();
  T* row = qkv + (size_t)t * qkv_stride;
  const int page_idx = pos / page_size;
  int page = -1;
  if (k_pool != nullptr) {  // a layer that reads another layer's cache stores nothing
    page = (page_idx < table_width) ? block_table[(size_t)req * table_width + page_idx] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0 && bad_page) atomicExch(bad_page, 1);
      page = -1;
    }
  }
  const int off = pos - page_idx * page_size;
  // Q heads then K heads: (nh + g) * half rotation pairs.
  const int n_pairs = (nh + g) * half;
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int head = p / half, i = p - head * half;
    T* src = row + (size_t)head * hs;  // K heads follow the Q heads in the fused row
    float x1 = to_f32<T>(src[i]), x2 = to_f32<T>(src[i + half]);
    float o1 = x1, o2 = x2;
    if (inv_freq) {
      const float c = cs[i], s = cs[half + i];
      o1 = x1 * c - x2 * s;
      o2 = x2 * c + x1 * s;
    }
    if (head < nh) {
      src[i] = from_f32<T>(o1);
      src[i + half] = from_f32<T>(o2);
    } else if (page >= 0) {
      const int kvh = head - nh;
      T* dst = k_pool + (((size_t)page * g + kvh) * page_size + off) * hs;
      dst[i] = from_f32<T>(o1);
      dst[i + half] = from_f32<T>(o2);
    }
  }
  if (page >= 0) {
    const T* vsrc = row + (size_t)(nh + g) * hs;
    for (int p = threadIdx.x; p < g * hs; p += blockDim.x) {
      const int kvh = p / hs, d = p - kvh * hs;
      v_pool[(((size_t)page * g + kvh) * page_size + off) * hs + d] = vsrc[p];
    }
  }
}

YALIS_API int yalis_rope_kv_write(void* qkv, int dtype, int qkv_stride, const int32_t* positions,
                                  const int32_t* req_of_token, const float* inv_freq, void* k_pool, void* v_pool,
                                  const int32_t* block_table, int table_width, int page_size, int num_pages, int nh,
                                  int g, int hs, int n_tokens, int32_t* bad_page, cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (hs <= 0 || (hs & 1)) return YALIS_ERR_SHAPE;
  const size_t smem = (size_t)hs * sizeof(float);
  if (smem > 48 * 1024) return YALIS_ERR_SHAPE;
  YALIS_DISPATCH_DTYPE(dtype, T,
                       rope_kv_write_kernel<T><<<n_tokens, 256, smem, stream>>>(
                           (T*)qkv, qkv_stride, positions, req_of_token, inv_freq, (T*)k_pool, (T*)v_pool, block_table,
                           table_width, page_size, num_pages, nh, g, hs, bad_page));
  return yalis_launch_status();
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
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / inter;
  const int i = (int)(idx - t * inter);
  const T* row = in + t * 2 * (size_t)inter;
  const float gate = to_f32<T>(interleaved ? row[2 * i] : row[i]);
  const float up = to_f32<T>(interleaved ? row[2 * i + 1] : row[inter + i]);
  const float act = gate / (1.0f + expf(-gate));
  out[idx] = from_f32<T>(act * up);
}

YALIS_API int yalis_silu_mul(const void* in, void* out, int dtype, int n_tokens, int inter, int interleaved,
                             cudaStream_t stream) {
  const size_t total = (size_t)n_tokens * inter;
  if (total == 0) return YALIS_OK;
  const int threads = 256;
  const unsigned blocks = (unsigned)((total + threads - 1) / threads);
  YALIS_DISPATCH_DTYPE(dtype, T,
                       silu_mul_kernel<T><<<blocks, threads, 0, stream>>>((const T*)in, (T*)out, inter, interleaved,
                                                                          total));
  return yalis_launch_status();
}

// Gather rows of a float32 matrix: out[i, :] = x[rows[i], :].
__global__ void gather_rows_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows,
                                   float* __restrict__ out, int width) {
  const int r = rows[blockIdx.x];
  if (r < 0) return;
  for (int c = threadIdx.x; c < width; c += blockDim.x) out[(size_t)blockIdx.x * width + c] = x[(size_t)r * width + c];
}

YALIS_API int yalis_gather_rows_f32(const float* x, const int32_t* rows, float* out, int n_rows, int width,
                                    cudaStream_t stream) {
  if (n_rows <= 0) return YALIS_OK;
  gather_rows_kernel<<<n_rows, 256, 0, stream>>>(x, rows, out, width);
  return yalis_launch_status();
}
