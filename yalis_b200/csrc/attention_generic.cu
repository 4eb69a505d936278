// Paged causal attention, the exact one: any head size up to 256 (even), any
// number of heads and KV groups, any page size, float32 or bfloat16 storage,
// float32 arithmetic throughout.  One block per (token, head); each warp walks
// every fourth visible key in ascending order with an online softmax and the
// four partial results are merged in warp order.  For a given (position, head)
// the order of every sum is therefore fixed, whatever else is in the batch and
// however the request was cut into steps.  It is the kernel of the float32
// path and the twin against which the faster bfloat16 kernels are tested.
//
//   S = (q . k_j) / sqrt(hs) for keys j with  pos - window < j <= pos   (window 0: all j <= pos)
//   O = softmax(S) V
// Mask by absolute position: yalis/attention/backend_impl/sdpa_and_flex.py:15-19, 301-307.
// KV head of query head h: h / (nh / g)                                 (:59-67).
#include "common.cuh"

namespace {

constexpr int kWarps = 4;
constexpr int kMaxPerLane = 8;  // head size <= 256

template <typename T>
__global__ void paged_attention_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out,
                                               int out_stride, const T* __restrict__ k_pool,
                                               const T* __restrict__ v_pool, const int32_t* __restrict__ positions,
                                               const int32_t* __restrict__ req_of_token,
                                               const int32_t* __restrict__ block_table, int table_width,
                                               int page_size, int num_pages, int nh, int g, int hs, float scale,
                                               int window) {
  extern __shared__ float smem[];  // [kWarps][hs] accumulators, then m[kWarps], l[kWarps]
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int req = req_of_token[t];
  if (req < 0) return;
  const int pos = positions[t];
  const int kvh = h / (nh / g);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per_lane = (hs + 31) >> 5;

  float qr[kMaxPerLane], acc[kMaxPerLane];
  const T* qp = q + (size_t)t * q_stride + (size_t)h * hs;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    qr[i] = (i < per_lane && d < hs) ? to_f32<T>(qp[d]) : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int32_t* bt = block_table + (size_t)req * table_width;
  for (int j = lo + warp; j <= pos; j += kWarps) {
    const int pi = j / page_size;
    const int page = pi < table_width ? bt[pi] : -1;
    if (page < 0 || page >= num_pages) continue;  // unmapped: treated as masked
    const size_t base = (((size_t)page * g + kvh) * page_size + (j - pi * page_size)) * hs;
    const T* kp = k_pool + base;
    const T* vp = v_pool + base;
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int d = lane + 32 * i;
      if (i < per_lane && d < hs) dot += qr[i] * to_f32<T>(kp[d]);
    }
    const float s = warp_sum(dot) * scale;
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);
    const float p = expf(s - m_new);
    l = l * corr + p;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int d = lane + 32 * i;
      if (i < per_lane && d < hs) acc[i] = acc[i] * corr + p * to_f32<T>(vp[d]);
    }
    m = m_new;
  }
  float* acc_s = smem;
  float* m_s = smem + kWarps * hs;
  float* l_s = m_s + kWarps;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int d = lane + 32 * i;
    if (i < per_lane && d < hs) acc_s[warp * hs + d] = acc[i];
  }
  if (lane == 0) {
    m_s[warp] = m;
    l_s[warp] = l;
  }
  __syncthreads();
  float mm = -INFINITY;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, m_s[w]);
  float ll = 0.f;
  float wgt[kWarps];
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    wgt[w] = (m_s[w] == -INFINITY) ? 0.f : expf(m_s[w] - mm);
    ll += l_s[w] * wgt[w];
  }
  T* op = out + (size_t)t * out_stride + (size_t)h * hs;
  for (int d = threadIdx.x; d < hs; d += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) o += acc_s[w * hs + d] * wgt[w];
    op[d] = from_f32<T>(ll > 0.f ? o / ll : 0.f);
  }
}

}  // namespace

YALIS_API int yalis_paged_attention_generic(const void* q, int q_stride, void* out, int out_stride,
                                            const void* k_pool, const void* v_pool, int dtype,
                                            const int32_t* positions, const int32_t* req_of_token,
                                            const int32_t* block_table, int table_width, int page_size,
                                            int num_pages, int n_tokens, int nh, int g, int hs, float scale,
                                            int window, cudaStream_t stream) {
  if (n_tokens <= 0) return YALIS_OK;
  if (hs <= 0 || hs > 32 * kMaxPerLane || (hs & 1) || g <= 0 || nh % g != 0 || nh > 65535) return YALIS_ERR_SHAPE;
  const size_t smem = ((size_t)kWarps * hs + 2 * kWarps) * sizeof(float);
  dim3 grid(n_tokens, nh);
  YALIS_DISPATCH_DTYPE(dtype, T,
                       return yalis_launch(paged_attention_generic_kernel<T>, grid, dim3(kWarps * 32), smem, stream,
                                           (const T*)q, q_stride, (T*)out, out_stride, (const T*)k_pool,
                                           (const T*)v_pool, positions, req_of_token, block_table, table_width,
                                           page_size, num_pages, nh, g, hs, scale, window));
  return YALIS_OK;
}
