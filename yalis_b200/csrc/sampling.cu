// Token selection over float32 logits [rows, vocab]: argmax, and the
// reference's sampler (yalis/external/sampling.py:41-74) as one kernel:
//   1. top-k: logits below the k-th largest become -inf            (:51-62)
//   2. divide by the temperature if it is > 0                       (:65-66)
//   3. top-p: in descending order, drop every entry whose inclusive cumulative
//      probability exceeds top_p; the first is always kept          (:16-38)
//   4. softmax in float32 and one draw                              (:70-73)
//   greedy (argmax) iff temperature == 0 and top_p == 0             (:64,74)
// The draw is the exponential race the reference uses under compilation,
// argmax_i p_i / e_i with e_i ~ Exp(1) (:5-13), taken in log space, with e_i
// from Philox4x32-10 keyed by the request's seed and counted by (draw number,
// token index).  A request's draw therefore depends only on its own seed, its
// own draw count and its own logits, not on the batch it sits in.
//
// No sort: the k-th largest logit and the top-p cut are found by a radix
// descent over order-preserving 32-bit keys (four passes of 256 bins each).
// Bin masses are accumulated as 64-bit fixed point, so every sum is exact in
// its order and the kernel is deterministic.  Entries tied with the k-th value
// are all kept; entries tied with the top-p boundary value are all dropped
// (unless that value is the maximum).  One block per row.
#include "common.cuh"

namespace {

constexpr int kThreads = 1024;

__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3").
__device__ __forceinline__ uint4 philox4x32(uint4 ctr, uint2 key) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}

// Uniform in (0, 1) with 24 random bits.
__device__ __forceinline__ float uniform_open(uint32_t x) { return ((float)(x >> 8) + 0.5f) * (1.0f / 16777216.0f); }

struct ArgMax {
  float v;
  int i;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  // larger value wins; ties go to the lower index; index -1 means "nothing yet"
  if (b.i < 0) return a;
  if (a.i < 0) return b;
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ ArgMax block_argmax(ArgMax a, ArgMax* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = better(a, b);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = a;
  __syncthreads();
  ArgMax t;
  t.v = 0.f;
  t.i = -1;
  if (lane < nwarps) t = scratch[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, t.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, t.i, o);
    t = better(t, b);
  }
  return t;
}

__global__ void __launch_bounds__(kThreads) argmax_kernel(const float* __restrict__ logits, long long row_stride,
                                                          int vocab, int32_t* __restrict__ out) {
  __shared__ ArgMax scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const float* row = logits + (size_t)blockIdx.x * row_stride;
  ArgMax a;
  a.v = 0.f;
  a.i = -1;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    ArgMax b;
    b.v = row[i];
    b.i = i;
    if (b.v == b.v) a = better(a, b);  // NaN never wins
  }
  a = block_argmax(a, scratch);
  if (threadIdx.x == 0) out[blockIdx.x] = a.i < 0 ? 0 : a.i;
}

constexpr double kFixedOne = 1099511627776.0;  // 2^40

__global__ void __launch_bounds__(kThreads)
sample_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
              const float* __restrict__ temperature, const int32_t* __restrict__ top_k,
              const float* __restrict__ top_p, const unsigned long long* __restrict__ seed,
              const unsigned long long* __restrict__ draw_index, int32_t* __restrict__ out) {
  __shared__ ArgMax scratch[32];
  __shared__ float fscratch[32];
  __shared__ unsigned long long hist[256];
  __shared__ uint32_t sh_prefix;
  __shared__ unsigned long long sh_above;
  __shared__ int sh_remaining;
  __shared__ int sh_done;
  pdl_launch_dependents();
  pdl_wait();

  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  const float temp = temperature[r];
  const float tp = top_p[r];
  const int tk = top_k[r];

  if (!(temp > 0.f) && !(tp > 0.f)) {  // greedy
    ArgMax a;
    a.v = 0.f;
    a.i = -1;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      ArgMax b;
      b.v = row[i];
      b.i = i;
      if (b.v == b.v) a = better(a, b);
    }
    a = block_argmax(a, scratch);
    if (threadIdx.x == 0) out[r] = a.i < 0 ? 0 : a.i;
    return;
  }

  // ---- 1. top-k: key of the k-th largest logit --------------------------------
  uint32_t k_key = 0;  // keep entries with order_key >= k_key
  if (tk > 0 && tk < vocab) {
    if (threadIdx.x == 0) {
      sh_prefix = 0;
      sh_remaining = tk;
    }
    for (int pass = 3; pass >= 0; --pass) {
      for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0;
      __syncthreads();
      const uint32_t prefix = sh_prefix;
      const int shift = 8 * pass;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const uint32_t key = order_key(row[i]);
        const bool match = (pass == 3) || ((key >> (shift + 8)) == (prefix >> (shift + 8)));
        if (match) atomicAdd(&hist[(key >> shift) & 255u], 1ull);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        int remaining = sh_remaining;
        unsigned long long cum = 0;
        int chosen = 0;
        for (int b = 255; b >= 0; --b) {
          if (cum + hist[b] >= (unsigned long long)remaining) {
            chosen = b;
            break;
          }
          cum += hist[b];
        }
        sh_remaining = remaining - (int)cum;
        sh_prefix = prefix | ((uint32_t)chosen << shift);
      }
      __syncthreads();
    }
    k_key = sh_prefix;
    __syncthreads();
  }

  // ---- 2. scale, max and normaliser over the kept entries ----------------------
  const float inv_t = temp > 0.f ? 1.0f / temp : 1.0f;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (order_key(v) >= k_key && v == v) mx = fmaxf(mx, v);
  }
  mx = block_max(mx, fscratch);
  float z = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    if (order_key(v) >= k_key && v == v) z += expf((v - mx) * inv_t);
  }
  z = block_sum(z, fscratch);
  const float inv_z = 1.0f / z;

  // ---- 3. top-p: the key at which the cumulative probability passes top_p -------
  uint32_t p_key = 0;       // keep entries with order_key > p_key ...
  bool keep_equal = true;   // ... and those equal to it if this is set
  if (tp < 1.0f) {
    const unsigned long long limit = (unsigned long long)((double)tp * kFixedOne);
    if (threadIdx.x == 0) {
      sh_prefix = 0;
      sh_above = 0;
      sh_done = 0;
    }
    __syncthreads();
    for (int pass = 3; pass >= 0; --pass) {
      for (int b = threadIdx.x; b < 256; b += blockDim.x) hist[b] = 0;
      __syncthreads();
      const uint32_t prefix = sh_prefix;
      const int shift = 8 * pass;
      if (!sh_done) {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
          const float v = row[i];
          const uint32_t key = order_key(v);
          if (key < k_key || v != v) continue;
          const bool match = (pass == 3) || ((key >> (shift + 8)) == (prefix >> (shift + 8)));
          if (match) {
            const double p = (double)(expf((v - mx) * inv_t) * inv_z);
            atomicAdd(&hist[(key >> shift) & 255u], (unsigned long long)(p * kFixedOne));
          }
        }
      }
      __syncthreads();
      if (threadIdx.x == 0 && !sh_done) {
        unsigned long long above = sh_above;
        int chosen = -1;
        for (int b = 255; b >= 0; --b) {
          if (above + hist[b] > limit) {
            chosen = b;
            break;
          }
          above += hist[b];
        }
        if (chosen < 0) {
          // Only possible in the first pass (later passes split a bin whose mass is already
          // known to cross the limit, and the fixed-point masses add up exactly): the whole
          // row fits under top_p, nothing is dropped.
          sh_done = 1;
          sh_prefix = 0u;
        } else {
          sh_above = above;
          sh_prefix = prefix | ((uint32_t)chosen << shift);
        }
      }
      __syncthreads();
    }
    p_key = sh_prefix;
    // Either nothing is dropped (p_key 0, equal kept), or p_key is the exact key whose entries
    // carry the sum past top_p: they are dropped unless nothing lies above them (the first
    // entry is always kept).
    keep_equal = sh_done ? true : (sh_above == 0);
    __syncthreads();
  }

  // ---- 4. the draw ---------------------------------------------------------------
  const unsigned long long sd = seed[r], ctr = draw_index[r];
  const uint2 key2 = make_uint2((uint32_t)sd, (uint32_t)(sd >> 32));
  ArgMax a;
  a.v = 0.f;
  a.i = -1;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    const uint32_t key = order_key(v);
    if (v != v || key < k_key) continue;
    if (tp < 1.0f && !(key > p_key || (keep_equal && key == p_key))) continue;
    const uint4 rnd = philox4x32(make_uint4((uint32_t)i, (uint32_t)ctr, (uint32_t)(ctr >> 32), 0x59414c49u), key2);
    const float u = uniform_open(rnd.x);
    ArgMax b;
    b.v = (v - mx) * inv_t - logf(-logf(u));  // log p_i - log e_i, up to a constant
    b.i = i;
    a = better(a, b);
  }
  a = block_argmax(a, scratch);
  if (threadIdx.x == 0) out[r] = a.i < 0 ? 0 : a.i;
}

}  // namespace

constexpr int kArgmaxChunks = 32;   // blocks per row in the first phase for wide rows

// Phase 1 of the wide argmax: block (row, chunk) finds the best entry of its slice.
__global__ void __launch_bounds__(kThreads) argmax_partial_kernel(const float* __restrict__ logits, long long row_stride,
                                                                  int vocab, float* __restrict__ part_v,
                                                                  int32_t* __restrict__ part_i) {
  __shared__ ArgMax scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const float* row = logits + (size_t)blockIdx.x * row_stride;
  const int per = (vocab + kArgmaxChunks - 1) / kArgmaxChunks;
  const int lo = blockIdx.y * per, hi = min(vocab, lo + per);
  ArgMax a;
  a.v = 0.f;
  a.i = -1;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    ArgMax b;
    b.v = row[i];
    b.i = i;
    if (b.v == b.v) a = better(a, b);
  }
  a = block_argmax(a, scratch);
  if (threadIdx.x == 0) {
    part_v[blockIdx.x * kArgmaxChunks + blockIdx.y] = a.v;
    part_i[blockIdx.x * kArgmaxChunks + blockIdx.y] = a.i;
  }
}

// Phase 2: one warp per row merges the slices (ties still go to the lowest index).
__global__ void argmax_merge_kernel(const float* __restrict__ part_v, const int32_t* __restrict__ part_i,
                                    int32_t* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  ArgMax a;
  a.v = part_v[blockIdx.x * kArgmaxChunks + threadIdx.x];
  a.i = part_i[blockIdx.x * kArgmaxChunks + threadIdx.x];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = better(a, b);
  }
  if (threadIdx.x == 0) out[blockIdx.x] = a.i < 0 ? 0 : a.i;
}

// scratch: n_rows * 32 floats followed by n_rows * 32 int32 for rows wider than 16384 (may be null
// for narrower rows, which one block per row handles).
YALIS_API int yalis_argmax(const float* logits, long long row_stride, int n_rows, int vocab, int32_t* out,
                           float* scratch, cudaStream_t stream) {
  static_assert(kArgmaxChunks == 32, "the merge kernel is one warp wide");
  if (n_rows <= 0) return YALIS_OK;
  if (vocab <= 0) return YALIS_ERR_SHAPE;
  if (vocab <= 16384 || scratch == nullptr)
    return yalis_launch(argmax_kernel, dim3(n_rows), dim3(kThreads), 0, stream, logits, row_stride, vocab, out);
  float* part_v = scratch;
  int32_t* part_i = reinterpret_cast<int32_t*>(scratch + (size_t)n_rows * kArgmaxChunks);
  int st = yalis_launch(argmax_partial_kernel, dim3(n_rows, kArgmaxChunks), dim3(kThreads), 0, stream, logits,
                        row_stride, vocab, part_v, part_i);
  if (st != YALIS_OK) return st;
  return yalis_launch(argmax_merge_kernel, dim3(n_rows), dim3(32), 0, stream, (const float*)part_v,
                      (const int32_t*)part_i, out);
}

YALIS_API int yalis_sample(const float* logits, long long row_stride, int n_rows, int vocab, const float* temperature,
                           const int32_t* top_k, const float* top_p, const unsigned long long* seed,
                           const unsigned long long* draw_index, int32_t* out, cudaStream_t stream) {
  if (n_rows <= 0) return YALIS_OK;
  if (vocab <= 0) return YALIS_ERR_SHAPE;
  return yalis_launch(sample_kernel, dim3(n_rows), dim3(kThreads), 0, stream, logits, row_stride, vocab, temperature,
                      top_k, top_p, seed, draw_index, out);
}
