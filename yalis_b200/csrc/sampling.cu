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
// descent over order-preserving 32-bit keys (digits of 12, 12 and 8 bits; one
// block per row, or a cluster of eight blocks for a wide row, whose histograms
// the leading block adds through distributed shared memory; the wide first digit
// spreads the entries over enough bins that shared-memory atomics rarely collide).  Bin masses are accumulated as 64-bit fixed point, so
// every sum is exact in its order and the result is deterministic.  Entries
// tied with the k-th value are all kept; entries tied with the top-p boundary
// value are all dropped (unless that value is the maximum).  The draw itself is
// an argmax of perturbed logits and runs on 32 blocks per row with a merge, as
// the plain argmax does for wide rows.
#include "common.cuh"

#include <type_traits>

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

// Calls f(value, index) for every entry of row[0, n) that this thread owns, with many loads in
// flight at once: one block walking a wide row is bound by load latency otherwise.  Which thread
// sees which entry is unspecified; every entry is seen exactly once by the block.
template <class F>
__device__ __forceinline__ void for_each_entry(const float* __restrict__ row, int n, F f) {
  const int step = blockDim.x;
  int done = 0;
  if ((reinterpret_cast<uintptr_t>(row) & 15u) == 0) {
    const float4* __restrict__ row4 = reinterpret_cast<const float4*>(row);
    const int n4 = n >> 2;
    constexpr int U = 4;
    int i = threadIdx.x;
    for (; i + (U - 1) * step < n4; i += U * step) {
      float4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = row4[i + u * step];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int at = 4 * (i + u * step);
        f(v[u].x, at);
        f(v[u].y, at + 1);
        f(v[u].z, at + 2);
        f(v[u].w, at + 3);
      }
    }
    for (; i < n4; i += step) {
      const float4 v = row4[i];
      f(v.x, 4 * i);
      f(v.y, 4 * i + 1);
      f(v.z, 4 * i + 2);
      f(v.w, 4 * i + 3);
    }
    done = n4 << 2;
  }
  for (int i = done + threadIdx.x; i < n; i += step) f(row[i], i);
}

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

// A chosen token goes to out[row] and, when `scatter_index` is given and not negative for the row, also to
// scatter[scatter_index[row]]: the engine keeps each request's last chosen token in a per-slot array on the
// device, from which the next step can take its input without the host in between.
__device__ __forceinline__ void put_choice(int row, int token, int32_t* __restrict__ out,
                                           const int32_t* __restrict__ scatter_index, int32_t* __restrict__ scatter) {
  out[row] = token;
  if (scatter_index != nullptr) {
    const int where = scatter_index[row];
    if (where >= 0) scatter[where] = token;
  }
}

__global__ void __launch_bounds__(kThreads) argmax_kernel(const float* __restrict__ logits, long long row_stride,
                                                          int vocab, int32_t* __restrict__ out,
                                                          const int32_t* __restrict__ scatter_index,
                                                          int32_t* __restrict__ scatter) {
  __shared__ ArgMax scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const float* row = logits + (size_t)blockIdx.x * row_stride;
  ArgMax a;
  a.v = 0.f;
  a.i = -1;
  for_each_entry(row, vocab, [&](float v, int i) {
    ArgMax b;
    b.v = v;
    b.i = i;
    if (v == v) a = better(a, b);  // NaN never wins
  });
  a = block_argmax(a, scratch);
  if (threadIdx.x == 0) put_choice(blockIdx.x, a.i < 0 ? 0 : a.i, out, scatter_index, scatter);
}

constexpr double kFixedOne = 549755813888.0;  // 2^39
constexpr float kFixedOneF = 549755813888.0f;  // the same in float32: a power of two, the product is exact

// Per-row result of the threshold search: which entries survive top-k and top-p.
struct Cut {
  uint32_t k_key;       // keep order_key >= k_key
  uint32_t p_key;       // and order_key > p_key ...
  uint32_t keep_equal;  // ... or == p_key if this is 1
  uint32_t use_p;       // 0: no top-p cut
};

constexpr int kBins = 4096;            // bins of the first two passes (12 bits each); the third has 256

// Width and shift of the three digits of a 32-bit key: 12 + 12 + 8 bits, most significant first.
__device__ __forceinline__ int digit_bits(int pass) { return pass < 2 ? 12 : 8; }
__device__ __forceinline__ int digit_shift(int pass) { return pass == 0 ? 20 : pass == 1 ? 8 : 0; }

// Exclusive prefix sum over the block's threads (in thread order) of 64-bit values.
__device__ unsigned long long block_exclusive_scan(unsigned long long v, unsigned long long* warp_totals) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  unsigned long long inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();
  if (lane == 31) warp_totals[warp] = inc;
  __syncthreads();
  unsigned long long base = 0;
  for (int w = 0; w < warp; ++w) base += warp_totals[w];
  (void)nwarps;
  return base + inc - v;
}

// Walks the bins from the highest down and finds the first one at which `above` + the bins so
// far exceeds `limit`.  Returns the bin (or -1 if the total never exceeds it) in *chosen and the
// sum of the bins above it in *above_out; every thread gets the same answer.
__device__ void find_crossing(const unsigned long long* hist, int nb, unsigned long long above, unsigned long long limit,
                              unsigned long long* warp_totals, int* sh_pick, unsigned long long* sh_above_pick,
                              int* chosen, unsigned long long* above_out) {
  const int per = (nb + blockDim.x - 1) / blockDim.x;          // bins per thread, walked downwards
  const int first = nb - 1 - threadIdx.x * per;                 // this thread's highest bin
  unsigned long long mine = 0;
  for (int j = 0; j < per; ++j) {
    const int b = first - j;
    if (b >= 0) mine += hist[b];
  }
  if (threadIdx.x == 0) *sh_pick = 0x7fffffff;
  const unsigned long long before = above + block_exclusive_scan(mine, warp_totals);   // includes a __syncthreads
  unsigned long long run = before;
  for (int j = 0; j < per; ++j) {
    const int b = first - j;
    if (b < 0) break;
    if (run + hist[b] > limit) {
      atomicMin(sh_pick, threadIdx.x * per + j);                // position in walking order
      break;
    }
    run += hist[b];
  }
  __syncthreads();
  const int pick = *sh_pick;
  if (pick != 0x7fffffff && pick / per == (int)threadIdx.x) *sh_above_pick = run;   // the owner of the first crossing
  __syncthreads();
  if (pick == 0x7fffffff) {
    *chosen = -1;
    *above_out = above;
  } else {
    *chosen = nb - 1 - pick;
    *above_out = *sh_above_pick;
  }
  __syncthreads();
}

// ---- thread-block cluster helpers: the blocks of one row read each other's shared memory ----
__device__ __forceinline__ uint32_t smem_addr_of(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t map_to_block(uint32_t saddr, int rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ uint32_t ld_cluster_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_cluster_u64(uint32_t addr, unsigned long long v) {
  asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_cluster_u64(uint32_t addr) {
  unsigned long long v;
  asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(addr) : "memory");
  return v;
}
// Barrier over the CL blocks of a row (release/acquire: shared-memory writes before it are visible
// to the other blocks after it); over the block alone when CL is 1.
template <int CL>
__device__ __forceinline__ void row_sync() {
  if constexpr (CL > 1)
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  else
    __syncthreads();
}

// What the leading block found in a pass, read by the other blocks of the row.
struct Found {
  int chosen;
  int pad;
  unsigned long long above;
};

// The top-k and top-p cuts of the rows that ask for one.  A row is walked by CL blocks (one
// thread-block cluster, CL == 1: one block): each builds the histogram of its slice in its own
// shared memory, the leading block adds the slices' bins through distributed shared memory, finds
// the crossing and publishes it.  Integer bins make the result independent of CL; the softmax
// normaliser is summed block by block in rank order.
template <int CL>
__global__ void __launch_bounds__(kThreads)
sample_cut_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
                  const float* __restrict__ temperature, const int32_t* __restrict__ top_k,
                  const float* __restrict__ top_p, Cut* __restrict__ cuts) {
  extern __shared__ unsigned long long hist[];          // [kBins] 64-bit bins (leading block), then [3][kBins] 32-bit pieces
  __shared__ float fscratch[32];
  __shared__ unsigned long long warp_totals[32];
  __shared__ int sh_pick;
  __shared__ unsigned long long sh_above_pick;
  __shared__ float exchange[2];                          // this block's maximum and sum
  __shared__ Found found;
  pdl_launch_dependents();
  pdl_wait();

  const int r = blockIdx.y;
  const int rank = CL > 1 ? (int)blockIdx.x : 0;        // clusters are (CL, 1, 1) and the grid is (CL, rows)
  const float temp = temperature[r];
  const float tp = top_p[r];
  const int tk = top_k[r];
  const bool greedy = !(temp > 0.f) && !(tp > 0.f);
  const bool want_k = tk > 0 && tk < vocab, want_p = tp < 1.0f;
  if (greedy || (!want_k && !want_p)) {                  // the same decision in every block of the row
    if (rank == 0 && threadIdx.x == 0) cuts[r] = Cut{0u, 0u, 1u, 0u};
    return;
  }
  // This block's slice of the row; a multiple of four entries keeps the 16-byte loads.
  const int per = (((vocab + CL - 1) / CL) + 3) & ~3;
  const int lo = min(vocab, rank * per);
  const int n = min(vocab, lo + per) - lo;
  const float* row = logits + (size_t)r * row_stride + lo;
  unsigned int* pieces = reinterpret_cast<unsigned int*>(hist + kBins);   // [3][kBins], piece 0 doubles as counts
  const uint32_t pieces_addr = smem_addr_of(pieces);

  // hist[b] of the leading block = sum over the row's blocks of their pieces (13 bits apart).  Each
  // block adds its share of the bins, all loads of a bin in flight at once, and stores the sums
  // into the leading block's shared memory.
  const uint32_t hist_addr = smem_addr_of(hist);
  auto gather = [&](int nb, auto n_pieces) {
    constexpr int NP = decltype(n_pieces)::value;
    row_sync<CL>();                                      // every block's pieces are complete
    if constexpr (CL == 1) {
      for (int b = threadIdx.x; b < nb; b += blockDim.x) {
        unsigned long long s = 0;
#pragma unroll
        for (int p = 0; p < NP; ++p) s += (unsigned long long)pieces[p * kBins + b] << (13 * p);
        hist[b] = s;
      }
      __syncthreads();
    } else {
      const int share = nb / CL;                         // nb is 4096 or 256, CL a power of two up to 8
      for (int j = threadIdx.x; j < share; j += blockDim.x) {
        const int b = rank * share + j;
        unsigned int v[CL][NP];
#pragma unroll
        for (int c = 0; c < CL; ++c)
#pragma unroll
          for (int p = 0; p < NP; ++p) v[c][p] = ld_cluster_u32(map_to_block(pieces_addr + 4u * (uint32_t)(p * kBins + b), c));
        unsigned long long s = 0;
#pragma unroll
        for (int c = 0; c < CL; ++c)
#pragma unroll
          for (int p = 0; p < NP; ++p) s += (unsigned long long)v[c][p] << (13 * p);
        st_cluster_u64(map_to_block(hist_addr + 8u * (uint32_t)b, 0), s);
      }
      row_sync<CL>();                                    // the leading block's bins are complete
    }
  };
  // The crossing of the gathered bins, known to every thread of every block of the row afterwards.
  auto crossing = [&](int nb, unsigned long long above_in, unsigned long long limit, int* chosen,
                      unsigned long long* above_out) {
    if (rank == 0) {
      find_crossing(hist, nb, above_in, limit, warp_totals, &sh_pick, &sh_above_pick, chosen, above_out);
      if (CL > 1 && threadIdx.x == 0) {
        found.chosen = *chosen;
        found.above = *above_out;
      }
    }
    if constexpr (CL > 1) {
      row_sync<CL>();
      const uint32_t at = map_to_block(smem_addr_of(&found), 0);
      *chosen = (int)ld_cluster_u32(at);
      *above_out = ld_cluster_u64(at + 8);
    }
  };
  // ---- top-k: key of the k-th largest logit ---------------------------------------
  uint32_t k_key = 0;
  if (want_k) {
    uint32_t prefix = 0;
    unsigned long long remaining = (unsigned long long)tk;
    int done_bits = 0;
    for (int pass = 0; pass < 3; ++pass) {
      const int nb = 1 << digit_bits(pass), shift = digit_shift(pass);
      unsigned int* counts = pieces;                     // a count fits 32 bits: native shared atomics
      for (int b = threadIdx.x; b < nb; b += blockDim.x) counts[b] = 0;
      __syncthreads();
      for_each_entry(row, n, [&](float v, int) {
        const uint32_t key = order_key(v);
        if (done_bits == 0 || (key >> (32 - done_bits)) == (prefix >> (32 - done_bits)))
          atomicAdd(&counts[(key >> shift) & (nb - 1)], 1u);
      });
      gather(nb, std::integral_constant<int, 1>{});
      int chosen;
      unsigned long long above;
      crossing(nb, 0ull, remaining - 1, &chosen, &above);
      if (chosen < 0) chosen = 0;                        // cannot happen: k < vocab entries exist
      remaining -= above;
      prefix |= (uint32_t)chosen << shift;
      done_bits += digit_bits(pass);
    }
    k_key = prefix;
  }

  uint32_t p_key = 0;
  uint32_t keep_equal = 1;
  if (want_p) {
    // ---- scale, max and normaliser over the entries that survive top-k ---------------
    const float inv_t = temp > 0.f ? 1.0f / temp : 1.0f;
    // One walk: every thread keeps a running maximum and the sum of exponentials relative to it.
    float mx = -INFINITY, z = 0.f;
    for_each_entry(row, n, [&](float v, int) {
      if (order_key(v) >= k_key && v == v) {
        if (v > mx) {
          z = z * expf((mx - v) * inv_t) + 1.0f;         // mx == -inf: z is 0 and stays finite
          mx = v;
        } else {
          z += expf((v - mx) * inv_t);
        }
      }
    });
    const float mine = mx;
    mx = block_max(mx, fscratch);
    z = block_sum(mine == -INFINITY ? 0.f : z * expf((mine - mx) * inv_t), fscratch);
    if constexpr (CL > 1) {
      // The blocks' (maximum, sum) pairs, combined in rank order by every thread alike.
      if (threadIdx.x == 0) {
        exchange[0] = mx;
        exchange[1] = z;
      }
      row_sync<CL>();
      const uint32_t at = smem_addr_of(exchange);
      float m_c[CL], z_c[CL];
#pragma unroll
      for (int c = 0; c < CL; ++c) {
        m_c[c] = __uint_as_float(ld_cluster_u32(map_to_block(at, c)));
        z_c[c] = __uint_as_float(ld_cluster_u32(map_to_block(at + 4, c)));
      }
      mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < CL; ++c) mx = fmaxf(mx, m_c[c]);
      z = 0.f;
#pragma unroll
      for (int c = 0; c < CL; ++c) z += m_c[c] == -INFINITY ? 0.f : z_c[c] * expf((m_c[c] - mx) * inv_t);
    }
    const float inv_z = 1.0f / z;
    // ---- top-p: the key at which the cumulative probability passes top_p ---------------
    const unsigned long long limit = (unsigned long long)((double)tp * kFixedOne);
    uint32_t prefix = 0;
    unsigned long long above = 0;
    int done_bits = 0;
    bool all_fit = false;
    for (int pass = 0; pass < 3 && !all_fit; ++pass) {
      const int nb = 1 << digit_bits(pass), shift = digit_shift(pass);
      // A probability is a 39-bit fixed-point mass; it is added as three 13-bit pieces with native
      // 32-bit shared atomics (64-bit ones are compare-and-swap loops, slow where bins are hot).
      // A piece sum stays under 2^32 for rows of up to 2^19 entries.
      for (int b = threadIdx.x; b < nb; b += blockDim.x) pieces[b] = pieces[kBins + b] = pieces[2 * kBins + b] = 0;
      __syncthreads();
      for_each_entry(row, n, [&](float v, int) {
        const uint32_t key = order_key(v);
        if (key < k_key || v != v) return;
        if (done_bits == 0 || (key >> (32 - done_bits)) == (prefix >> (32 - done_bits))) {
          const unsigned long long mass = __float2ull_rz(expf((v - mx) * inv_t) * inv_z * kFixedOneF);
          const int b = (key >> shift) & (nb - 1);
          if (mass & 0x1fffull) atomicAdd(&pieces[b], (unsigned int)(mass & 0x1fffull));
          if ((mass >> 13) & 0x1fffull) atomicAdd(&pieces[kBins + b], (unsigned int)((mass >> 13) & 0x1fffull));
          if (mass >> 26) atomicAdd(&pieces[2 * kBins + b], (unsigned int)(mass >> 26));
        }
      });
      gather(nb, std::integral_constant<int, 3>{});
      int chosen;
      unsigned long long new_above;
      crossing(nb, above, limit, &chosen, &new_above);
      if (chosen < 0) {
        // Only possible in the first pass (later passes split a bin whose mass is already known
        // to cross the limit, and the fixed-point masses add up exactly): the whole row fits
        // under top_p, nothing is dropped.
        all_fit = true;
        prefix = 0;
      } else {
        above = new_above;
        prefix |= (uint32_t)chosen << shift;
        done_bits += digit_bits(pass);
      }
    }
    p_key = prefix;
    // Either nothing is dropped (p_key 0, equal kept), or p_key is the exact key whose entries
    // carry the sum past top_p: they are dropped unless nothing lies above them (the first
    // entry is always kept).
    keep_equal = all_fit ? 1u : (above == 0 ? 1u : 0u);
  }
  if (rank == 0 && threadIdx.x == 0) cuts[r] = Cut{k_key, p_key, keep_equal, want_p ? 1u : 0u};
  // No block leaves while another may still read its shared memory.
  if constexpr (CL > 1) row_sync<CL>();
}

// The draw, spread over kChunks blocks per row: each finds the best perturbed logit of its slice
// among the entries the cut keeps (greedy rows: the plain maximum); a second kernel merges.
// argmax_i (l_i / T + Gumbel_i) needs neither the maximum nor the normaliser.
constexpr int kDrawChunks = 32;

__global__ void __launch_bounds__(kThreads)
sample_draw_partial_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
                           const float* __restrict__ temperature, const float* __restrict__ top_p,
                           const unsigned long long* __restrict__ seed,
                           const unsigned long long* __restrict__ draw_index, const Cut* __restrict__ cuts,
                           float* __restrict__ part_v, int32_t* __restrict__ part_i) {
  __shared__ ArgMax scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  const float temp = temperature[r];
  const bool greedy = !(temp > 0.f) && !(top_p[r] > 0.f);
  const float inv_t = temp > 0.f ? 1.0f / temp : 1.0f;
  const Cut cut = cuts[r];
  const unsigned long long sd = seed[r], ctr = draw_index[r];
  const uint2 key2 = make_uint2((uint32_t)sd, (uint32_t)(sd >> 32));
  const int per = (vocab + kDrawChunks - 1) / kDrawChunks;
  const int lo = blockIdx.y * per, hi = min(vocab, lo + per);
  ArgMax a;
  a.v = 0.f;
  a.i = -1;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = row[i];
    if (v != v) continue;
    ArgMax b;
    b.i = i;
    if (greedy) {
      b.v = v;
    } else {
      const uint32_t key = order_key(v);
      if (key < cut.k_key) continue;
      if (cut.use_p && !(key > cut.p_key || (cut.keep_equal && key == cut.p_key))) continue;
      const uint4 rnd = philox4x32(make_uint4((uint32_t)i, (uint32_t)ctr, (uint32_t)(ctr >> 32), 0x59414c49u), key2);
      b.v = v * inv_t - logf(-logf(uniform_open(rnd.x)));     // log p_i - log e_i, up to a constant
    }
    a = better(a, b);
  }
  a = block_argmax(a, scratch);
  if (threadIdx.x == 0) {
    part_v[r * kDrawChunks + blockIdx.y] = a.v;
    part_i[r * kDrawChunks + blockIdx.y] = a.i;
  }
}

}  // namespace

constexpr int kArgmaxChunks = 32;   // blocks per row in the first phase for wide rows
constexpr int kCutBlocks = 8;       // most blocks per row of the cut search (one portable cluster)
constexpr int kCutClusterVocab = 16384;

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
                                    int32_t* __restrict__ out, const int32_t* __restrict__ scatter_index,
                                    int32_t* __restrict__ scatter) {
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
  if (threadIdx.x == 0) put_choice(blockIdx.x, a.i < 0 ? 0 : a.i, out, scatter_index, scatter);
}

// scratch: n_rows * 32 floats followed by n_rows * 32 int32 for rows wider than 16384 (may be null
// for narrower rows, which one block per row handles).
// scatter_index / scatter: see put_choice (both may be null).
YALIS_API int yalis_argmax(const float* logits, long long row_stride, int n_rows, int vocab, int32_t* out,
                           float* scratch, const int32_t* scatter_index, int32_t* scatter, cudaStream_t stream) {
  static_assert(kArgmaxChunks == 32, "the merge kernel is one warp wide");
  if (n_rows <= 0) return YALIS_OK;
  if (vocab <= 0) return YALIS_ERR_SHAPE;
  if (vocab <= 16384 || scratch == nullptr)
    return yalis_launch(argmax_kernel, dim3(n_rows), dim3(kThreads), 0, stream, logits, row_stride, vocab, out,
                        scatter_index, scatter);
  float* part_v = scratch;
  int32_t* part_i = reinterpret_cast<int32_t*>(scratch + (size_t)n_rows * kArgmaxChunks);
  int st = yalis_launch(argmax_partial_kernel, dim3(n_rows, kArgmaxChunks), dim3(kThreads), 0, stream, logits,
                        row_stride, vocab, part_v, part_i);
  if (st != YALIS_OK) return st;
  return yalis_launch(argmax_merge_kernel, dim3(n_rows), dim3(32), 0, stream, (const float*)part_v,
                      (const int32_t*)part_i, out, scatter_index, scatter);
}

// scratch: n_rows * (64 + 4) 32-bit words (partial results of the draw, then the cuts).
YALIS_API int yalis_sample(const float* logits, long long row_stride, int n_rows, int vocab, const float* temperature,
                           const int32_t* top_k, const float* top_p, const unsigned long long* seed,
                           const unsigned long long* draw_index, int32_t* out, float* scratch,
                           const int32_t* scatter_index, int32_t* scatter, cudaStream_t stream) {
  static_assert(kDrawChunks == kArgmaxChunks, "the merge kernel is shared with argmax");
  if (n_rows <= 0) return YALIS_OK;
  if (vocab <= 0 || vocab > (1 << 19) || scratch == nullptr) return YALIS_ERR_SHAPE;   // see the piece sums of top-p
  float* part_v = scratch;
  int32_t* part_i = reinterpret_cast<int32_t*>(scratch + (size_t)n_rows * kDrawChunks);
  Cut* cuts = reinterpret_cast<Cut*>(scratch + (size_t)n_rows * 2 * kDrawChunks);
  const size_t smem = (size_t)kBins * (sizeof(unsigned long long) + 3 * sizeof(unsigned int));
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0, sms = 0;
    const int bytes = (int)smem;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0 ||
        cudaFuncSetAttribute(sample_cut_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess ||
        cudaFuncSetAttribute(sample_cut_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess ||
        cudaFuncSetAttribute(sample_cut_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess ||
        cudaFuncSetAttribute(sample_cut_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
      return YALIS_ERR_LAUNCH;
    sm_count = sms;
  }
  // A wide row is walked by a cluster of blocks, the more the fewer rows there are: one block per
  // multiprocessor at most, since every pass ends in barriers over the cluster.
  int blocks = 1;
  if (vocab >= kCutClusterVocab)
    while (blocks < kCutBlocks && (long long)n_rows * (2 * blocks) <= sm_count) blocks *= 2;
  const dim3 grid(blocks, n_rows), block(kThreads), cluster(blocks, 1, 1);
  int st;
  if (blocks == 8)
    st = yalis_launch_cluster(sample_cut_kernel<8>, grid, block, cluster, smem, stream, logits, row_stride, vocab, temperature,
                              top_k, top_p, cuts);
  else if (blocks == 4)
    st = yalis_launch_cluster(sample_cut_kernel<4>, grid, block, cluster, smem, stream, logits, row_stride, vocab, temperature,
                              top_k, top_p, cuts);
  else if (blocks == 2)
    st = yalis_launch_cluster(sample_cut_kernel<2>, grid, block, cluster, smem, stream, logits, row_stride, vocab, temperature,
                              top_k, top_p, cuts);
  else
    st = yalis_launch(sample_cut_kernel<1>, grid, block, smem, stream, logits, row_stride, vocab, temperature, top_k, top_p,
                      cuts);
  if (st != YALIS_OK) return st;
  st = yalis_launch(sample_draw_partial_kernel, dim3(n_rows, kDrawChunks), dim3(kThreads), 0, stream, logits, row_stride,
                    vocab, temperature, top_p, seed, draw_index, (const Cut*)cuts, part_v, part_i);
  if (st != YALIS_OK) return st;
  return yalis_launch(argmax_merge_kernel, dim3(n_rows), dim3(32), 0, stream, (const float*)part_v,
                      (const int32_t*)part_i, out, scatter_index, scatter);
}
