// Decode attention with TMA-fed key/value tiles: one query token per request, the keys of a
// (request, KV head) divided among `n_splits` blocks.
//
// It computes what paged_attention_mma_kernel<HS, true> computes (attention_mma.cu); what differs
// is how K and V reach shared memory and how the splits are merged.
//   * There every thread computes page addresses and issues 16-byte cp.async copies, which made
//     the kernel instruction-bound.  Here a producer warp walks the block table and issues one TMA
//     box copy per (page, 64-column half) for K and for V (cp.async.bulk.tensor.2d over the pool
//     seen as a matrix [pages*kv_heads*page_size, head_dim], 128-byte swizzle; the lanes share
//     the copies of a tile), completion is counted by an mbarrier per stage, and the four consumer
//     warps only wait, run ldmatrix on the swizzled tiles and mma.sync.  The ring has three stages
//     (two blocks per SM keep six tiles in flight).
//   * Up to 8 splits are launched as one thread-block cluster and merged through distributed
//     shared memory: every block leaves its (max, sum, unnormalised output) in its own shared
//     memory, and after a cluster barrier each block finishes a share of the outputs, summing in
//     split order.  More splits go through global memory with a ticket per (request, KV head).
//   * Tiles that lie wholly below the query's position can be fetched before the preceding
//     kernel has finished (early_fetch; see the entry point for what the caller promises).
//   * Fused mode: the kernel takes the step's QKV projection instead of rotated queries, rotates
//     the queries of its KV head itself and, in the block that owns the query's own position,
//     the new key; that block writes the new key and value to the pools and into its tile.
//
// Limits (the launcher refuses anything else, the caller then uses the cp.async kernel):
// bfloat16, head_dim a multiple of 64 up to 256, page_size 8, 16, 32 or 64, no window, at most
// 16 query heads per KV head, one token per request.
//
// Keys beyond the query's position share the last page with visible ones and may hold anything:
// their scores are masked by index and their V rows are zeroed in shared memory before use.
// Every mbarrier wait is bounded; on a timeout the block raises the error word, drains its
// outstanding copies and returns (it still meets its cluster at both barriers).
#include "decode_tiles.cuh"

namespace {

struct DecParams {
  const __nv_bfloat16* q;      // [N, q_stride]; null when the kernel rotates the queries itself (fused mode)
  int q_stride;
  // Fused mode: the step's fused QKV rows [N, (nh + 2 g) * HS] (bfloat16, or n_parts float32 partial sums that are
  // added in order), rotated here by float(position) * inv_freq (null: no rotation).  The block that owns the tile
  // of the query's own position also rotates the new key, writes it and the new value to the pools (null: the
  // cache belongs to another layer, which has written them) and patches them into its tile.
  const void* qkv;
  int qkv_f32, n_parts, qkv_stride;
  size_t part_stride;
  const float* inv_freq;
  __nv_bfloat16* k_pool_w;
  __nv_bfloat16* v_pool_w;
  __nv_bfloat16* out;          // [N, out_stride]
  int out_stride;
  const int32_t* positions;    // [N]
  const int32_t* q_start;      // [R+1]
  const int32_t* block_table;  // [R, table_width]
  int table_width, page_size, num_pages;
  int nh, g, per;
  float scale_log2;
  int n_splits;
  int cluster_merge;           // 1: the splits of a (request, KV head) are one cluster and merge through shared memory
  int early_fetch;             // 1: keys below the queries' positions and the index arrays are settled (see the entry point)
  float* part_o;               // [N, nh, n_splits, HS]
  float* part_ml;              // [N, nh, n_splits, 2]
  int32_t* tickets;            // [R * g]
  int32_t* error;
};

constexpr int kMaxCluster = 8;    // portable cluster size: the most splits merged through shared memory
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, int rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ float2 ld_cluster_f2(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
template <int HS>
__global__ void __launch_bounds__(kThreads)
decode_attention_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const DecParams p) {
  constexpr int H2 = HS / 64;                  // 64-column halves of a row
  constexpr int TILE_BYTES = BN * HS * 2;      // one K (or V) tile
  constexpr int LDQ = HS + 8;                  // padded Q rows
  constexpr int KSTEPS = HS / 16, DT = HS / 8;
  constexpr int WKEYS = BN / CWARPS;           // 16 keys of a tile per consumer warp
  static_assert(STAGES * TILE_BYTES >= CWARPS * 16 * HS * 4, "the K ring is reused for the warps' results");
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* k_s = base;                                 // [STAGES][TILE_BYTES]
  unsigned char* v_s = base + STAGES * TILE_BYTES;           // [STAGES][TILE_BYTES]
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(v_s + STAGES * TILE_BYTES);   // [16][LDQ]
  uint64_t* full = reinterpret_cast<uint64_t*>(q_s + 16 * LDQ);
  uint64_t* empty = full + STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + STAGES);
  int* s_last = const_cast<int*>(abort_flag) + 1;
  __nv_bfloat16* kv_new = reinterpret_cast<__nv_bfloat16*>(s_last + 3);   // [2][HS] new key and value (16-byte aligned)
  constexpr int VEC = HS / 4;                  // float4 groups of a row
  // after the tiles: per-warp results in k_s, their (max, sum) in v_s, then the block's merged result
  float* co = reinterpret_cast<float*>(v_s + 1024);          // [16][HS] merged, unnormalised
  float* cml = co + 16 * HS;                                  // [16][2] max and sum

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int req = blockIdx.x / p.g, kvh = blockIdx.x - req * p.g;
  const int split = blockIdx.y;
  const bool is_producer = threadIdx.x == CWARPS * 32;
  if (is_producer) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], CWARPS);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }

  int armed = 0;
  // One tile, issued by the whole producer warp: lane 0 waits for the stage to be free and arms its barrier,
  // then every lane issues its share of the box copies (one per page, 64-column half and K or V: with small
  // pages a single thread would spend longer issuing them than the copies take).
  const int lane_p = threadIdx.x & 31;
  auto issue_tile = [&](int it, int tile_lo, int hi_key, const int32_t* bt) -> bool {
    const int pages_per_tile = BN / p.page_size;
    const uint32_t page_bytes = (uint32_t)p.page_size * HS * 2;
    const int s = it % STAGES;
    const uint32_t ph = (it / STAGES) & 1;
    const int key0 = (tile_lo + it) * BN;
    const int n_pages = min(pages_per_tile, (hi_key - key0) / p.page_size + 1);
    int ok = 1;
    if (lane_p == 0) {
      ok = mbar_wait(&empty[s], ph ^ 1, abort_flag) ? 1 : 0;
      if (ok) mbar_expect_tx(&full[s], 2u * page_bytes * (uint32_t)n_pages);
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (!ok) return false;
    for (int c = lane_p; c < n_pages * 2 * H2; c += 32) {
      const int i = c / (2 * H2), kv = (c / H2) & 1, h = c % H2;
      const int pi = key0 / p.page_size + i;
      int page = pi < p.table_width ? bt[pi] : -1;
      if (page < 0 || page >= p.num_pages) {   // a visible key without a page: a caller's bug
        if (p.error) atomicOr(p.error, YALIS_FLAG_BAD_PAGE);
        page = 0;
      }
      const int y = (page * p.g + kvh) * p.page_size;
      const int off = h * (BN * 128) + i * p.page_size * 128;
      tma_load_2d((kv ? v_s : k_s) + s * TILE_BYTES + off, kv ? &map_v : &map_k, h * 64, y, &full[s]);
    }
    __syncwarp();
    armed = it + 1;
    return true;
  };

  if (p.early_fetch && warp == CWARPS) {
    // Tiles that end below the query's position hold keys of earlier steps only, and the caller
    // promises that the step's index arrays were complete before the preceding kernel began:
    // fetch them while that kernel (which writes this step's key and value) is still running.
    const int tok = p.q_start[req];
    if (p.q_start[req + 1] - tok > 0) {
      const int pos = p.positions[tok];
      const int total = pos / BN + 1;
      const int per_split = (total + p.n_splits - 1) / p.n_splits;
      const int tile_lo = split * per_split;
      const int early = min(min(total - 1, tile_lo + per_split) - tile_lo, STAGES);
      const int32_t* bt = p.block_table + (size_t)req * p.table_width;
      for (int it = 0; it < early; ++it)
        if (!issue_tile(it, tile_lo, pos, bt)) break;
    }
  }
  // Fused mode: the cosines and sines of the query's position do not depend on the preceding kernel either.
  // A thread rotates the pairs e = threadIdx.x + 128 k; their frequency index e % (HS/2) repeats with period 3
  // in k for every head size the kernel takes.
  constexpr int HALF = HS / 2;
  static_assert((3 * CWARPS * 32) % HALF == 0, "frequency indices of a thread repeat with period 3");
  float cs3[3] = {1.f, 1.f, 1.f}, sn3[3] = {0.f, 0.f, 0.f};
  bool trig_ready = false;
  if (p.qkv != nullptr && p.inv_freq != nullptr && p.early_fetch && warp < CWARPS) {
    const int tok_e = p.q_start[req];
    if (p.q_start[req + 1] - tok_e > 0) {
      const float fpos = (float)p.positions[tok_e];
#pragma unroll
      for (int j = 0; j < 3; ++j) sincosf(fpos * p.inv_freq[(threadIdx.x + CWARPS * 32 * j) % HALF], &sn3[j], &cs3[j]);
      trig_ready = true;
    }
  }
  pdl_wait();
  __syncthreads();

  const int tok = p.q_start[req];
  const int n_tok = p.q_start[req + 1] - tok;
  if (n_tok <= 0) return;                      // padding request (uniform for the block; nothing was fetched)
  const int pos = p.positions[tok];
  const int hi_key = pos;
  const int total = hi_key / BN + 1;
  const int per_split = (total + p.n_splits - 1) / p.n_splits;
  const int tile_lo = split * per_split;
  const int tile_hi = min(total, tile_lo + per_split);
  const int n_tiles = max(0, tile_hi - tile_lo);
  const int32_t* bt = p.block_table + (size_t)req * p.table_width;

  if (warp == CWARPS) {
    // ---- producer -------------------------------------------------------------------------
    for (int it = armed; it < n_tiles; ++it)
      if (!issue_tile(it, tile_lo, hi_key, bt)) break;
    if (lane == 0) pdl_launch_dependents();     // the last tile is on its way: the next kernel's blocks may start filling their rings
    __syncwarp();
  } else {
    // ---- consumers ---------------------------------------------------------------------------
    const int gid = lane >> 2, tig = lane & 3;
    const int wkey = warp * WKEYS;
    const int n_rows = p.per;                  // rows = query heads of this KV head
    const bool owns_pos = tile_lo < total && tile_hi == total;     // this block's last tile holds the query's own position
    if (p.qkv == nullptr) {
      constexpr int CHUNKS = HS / 8;
      for (int c = threadIdx.x; c < 16 * CHUNKS; c += CWARPS * 32) {
        const int r = c / CHUNKS, ch = c - r * CHUNKS;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < n_rows)
          v = *reinterpret_cast<const uint4*>(p.q + (size_t)tok * p.q_stride + (size_t)(kvh * p.per + r) * HS + ch * 8);
        *reinterpret_cast<uint4*>(q_s + r * LDQ + ch * 8) = v;
      }
    } else {
      // Rotate this KV head's queries (and, in the owning block, the new key) as the rotary kernel does:
      // partial sums in index order, angle float(pos) * inv_freq, accurate sincosf, one rounding to bfloat16.
      if (p.inv_freq && !trig_ready) {
#pragma unroll
        for (int j = 0; j < 3; ++j)
          sincosf((float)pos * p.inv_freq[(threadIdx.x + CWARPS * 32 * j) % HALF], &sn3[j], &cs3[j]);
      }
      const size_t row0 = (size_t)tok * p.qkv_stride;
      auto load = [&](size_t col) -> float {
        if (p.qkv_f32) return sum_parts<float>(reinterpret_cast<const float*>(p.qkv) + row0 + col, p.n_parts, p.part_stride);
        return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.qkv)[row0 + col]);
      };
      const int n_q = n_rows * HALF;
      const int n_kv = (owns_pos && p.k_pool_w != nullptr) ? 2 * HALF : 0;      // HALF key pairs, then HALF value pairs
      int k3 = 0;                                   // (e - threadIdx.x) / 128 modulo 3
      for (int e = threadIdx.x; e < 16 * HALF + n_kv; e += CWARPS * 32, k3 = k3 == 2 ? 0 : k3 + 1) {
        const float cs = k3 == 0 ? cs3[0] : k3 == 1 ? cs3[1] : cs3[2], sn = k3 == 0 ? sn3[0] : k3 == 1 ? sn3[1] : sn3[2];
        if (e < 16 * HALF) {
          const int r = e / HALF, i = e - r * HALF;
          float o1 = 0.f, o2 = 0.f;
          if (e < n_q) {
            const size_t col = (size_t)(kvh * p.per + r) * HS + i;
            const float x1 = load(col), x2 = load(col + HALF);
            o1 = x1; o2 = x2;
            if (p.inv_freq) rotate_pair(x1, x2, cs, sn, o1, o2);
          }
          q_s[r * LDQ + i] = __float2bfloat16_rn(o1);
          q_s[r * LDQ + i + HALF] = __float2bfloat16_rn(o2);
        } else {
          const int f = e - 16 * HALF;
          const bool is_v = f >= HALF;
          const int i = is_v ? f - HALF : f;
          const size_t col = (size_t)(p.nh + (is_v ? p.g : 0) + kvh) * HS + i;
          const float x1 = load(col), x2 = load(col + HALF);
          float o1 = x1, o2 = x2;
          if (!is_v && p.inv_freq) rotate_pair(x1, x2, cs, sn, o1, o2);
          __nv_bfloat16* dst = kv_new + (is_v ? HS : 0);
          dst[i] = __float2bfloat16_rn(o1);
          dst[i + HALF] = __float2bfloat16_rn(o2);
        }
      }
    }
    consumer_sync();
    if (p.qkv != nullptr && owns_pos && p.k_pool_w != nullptr) {
      // the new key and value go to their place in the cache (16 bytes per thread)
      const int pi = pos / p.page_size;
      int page = pi < p.table_width ? bt[pi] : -1;
      if (page < 0 || page >= p.num_pages) {
        if (threadIdx.x == 0 && p.error) atomicOr(p.error, YALIS_FLAG_BAD_PAGE);
      } else {
        const size_t at = (((size_t)page * p.g + kvh) * p.page_size + (pos - pi * p.page_size)) * HS;
        for (int c = threadIdx.x; c < 2 * (HS / 8); c += CWARPS * 32) {
          const bool is_v = c >= HS / 8;
          const int ch = is_v ? c - HS / 8 : c;
          *reinterpret_cast<uint4*>((is_v ? p.v_pool_w : p.k_pool_w) + at + ch * 8) =
              *reinterpret_cast<const uint4*>(kv_new + (is_v ? HS : 0) + ch * 8);
        }
      }
    }
    unsigned qf[KSTEPS][4];
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
      const int c = ks * 16 + (lane >> 4) * 8;
      ldmatrix_x4(qf[ks], smem_u32(q_s + r * LDQ + c));
    }
    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const bool row_ok[2] = {gid < n_rows, gid + 8 < n_rows};

    bool alive = true;
    for (int it = 0; it < n_tiles && alive; ++it) {
      const int s = it % STAGES;
      const uint32_t ph = (it / STAGES) & 1;
      int ok = 1;
      if (lane == 0) ok = mbar_wait(&full[s], ph, abort_flag) ? 1 : 0;
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) { alive = false; break; }
      const int key0 = (tile_lo + it) * BN;
      const uint32_t kt = smem_u32(k_s + s * TILE_BYTES), vt = smem_u32(v_s + s * TILE_BYTES);
      const bool last = key0 + BN - 1 > hi_key;
      if (p.qkv != nullptr && p.k_pool_w != nullptr && key0 + BN > hi_key) {
        // The tile holds the query's own position: what the copy brought for that row is older than this step
        // (it may have been issued before the row was written).  The warp that owns the row replaces it.
        const int row = hi_key - key0;
        if (row >= wkey && row < wkey + WKEYS) {
          for (int c = lane; c < 2 * (HS / 8); c += 32) {
            const bool is_v = c >= HS / 8;
            const int ch = is_v ? c - HS / 8 : c;
            unsigned char* tile = (is_v ? v_s : k_s) + s * TILE_BYTES;
            *reinterpret_cast<uint4*>(tile + tile_off(row, ch * 8)) = *reinterpret_cast<const uint4*>(kv_new + (is_v ? HS : 0) + ch * 8);
          }
        }
        __syncwarp();
      }
      if (last) {
        // Zero this warp's V rows past the query's position (they may hold anything).
        unsigned char* vrow = v_s + s * TILE_BYTES;
        for (int e = lane; e < WKEYS * (HS / 8); e += 32) {
          const int r = wkey + e / (HS / 8), c = e % (HS / 8);
          if (key0 + r > hi_key) *reinterpret_cast<uint4*>(vrow + tile_off(r, c * 8)) = make_uint4(0u, 0u, 0u, 0u);
        }
        __syncwarp();
      }
      // S = Q K^T for this warp's 16 keys
      float sc[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        unsigned kb[4];
        const int key = wkey + (lane & 7) + (lane >> 4) * 8;
        const int dim = ks * 16 + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(kb, kt + tile_off(key, dim));
        mma_bf16(sc[0], qf[ks], kb[0], kb[1]);
        mma_bf16(sc[1], qf[ks], kb[2], kb[3]);
      }
      float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1;
          const int key = key0 + wkey + j * 8 + tig * 2 + (e & 1);
          const float v = (row_ok[i] && (!last || key <= hi_key)) ? sc[j][e] * p.scale_log2 : -INFINITY;
          sc[j][e] = v;
          m_new[i] = fmaxf(m_new[i], v);
        }
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
        m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
      }
      float corr[2], bs[2], l_add[2] = {0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        bs[i] = (m_new[i] == -INFINITY) ? 0.f : m_new[i];
        corr[i] = exp2f(m_run[i] - bs[i]);
        m_run[i] = m_new[i];
      }
      unsigned pf[4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float p0 = exp2f(sc[j][0] - bs[0]), p1 = exp2f(sc[j][1] - bs[0]);
        const float p2 = exp2f(sc[j][2] - bs[1]), p3 = exp2f(sc[j][3] - bs[1]);
        l_add[0] += p0 + p1;
        l_add[1] += p2 + p3;
        pf[j * 2 + 0] = pack_bf16(p0, p1);
        pf[j * 2 + 1] = pack_bf16(p2, p3);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * corr[i] + l_add[i];
#pragma unroll
      for (int d = 0; d < DT; ++d) {
        o[d][0] *= corr[0]; o[d][1] *= corr[0];
        o[d][2] *= corr[1]; o[d][3] *= corr[1];
      }
      // O += P V over the warp's 16 keys
#pragma unroll
      for (int d = 0; d < DT; d += 2) {
        unsigned vb[4];
        const int key = wkey + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int dim = d * 8 + (lane >> 4) * 8;
        ldmatrix_x4_trans(vb, vt + tile_off(key, dim));
        mma_bf16(o[d], pf, vb[0], vb[1]);
        mma_bf16(o[d + 1], pf, vb[2], vb[3]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }

    // ---- merge the four warps, write the split's partial or the result ---------------------
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
      l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
    consumer_sync();                                        // all warps are done with the tiles
    float* mo = reinterpret_cast<float*>(k_s);             // [CWARPS][16][HS]
    float* mml = reinterpret_cast<float*>(v_s);            // [CWARPS][16][2]
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = gid + i * 8;
      if (r >= n_rows) continue;                            // padding rows of the 16-row MMA tile are never read
#pragma unroll
      for (int d = 0; d < DT; ++d)
        *reinterpret_cast<float2*>(mo + ((size_t)warp * 16 + r) * HS + d * 8 + tig * 2) = make_float2(o[d][i * 2], o[d][i * 2 + 1]);
      if (tig == 0) {
        mml[(warp * 16 + r) * 2] = m_run[i];
        mml[(warp * 16 + r) * 2 + 1] = l_run[i];
      }
    }
    consumer_sync();
    // The block's result: its four warps merged, four dims per thread.
    for (int e = threadIdx.x; e < n_rows * VEC; e += CWARPS * 32) {
      const int r = e / VEC, d = (e - r * VEC) * 4;
      float mw[CWARPS], mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < CWARPS; ++w) {
        mw[w] = mml[(w * 16 + r) * 2];
        mm = fmaxf(mm, mw[w]);
      }
      float ll = 0.f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < CWARPS; ++w) {
        const float f = (mw[w] == -INFINITY) ? 0.f : exp2f(mw[w] - mm);
        ll += mml[(w * 16 + r) * 2 + 1] * f;
        const float4 v = *reinterpret_cast<const float4*>(mo + ((size_t)w * 16 + r) * HS + d);
        acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
      }
      const int head = kvh * p.per + r;
      if (p.n_splits == 1) {
        store_bf16x4(p.out + (size_t)tok * p.out_stride + (size_t)head * HS + d, acc, ll > 0.f ? 1.0f / ll : 0.f);
      } else if (p.cluster_merge) {
        *reinterpret_cast<float4*>(co + r * HS + d) = acc;
        if (d == 0) *reinterpret_cast<float2*>(cml + r * 2) = make_float2(mm, ll);
      } else {
        const size_t slot = ((size_t)tok * p.nh + head) * p.n_splits + split;
        *reinterpret_cast<float4*>(p.part_o + slot * HS + d) = acc;
        if (d == 0) *reinterpret_cast<float2*>(p.part_ml + slot * 2) = make_float2(mm, ll);
      }
    }
    if (p.n_splits > 1 && !p.cluster_merge) {
      // ---- splits merged through global memory: the last block to arrive does it ------------
      __threadfence();
      consumer_sync();
      if (threadIdx.x == 0) *s_last = (atomicAdd(&p.tickets[blockIdx.x], 1) == p.n_splits - 1) ? 1 : 0;
      consumer_sync();
      if (*s_last) {
        __threadfence();
        // The other splits' results were written by other blocks: read them past the L1 (ld.global.cg),
        // many loads in flight at once.  First the (max, sum) pairs of every (row, split) into shared
        // memory, turned into the weight of each split; then the weighted sum over splits, in split order.
        const int ns = p.n_splits;
        float* w_s = reinterpret_cast<float*>(k_s);            // [n_rows][ns] max, then weight
        float* l_s = w_s + 16 * 64;                             // [n_rows][ns] sums
        float* inv_s = l_s + 16 * 64;                           // [n_rows] 1 / total
        for (int e = threadIdx.x; e < n_rows * ns; e += CWARPS * 32) {
          const int r = e / ns, sp = e - r * ns;
          const size_t slot = ((size_t)tok * p.nh + kvh * p.per + r) * ns + sp;
          const float2 v = __ldcg(reinterpret_cast<const float2*>(p.part_ml + slot * 2));
          w_s[e] = v.x;
          l_s[e] = v.y;
        }
        consumer_sync();
        if (threadIdx.x < n_rows) {
          const int r = threadIdx.x;
          float mm = -INFINITY;
          for (int sp = 0; sp < ns; ++sp) mm = fmaxf(mm, w_s[r * ns + sp]);
          float ll = 0.f;
          for (int sp = 0; sp < ns; ++sp) {
            const float m = w_s[r * ns + sp];
            const float f = (m == -INFINITY) ? 0.f : exp2f(m - mm);
            w_s[r * ns + sp] = f;
            ll += l_s[r * ns + sp] * f;
          }
          inv_s[r] = ll > 0.f ? 1.0f / ll : 0.f;
        }
        consumer_sync();
        for (int e = threadIdx.x; e < n_rows * VEC; e += CWARPS * 32) {
          const int r = e / VEC, d = (e - r * VEC) * 4;
          const int head = kvh * p.per + r;
          const float* po = p.part_o + ((size_t)tok * p.nh + head) * ns * HS + d;
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int sp0 = 0; sp0 < ns; sp0 += 8) {
            float4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              v[j] = sp0 + j < ns ? __ldcg(reinterpret_cast<const float4*>(po + (size_t)(sp0 + j) * HS)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (sp0 + j < ns) {
                const float f = w_s[r * ns + sp0 + j];
                acc.x += v[j].x * f; acc.y += v[j].y * f; acc.z += v[j].z * f; acc.w += v[j].w * f;
              }
            }
          }
          store_bf16x4(p.out + (size_t)tok * p.out_stride + (size_t)head * HS + d, acc, inv_s[r]);
        }
        if (threadIdx.x == 0) p.tickets[blockIdx.x] = 0;
      }
    }
  }

  if (p.n_splits > 1 && p.cluster_merge) {
    // ---- splits merged through distributed shared memory: the blocks of a (request, KV head)
    // form one cluster; each reads every block's merged result and finishes its share of the
    // (row, dim) outputs, summing in split order.
    cluster_sync_all();
    if (warp < CWARPS) {
      const int ns = p.n_splits, n_rows = p.per;
      const int n_vec = n_rows * VEC;
      const int chunk = (n_vec + ns - 1) / ns;
      const int lo = split * chunk, hi = min(n_vec, lo + chunk);
      const uint32_t co_a = smem_u32(co), cml_a = smem_u32(cml);
      for (int e = lo + threadIdx.x; e < hi; e += CWARPS * 32) {
        const int r = e / VEC, d = (e - r * VEC) * 4;
        float2 ml[kMaxCluster];
        float mm = -INFINITY;
#pragma unroll
        for (int sp = 0; sp < kMaxCluster; ++sp) {
          ml[sp] = sp < ns ? ld_cluster_f2(map_to_cta(cml_a + (uint32_t)r * 8u, sp)) : make_float2(-INFINITY, 0.f);
          mm = fmaxf(mm, ml[sp].x);
        }
        float4 v[kMaxCluster];
#pragma unroll
        for (int sp = 0; sp < kMaxCluster; ++sp)
          v[sp] = sp < ns ? ld_cluster_f4(map_to_cta(co_a + (uint32_t)(r * HS + d) * 4u, sp)) : make_float4(0.f, 0.f, 0.f, 0.f);
        float ll = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int sp = 0; sp < kMaxCluster; ++sp) {
          const float f = (ml[sp].x == -INFINITY) ? 0.f : exp2f(ml[sp].x - mm);
          ll += ml[sp].y * f;
          acc.x += v[sp].x * f; acc.y += v[sp].y * f; acc.z += v[sp].z * f; acc.w += v[sp].w * f;
        }
        const int head = kvh * p.per + r;
        store_bf16x4(p.out + (size_t)tok * p.out_stride + (size_t)head * HS + d, acc, ll > 0.f ? 1.0f / ll : 0.f);
      }
    }
    cluster_sync_all();                                     // nobody leaves while its memory may still be read
  }

  // ---- exit: on an abort wait (bounded) for copies in flight so none lands after the block ---
  __syncthreads();
  if (*abort_flag && threadIdx.x == CWARPS * 32) {
    if (p.error) atomicOr(p.error, YALIS_FLAG_WAIT_ATTENTION);
    for (int it = max(0, armed - STAGES); it < armed; ++it) {
      const int s = it % STAGES;
      const uint32_t ph = (it / STAGES) & 1;
      for (uint32_t i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(&full[s], ph)) break;
    }
  }
  __syncthreads();
}

template <int HS>
int launch(const CUtensorMap& mk, const CUtensorMap& mv, const DecParams& p, int n_requests, cudaStream_t stream) {
  const size_t smem = 1024 + (size_t)2 * STAGES * BN * HS * 2 + (size_t)16 * (HS + 8) * 2 + 2 * STAGES * 8 + 16 + 32 +
                      (size_t)2 * HS * 2;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(decode_attention_tma_kernel<HS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return YALIS_ERR_LAUNCH;
    configured = true;
  }
  dim3 grid(n_requests * p.g, p.n_splits);
  if (grid.y > 65535) return YALIS_ERR_SHAPE;
  if (p.cluster_merge)
    return yalis_launch_cluster(decode_attention_tma_kernel<HS>, grid, dim3(kThreads), dim3(1, p.n_splits, 1), smem, stream,
                                mk, mv, p);
  return yalis_launch(decode_attention_tma_kernel<HS>, grid, dim3(kThreads), smem, stream, mk, mv, p);
}

}  // namespace

// Whether the TMA decode kernel takes this shape.
YALIS_API int yalis_decode_attention_tma_supports(int hs, int page_size, int per) {
  const bool hs_ok = hs == 64 || hs == 128 || hs == 192 || hs == 256;
  const bool page_ok = page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64;
  return (hs_ok && page_ok && per >= 1 && per <= 16) ? 1 : 0;
}

// One query token per request.  Up to 8 splits are merged through distributed shared memory (the splits of a
// (request, KV head) are launched as one thread-block cluster); more go through global memory and need
// scratch: n_tokens*nh*n_splits*(hs+2) floats and tickets: n_requests*g zeroed int32 (as for
// yalis_paged_attention_mma).  error: device int32 raised on a timed-out wait or
// an unmapped page.
// early_fetch = 1 lets a block fetch the tiles that lie wholly below its query's position before the preceding
// kernel on the stream has finished (programmatic dependent launch).  The caller then promises that those keys and
// values, positions, q_start and the block table were written before the preceding kernel began - true inside a
// model step, where a host copy brings the index arrays and only this step's token is written to the pool.
namespace {
struct FusedArgs {
  const void* qkv = nullptr;
  int qkv_f32 = 0, n_parts = 1, qkv_stride = 0;
  long long part_stride = 0;
  const float* inv_freq = nullptr;
  int store = 0;
};

int decode_attention_tma_impl(const void* q, int q_stride, const FusedArgs& f, void* out, int out_stride, const void* k_pool,
                              const void* v_pool, const int32_t* positions, const int32_t* q_start,
                              const int32_t* block_table, int table_width, int page_size, int num_pages,
                              int n_tokens, int n_requests, int nh, int g, int hs, float scale,
                              int n_splits, int early_fetch, float* scratch, int32_t* tickets,
                              int32_t* error, cudaStream_t stream) {
  if (n_tokens <= 0 || n_requests <= 0) return YALIS_OK;
  if (g <= 0 || nh % g != 0 || n_splits < 1 || n_splits > 64) return YALIS_ERR_SHAPE;   // the merge stages 64 splits
  if (!yalis_decode_attention_tma_supports(hs, page_size, nh / g)) return YALIS_ERR_SHAPE;
  if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15) return YALIS_ERR_ALIGN;
  if ((q_stride % 8) || (out_stride % 4)) return YALIS_ERR_ALIGN;
  if ((q == nullptr) == (f.qkv == nullptr)) return YALIS_ERR_SHAPE;           // queries come one way or the other
  if (f.qkv != nullptr && (f.n_parts < 1 || (!f.qkv_f32 && f.n_parts != 1))) return YALIS_ERR_SHAPE;
  const bool cluster_merge = n_splits > 1 && n_splits <= kMaxCluster;
  if (n_splits > 1 && !cluster_merge && (scratch == nullptr || tickets == nullptr)) return YALIS_ERR_SHAPE;
  CUtensorMap mk, mv;
  const long long rows = (long long)num_pages * g * page_size;
  if (!make_pool_map(&mk, k_pool, rows, hs, page_size) || !make_pool_map(&mv, v_pool, rows, hs, page_size))
    return YALIS_ERR_LAUNCH;
  DecParams p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride;
  p.qkv = f.qkv; p.qkv_f32 = f.qkv_f32; p.n_parts = f.n_parts; p.qkv_stride = f.qkv_stride;
  p.part_stride = (size_t)f.part_stride; p.inv_freq = f.inv_freq;
  p.k_pool_w = f.store ? (__nv_bfloat16*)const_cast<void*>(k_pool) : nullptr;
  p.v_pool_w = f.store ? (__nv_bfloat16*)const_cast<void*>(v_pool) : nullptr;
  p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.positions = positions; p.q_start = q_start; p.block_table = block_table;
  p.table_width = table_width; p.page_size = page_size; p.num_pages = num_pages;
  p.nh = nh; p.g = g; p.per = nh / g;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.n_splits = n_splits;
  p.early_fetch = early_fetch ? 1 : 0;
  p.cluster_merge = cluster_merge ? 1 : 0;
  p.part_o = scratch;
  p.part_ml = scratch ? scratch + (size_t)n_tokens * nh * n_splits * hs : nullptr;
  p.tickets = tickets;
  p.error = error;
  switch (hs) {
    case 64: return launch<64>(mk, mv, p, n_requests, stream);
    case 128: return launch<128>(mk, mv, p, n_requests, stream);
    case 192: return launch<192>(mk, mv, p, n_requests, stream);
    default: return launch<256>(mk, mv, p, n_requests, stream);
  }
}
}  // namespace

YALIS_API int yalis_decode_attention_tma(const void* q, int q_stride, void* out, int out_stride, const void* k_pool,
                                         const void* v_pool, const int32_t* positions, const int32_t* q_start,
                                         const int32_t* block_table, int table_width, int page_size, int num_pages,
                                         int n_tokens, int n_requests, int nh, int g, int hs, float scale,
                                         int n_splits, int early_fetch, float* scratch, int32_t* tickets,
                                         int32_t* error, cudaStream_t stream) {
  return decode_attention_tma_impl(q, q_stride, FusedArgs(), out, out_stride, k_pool, v_pool, positions, q_start,
                                   block_table, table_width, page_size, num_pages, n_tokens, n_requests, nh, g, hs, scale,
                                   n_splits, early_fetch, scratch, tickets, error, stream);
}

// The same with the rotary kernel's work done inside: qkv is the step's fused projection [N, (nh + 2 g) * hs] in
// bfloat16 (qkv_f32 = 0, n_parts = 1) or n_parts float32 partial sums part_stride elements apart; inv_freq
// [hs / 2] float32 or null for no rotation; store = 1 writes the new key and value to the pools (0: the cache
// belongs to another layer that has written them in this step).  Bits of yalis_rope_kv_write followed by
// yalis_decode_attention_tma.
YALIS_API int yalis_decode_attention_tma_fused(const void* qkv, int qkv_f32, int n_parts, long long part_stride,
                                               int qkv_stride, const float* inv_freq, int store, void* out,
                                               int out_stride, void* k_pool, void* v_pool, const int32_t* positions,
                                               const int32_t* q_start, const int32_t* block_table, int table_width,
                                               int page_size, int num_pages, int n_tokens, int n_requests, int nh,
                                               int g, int hs, float scale, int n_splits, int early_fetch,
                                               float* scratch, int32_t* tickets, int32_t* error, cudaStream_t stream) {
  if (qkv == nullptr) return YALIS_ERR_SHAPE;
  if (((uintptr_t)qkv & 15) || (qkv_stride % 8) || (part_stride % 4)) return YALIS_ERR_ALIGN;
  FusedArgs f;
  f.qkv = qkv; f.qkv_f32 = qkv_f32; f.n_parts = n_parts; f.part_stride = part_stride; f.qkv_stride = qkv_stride;
  f.inv_freq = inv_freq; f.store = store;
  return decode_attention_tma_impl(nullptr, 8, f, out, out_stride, k_pool, v_pool, positions, q_start, block_table,
                                   table_width, page_size, num_pages, n_tokens, n_requests, nh, g, hs, scale, n_splits,
                                   early_fetch, scratch, tickets, error, stream);
}
