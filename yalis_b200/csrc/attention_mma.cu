// Paged causal attention on the tensor cores (bfloat16 in, float32 softmax and
// accumulation), one kernel for prompt portions, single decoded tokens and any
// mix of them.
//
// Work is cut by (request, KV head): all query heads that share a KV head and
// all tokens the request brings to this step form the rows of one problem,
// row = token * heads_per_group + head_in_group, so a K/V tile read from the
// cache serves every one of them (for a decode step that is the whole GQA group
// of one token).  A block takes 64 rows (4 warps x 16) and walks the visible
// keys in tiles of 64: K and V tiles are gathered page by page with cp.async
// into padded shared memory (double buffered), S = Q K^T and O += P V run on
// mma.sync.m16n8k16 with ldmatrix operand loads, the online softmax is kept in
// registers in the exp2 domain.  The mask is by absolute position: the row of a
// token at position p sees keys j with p - window < j <= p
// (yalis/attention/backend_impl/sdpa_and_flex.py:15-19, 301-307).
//
// When a (request, KV head) has at most 16 rows (a decode step: one token, up to 16 heads per
// group) the four warps do not own rows: all work on the same 16 rows and each takes a
// quarter of every key tile, and their four partial softmax states are merged through
// shared memory at the end.
//
// With n_splits > 1 (decode steps of few requests) the keys of a request are
// divided among blocks; each writes an unnormalised partial result with its
// running maximum and sum to scratch memory and takes a ticket from a counter of
// its (request, KV head); the block that draws the last ticket merges all splits
// in index order (so the result does not depend on which block came last) and
// resets the counter for the next launch.
#include "common.cuh"

namespace {

constexpr int BM = 64;   // rows per block
constexpr int BN = 64;   // keys per tile
constexpr int NWARPS = 4;

struct AttnParams {
  const __nv_bfloat16* q;      // [N, q_stride], head h at column h*HS
  int q_stride;
  __nv_bfloat16* out;          // [N, out_stride]
  int out_stride;
  const __nv_bfloat16* k_pool; // [pages, g, page_size, HS]
  const __nv_bfloat16* v_pool;
  const int32_t* positions;    // [N]
  const int32_t* q_start;      // [R+1]
  const int32_t* block_table;  // [R, table_width]
  int table_width, page_size, num_pages;
  int page_shift;              // log2(page_size) if it is a power of two, else -1
  int nh, g, per;              // per = nh / g
  float scale_log2;            // scale * log2(e)
  int window;                  // 0: none
  int n_splits;
  float* part_o;               // [N, nh, n_splits, HS] (split mode)
  float* part_ml;              // [N, nh, n_splits, 2]
  int32_t* tickets;            // [R * g] zero before the launch and zero again after it (split mode)
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// Gathers keys [key0, key0 + BN) of one KV head into two [BN][HS + 8] tiles (K and V); rows
// outside [lo_key, hi_key] or on an unmapped page are zero-filled.  Consecutive threads copy
// consecutive 16-byte chunks of a row (coalesced); all page lookups of a thread are done
// before its first copy is issued, so that they overlap.
template <int HS>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* k_dst, __nv_bfloat16* v_dst, const int32_t* bt,
                                             const AttnParams& p, int kvh, int key0, int lo_key, int hi_key) {
  constexpr int CHUNKS = HS / 8;                          // 16-byte chunks per row
  constexpr int LD = HS + 8;
  constexpr int ITERS = BN * CHUNKS / (NWARPS * 32);      // chunks per thread (HS % 16 == 0 makes it whole)
  static_assert(BN * CHUNKS % (NWARPS * 32) == 0, "tile chunks must divide among the threads");
  long long src[ITERS];
  const int head_stride = p.page_size * HS;               // elements of one (page, kv head) block
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    const int c = threadIdx.x + i * (NWARPS * 32);
    const int row = c / CHUNKS, ch = c - row * CHUNKS;
    const int key = key0 + row;
    src[i] = -1;
    if (key >= lo_key && key <= hi_key) {
      const int pi = p.page_shift >= 0 ? (key >> p.page_shift) : (key / p.page_size);
      const int page = pi < p.table_width ? bt[pi] : -1;
      if (page >= 0 && page < p.num_pages)
        src[i] = (long long)(page * p.g + kvh) * head_stride + (key - pi * p.page_size) * HS + ch * 8;
    }
  }
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    const int c = threadIdx.x + i * (NWARPS * 32);
    const int row = c / CHUNKS, ch = c - row * CHUNKS;
    __nv_bfloat16* kd = k_dst + row * LD + ch * 8;
    __nv_bfloat16* vd = v_dst + row * LD + ch * 8;
    if (src[i] >= 0) {
      cp_async16(kd, p.k_pool + src[i]);
      cp_async16(vd, p.v_pool + src[i]);
    } else {
      *reinterpret_cast<uint4*>(kd) = make_uint4(0u, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(vd) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

// DEC: the block has at most 16 rows; warps split the keys of a tile instead of the rows.
template <int HS, bool DEC>
__global__ void __launch_bounds__(NWARPS * 32) paged_attention_mma_kernel(const AttnParams p) {
  constexpr int LD = HS + 8;            // padded row: ldmatrix rows fall into distinct banks
  constexpr int KSTEPS = HS / 16;       // k-steps of Q K^T
  constexpr int DT = HS / 8;            // n8 tiles of the output along the head dimension
  constexpr int WKEYS = DEC ? BN / NWARPS : BN;   // keys of a tile that one warp handles
  constexpr int ST = WKEYS / 8;         // n8 tiles of S along this warp's keys
  constexpr int RB = DEC ? 16 : BM;     // rows per block
  constexpr int NST = DEC ? 3 : 2;      // K/V tiles in flight: decode blocks are latency bound
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [RB][LD]
  __nv_bfloat16* k_s = q_s + RB * LD;                                 // [NST][BN][LD]
  __nv_bfloat16* v_s = k_s + NST * BN * LD;                           // [NST][BN][LD]
  pdl_launch_dependents();
  pdl_wait();

  const int req = blockIdx.y / p.g, kvh = blockIdx.y - req * p.g;
  const int tok0 = p.q_start[req], q_len = p.q_start[req + 1] - tok0;
  const int n_rows = q_len * p.per;
  const int row0 = blockIdx.x * RB;
  if (row0 >= n_rows) return;
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tig = lane & 3;
  const int wrow = DEC ? 0 : warp * 16;           // first row of this warp within the block's tile
  const int wkey = DEC ? warp * WKEYS : 0;        // first key of this warp within a key tile
  const int32_t* bt = p.block_table + (size_t)req * p.table_width;

  // Positions of the tile's first and last token bound the keys this block needs.
  const int first_tok = row0 / p.per;
  const int last_row = min(row0 + RB, n_rows) - 1;
  const int last_tok = last_row / p.per;
  const int pos_first = p.positions[tok0 + first_tok];
  const int pos_last = p.positions[tok0 + last_tok];
  const int lo_key = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
  const int hi_key = pos_last;
  int tile_lo = lo_key / BN, tile_hi = hi_key / BN + 1;     // key tiles [tile_lo, tile_hi)
  if (p.n_splits > 1) {
    const int total = tile_hi - tile_lo;
    const int per_split = (total + p.n_splits - 1) / p.n_splits;
    tile_lo = tile_lo + split * per_split;
    tile_hi = min(tile_hi, tile_lo + per_split);
  }
  const int n_tiles = max(0, tile_hi - tile_lo);

  // ---- Q tile -> shared memory, then this warp's A fragments ----------------------
  {
    constexpr int CHUNKS = HS / 8;
    for (int c = threadIdx.x; c < RB * CHUNKS; c += NWARPS * 32) {
      const int r = c / CHUNKS, ch = c - r * CHUNKS;
      const int row = row0 + r;
      __nv_bfloat16* d = q_s + r * LD + ch * 8;
      if (row < n_rows) {
        const int t = row / p.per, h = row - t * p.per;
        cp_async16(d, p.q + (size_t)(tok0 + t) * p.q_stride + (size_t)(kvh * p.per + h) * HS + ch * 8);
      } else {
        *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  }
  // Prologue: Q and the first tile form one group, then NST-2 further tiles one group each.
#pragma unroll
  for (int t = 0; t < NST - 1; ++t) {
    if (t < n_tiles)
      load_kv_tile<HS>(k_s + t * BN * LD, v_s + t * BN * LD, bt, p, kvh, (tile_lo + t) * BN, lo_key, hi_key);
    cp_async_commit();
  }
  cp_async_wait<NST - 2>();     // the group with Q and tile 0 has landed
  __syncthreads();

  unsigned qf[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    const int r = wrow + (lane & 7) + ((lane >> 3) & 1) * 8;
    const int c = ks * 16 + (lane >> 4) * 8;
    ldmatrix_x4(qf[ks], q_s + r * LD + c);
  }
  // Rows of this thread: gid and gid + 8 of the warp's 16.
  int row_pos[2];
  bool row_ok[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + wrow + gid + i * 8;
    row_ok[i] = row < n_rows;
    row_pos[i] = row_ok[i] ? p.positions[tok0 + row / p.per] : -1;
  }

  float o[DT][4];
#pragma unroll
  for (int d = 0; d < DT; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  for (int it = 0; it < n_tiles; ++it) {
    const int buf = it % NST;
    const int key0 = (tile_lo + it) * BN;
    // prefetch tile it + NST - 1 into the buffer that tile it - 1 has left
    if (it + NST - 1 < n_tiles) {
      const int nb = (it + NST - 1) % NST;
      load_kv_tile<HS>(k_s + nb * BN * LD, v_s + nb * BN * LD, bt, p, kvh, key0 + (NST - 1) * BN, lo_key, hi_key);
    }
    cp_async_commit();
    const __nv_bfloat16* kt = k_s + buf * BN * LD;
    const __nv_bfloat16* vt = v_s + buf * BN * LD;

    // ---- S = Q K^T ------------------------------------------------------------------
    float s[ST][4];
#pragma unroll
    for (int j = 0; j < ST; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
      for (int j = 0; j < ST; j += 2) {
        unsigned kb[4];
        const int key = wkey + j * 8 + (lane & 7) + (lane >> 4) * 8;
        const int dim = ks * 16 + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(kb, kt + key * LD + dim);
        mma_bf16(s[j], qf[ks], kb[0], kb[1]);
        mma_bf16(s[j + 1], qf[ks], kb[2], kb[3]);
      }
    }
    // ---- mask, online softmax (exp2 domain) -----------------------------------------
    float m_new[2] = {m_run[0], m_run[1]};
    // A tile strictly inside every row's visible range needs no mask (the common case in decode).
    const bool inner = key0 + BN - 1 <= pos_first && (p.window <= 0 || key0 > pos_last - p.window) &&
                       row0 + RB <= n_rows;
    if (inner) {
#pragma unroll
      for (int j = 0; j < ST; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s[j][e] *= p.scale_log2;
          m_new[e >> 1] = fmaxf(m_new[e >> 1], s[j][e]);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < ST; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = e >> 1;
          const int key = key0 + wkey + j * 8 + tig * 2 + (e & 1);
          const bool vis = row_ok[i] && key <= row_pos[i] && (p.window <= 0 || key > row_pos[i] - p.window);
          const float v = vis ? s[j][e] * p.scale_log2 : -INFINITY;
          s[j][e] = v;
          m_new[i] = fmaxf(m_new[i], v);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
      m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
    }
    float corr[2], base[2], l_add[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      base[i] = (m_new[i] == -INFINITY) ? 0.f : m_new[i];
      corr[i] = exp2f(m_run[i] - base[i]);          // m_run = -inf gives 0
      m_run[i] = m_new[i];
    }
    unsigned pf[ST / 2][4];
#pragma unroll
    for (int j = 0; j < ST; ++j) {
      const float p0 = exp2f(s[j][0] - base[0]), p1 = exp2f(s[j][1] - base[0]);
      const float p2 = exp2f(s[j][2] - base[1]), p3 = exp2f(s[j][3] - base[1]);
      l_add[0] += p0 + p1;
      l_add[1] += p2 + p3;
      pf[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
      pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * corr[i] + l_add[i];
#pragma unroll
    for (int d = 0; d < DT; ++d) {
      o[d][0] *= corr[0]; o[d][1] *= corr[0];
      o[d][2] *= corr[1]; o[d][3] *= corr[1];
    }
    // ---- O += P V -------------------------------------------------------------------
#pragma unroll
    for (int kk = 0; kk < ST / 2; ++kk) {
#pragma unroll
      for (int d = 0; d < DT; d += 2) {
        unsigned vb[4];
        const int key = wkey + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int dim = d * 8 + (lane >> 4) * 8;
        ldmatrix_x4_trans(vb, vt + key * LD + dim);
        mma_bf16(o[d], pf[kk], vb[0], vb[1]);
        mma_bf16(o[d + 1], pf[kk], vb[2], vb[3]);
      }
    }
    cp_async_wait<NST - 2>();   // tile it + 1 has landed (later ones may still fly)
    __syncthreads();
  }

  // ---- finish -----------------------------------------------------------------------
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }
  if constexpr (DEC) {
    // The four warps hold partial states of the same 16 rows: merge them in warp order.
    float* mo = reinterpret_cast<float*>(k_s);        // [NWARPS][16][HS]
    float* mml = reinterpret_cast<float*>(v_s);       // [NWARPS][16][2]
    __syncthreads();                                    // every warp is done with the K/V tiles
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = gid + i * 8;
#pragma unroll
      for (int d = 0; d < DT; ++d)
        *reinterpret_cast<float2*>(mo + ((size_t)warp * 16 + r) * HS + d * 8 + tig * 2) =
            make_float2(o[d][i * 2], o[d][i * 2 + 1]);
      if (tig == 0) {
        mml[(warp * 16 + r) * 2] = m_run[i];
        mml[(warp * 16 + r) * 2 + 1] = l_run[i];
      }
    }
    __syncthreads();
    const int rows_here = min(16, n_rows - row0);
    for (int e = threadIdx.x; e < rows_here * HS; e += NWARPS * 32) {
      const int r = e / HS, d = e - r * HS;
      float mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < NWARPS; ++w) mm = fmaxf(mm, mml[(w * 16 + r) * 2]);
      float ll = 0.f, acc = 0.f;
#pragma unroll
      for (int w = 0; w < NWARPS; ++w) {
        const float m = mml[(w * 16 + r) * 2];
        const float f = (m == -INFINITY) ? 0.f : exp2f(m - mm);
        ll += mml[(w * 16 + r) * 2 + 1] * f;
        acc += mo[((size_t)w * 16 + r) * HS + d] * f;
      }
      const int row = row0 + r;
      const int t = row / p.per, h = row - t * p.per;
      const int tok = tok0 + t, head = kvh * p.per + h;
      if (p.n_splits == 1) {
        p.out[(size_t)tok * p.out_stride + (size_t)head * HS + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
      } else {
        const size_t slot = ((size_t)tok * p.nh + head) * p.n_splits + split;
        p.part_o[slot * HS + d] = acc;
        if (d == 0) {
          p.part_ml[slot * 2] = mm;
          p.part_ml[slot * 2 + 1] = ll;
        }
      }
    }
    if (p.n_splits > 1) {
      // Ticket: the block that finds every other split already done merges them all.
      __shared__ int s_last;
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) s_last = (atomicAdd(&p.tickets[blockIdx.y], 1) == p.n_splits - 1) ? 1 : 0;
      __syncthreads();
      if (s_last) {
        __threadfence();
        for (int e = threadIdx.x; e < rows_here * HS; e += NWARPS * 32) {
          const int r = e / HS, d = e - r * HS;
          const int row = row0 + r;
          const int t = row / p.per, h = row - t * p.per;
          const int tok = tok0 + t, head = kvh * p.per + h;
          const size_t base = ((size_t)tok * p.nh + head) * p.n_splits;
          const volatile float* ml = p.part_ml;
          const volatile float* po = p.part_o;
          float mm = -INFINITY;
          for (int sp = 0; sp < p.n_splits; ++sp) mm = fmaxf(mm, ml[(base + sp) * 2]);
          float ll = 0.f, acc = 0.f;
          for (int sp = 0; sp < p.n_splits; ++sp) {
            const float m = ml[(base + sp) * 2];
            const float f = (m == -INFINITY) ? 0.f : exp2f(m - mm);
            ll += ml[(base + sp) * 2 + 1] * f;
            acc += po[(base + sp) * HS + d] * f;
          }
          p.out[(size_t)tok * p.out_stride + (size_t)head * HS + d] = __float2bfloat16_rn(ll > 0.f ? acc / ll : 0.f);
        }
        if (threadIdx.x == 0) p.tickets[blockIdx.y] = 0;
      }
    }
  } else {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!row_ok[i]) continue;
    const int row = row0 + wrow + gid + i * 8;
    const int t = row / p.per, h = row - t * p.per;
    const int tok = tok0 + t, head = kvh * p.per + h;
    const float inv = l_run[i] > 0.f ? 1.0f / l_run[i] : 0.f;
    __nv_bfloat16* dst = p.out + (size_t)tok * p.out_stride + (size_t)head * HS;
#pragma unroll
    for (int d = 0; d < DT; ++d) {
      __nv_bfloat162 v = __floats2bfloat162_rn(o[d][i * 2] * inv, o[d][i * 2 + 1] * inv);
      *reinterpret_cast<__nv_bfloat162*>(dst + d * 8 + tig * 2) = v;
    }
  }
  }
}

template <int HS, bool DEC>
int launch_mode(const AttnParams& p, int n_requests, int max_rows, cudaStream_t stream) {
  constexpr int LD = HS + 8;
  constexpr int RB = DEC ? 16 : BM, NST = DEC ? 3 : 2;
  const size_t smem = (size_t)(RB + 2 * NST * BN) * LD * sizeof(__nv_bfloat16);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(paged_attention_mma_kernel<HS, DEC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return YALIS_ERR_LAUNCH;
    configured = true;
  }
  dim3 grid((max_rows + RB - 1) / RB, n_requests * p.g, p.n_splits);
  if (grid.y > 65535 || grid.z > 65535) return YALIS_ERR_SHAPE;
  return yalis_launch(paged_attention_mma_kernel<HS, DEC>, grid, dim3(NWARPS * 32), smem, stream, p);
}

template <int HS>
int launch(const AttnParams& p, int n_requests, int max_rows, cudaStream_t stream) {
  return max_rows <= 16 ? launch_mode<HS, true>(p, n_requests, max_rows, stream)
                        : launch_mode<HS, false>(p, n_requests, max_rows, stream);
}

}  // namespace

// Head sizes this kernel is built for.
YALIS_API int yalis_attention_mma_supports(int hs) {
  switch (hs) {
    case 16: case 32: case 48: case 64: case 80: case 96: case 112: case 128: case 160: case 192: case 224: case 256:
      return 1;
    default:
      return 0;
  }
}

// Scratch floats needed for n_splits > 1: part_o then part_ml.  Besides, `tickets` needs
// n_requests * g int32 that are zero before the first launch (each launch leaves them zero).
YALIS_API long long yalis_attention_mma_scratch_floats(int n_tokens, int nh, int hs, int n_splits) {
  return n_splits > 1 ? (long long)n_tokens * nh * n_splits * (hs + 2) : 0;
}

YALIS_API int yalis_paged_attention_mma(const void* q, int q_stride, void* out, int out_stride, const void* k_pool,
                                        const void* v_pool, const int32_t* positions, const int32_t* q_start,
                                        const int32_t* req_of_token, const int32_t* block_table, int table_width,
                                        int page_size, int num_pages, int n_tokens, int n_requests, int max_q_len,
                                        int nh, int g, int hs, float scale, int window, int n_splits, float* scratch,
                                        int32_t* tickets, cudaStream_t stream) {
  if (n_tokens <= 0 || n_requests <= 0) return YALIS_OK;
  if (g <= 0 || nh % g != 0 || n_splits < 1 || max_q_len < 1) return YALIS_ERR_SHAPE;
  if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15) return YALIS_ERR_ALIGN;
  if ((q_stride % 8) || (out_stride % 2)) return YALIS_ERR_ALIGN;
  AttnParams p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride;
  p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.k_pool = (const __nv_bfloat16*)k_pool; p.v_pool = (const __nv_bfloat16*)v_pool;
  p.positions = positions; p.q_start = q_start; p.block_table = block_table;
  p.table_width = table_width; p.page_size = page_size; p.num_pages = num_pages;
  p.page_shift = -1;
  for (int sh = 0; sh < 31; ++sh)
    if ((1 << sh) == page_size) p.page_shift = sh;
  p.nh = nh; p.g = g; p.per = nh / g;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window; p.n_splits = n_splits;
  p.part_o = nullptr; p.part_ml = nullptr; p.tickets = tickets;
  if (n_splits > 1) {
    if (scratch == nullptr || tickets == nullptr || max_q_len * p.per > 16) return YALIS_ERR_SHAPE;
    p.part_o = scratch;
    p.part_ml = scratch + (size_t)n_tokens * nh * n_splits * hs;
  }
  const int max_rows = max_q_len * p.per;
  int st;
  switch (hs) {
    case 16: st = launch<16>(p, n_requests, max_rows, stream); break;
    case 32: st = launch<32>(p, n_requests, max_rows, stream); break;
    case 48: st = launch<48>(p, n_requests, max_rows, stream); break;
    case 64: st = launch<64>(p, n_requests, max_rows, stream); break;
    case 80: st = launch<80>(p, n_requests, max_rows, stream); break;
    case 96: st = launch<96>(p, n_requests, max_rows, stream); break;
    case 112: st = launch<112>(p, n_requests, max_rows, stream); break;
    case 128: st = launch<128>(p, n_requests, max_rows, stream); break;
    case 160: st = launch<160>(p, n_requests, max_rows, stream); break;
    case 192: st = launch<192>(p, n_requests, max_rows, stream); break;
    case 224: st = launch<224>(p, n_requests, max_rows, stream); break;
    case 256: st = launch<256>(p, n_requests, max_rows, stream); break;
    default: return YALIS_ERR_SHAPE;
  }
  return st;
}

// ---------------------------------------------------------------------------------------
// The same kernel with its temporary memory in a fixed array of the library, for callers that
// must not allocate (see attention_noalloc.h for who they are and for the rules).
// ---------------------------------------------------------------------------------------
#include <atomic>

#include "attention_noalloc.h"

namespace {

// Counters first (must be zero when a launch starts), then the partial results.  The name is
// usable as an address in device code only; host code has to ask the runtime for its address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[YALIS_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
// Device address of the array, per device.  Threads that make a device's first call at the same time all ask
// the runtime and store the same address: the slots are atomic so that none of them reads a half-written one.
std::atomic<void*> g_noalloc_ptr[kMaxDevices];

// Device address of the array on the current device; looked up on the first call there.
int noalloc_scratch(unsigned char** ptr) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return YALIS_ERR_LAUNCH;
  void* p = g_noalloc_ptr[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) return YALIS_ERR_LAUNCH;
    g_noalloc_ptr[dev].store(p, std::memory_order_release);
  }
  *ptr = static_cast<unsigned char*>(p);
  return YALIS_OK;
}

}  // namespace

YALIS_API long long yalis_paged_attention_mma_noalloc_needed(int n_tokens, int n_requests, int nh, int g, int hs,
                                                             int n_splits, long long* ticket_bytes,
                                                             long long* partial_bytes) {
  const long long t = n_splits > 1 ? (long long)n_requests * g * (long long)sizeof(int32_t) : 0;
  const long long f = yalis_attention_mma_scratch_floats(n_tokens, nh, hs, n_splits) * (long long)sizeof(float);
  if (ticket_bytes) *ticket_bytes = t;
  if (partial_bytes) *partial_bytes = f;
  return t + f;
}

YALIS_API int yalis_paged_attention_mma_noalloc(const void* q, int q_stride, void* out, int out_stride,
                                                const void* k_pool, const void* v_pool, const int32_t* positions,
                                                const int32_t* q_start, const int32_t* req_of_token,
                                                const int32_t* block_table, int table_width, int page_size,
                                                int num_pages, int n_tokens, int n_requests, int max_q_len, int nh,
                                                int g, int hs, float scale, int window, int n_splits,
                                                cudaStream_t stream) {
  if (n_tokens <= 0 || n_requests <= 0) return YALIS_OK;
  if (n_splits < 1 || g <= 0) return YALIS_ERR_SHAPE;
  long long ticket_bytes = 0, partial_bytes = 0;
  yalis_paged_attention_mma_noalloc_needed(n_tokens, n_requests, nh, g, hs, n_splits, &ticket_bytes, &partial_bytes);
  if (ticket_bytes > YALIS_NOALLOC_TICKET_BYTES || partial_bytes > YALIS_NOALLOC_PARTIAL_BYTES)
    return YALIS_ERR_SCRATCH;                       // refused: nothing was launched
  unsigned char* base = nullptr;
  if (int st = noalloc_scratch(&base)) return st;
  int32_t* tickets = reinterpret_cast<int32_t*>(base);
  float* partials = reinterpret_cast<float*>(base + YALIS_NOALLOC_TICKET_BYTES);
  if (n_splits > 1) {
    // The array keeps what the last call left: the counters have to start at zero.
    if (cudaMemsetAsync(tickets, 0, (size_t)ticket_bytes, stream) != cudaSuccess) return YALIS_ERR_LAUNCH;
  }
  return yalis_paged_attention_mma(q, q_stride, out, out_stride, k_pool, v_pool, positions, q_start, req_of_token,
                                   block_table, table_width, page_size, num_pages, n_tokens, n_requests, max_q_len, nh,
                                   g, hs, scale, window, n_splits, n_splits > 1 ? partials : nullptr,
                                   n_splits > 1 ? tickets : nullptr, stream);
}
