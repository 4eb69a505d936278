// Decode attention for steps with more (request, KV head) pairs than the GPU holds blocks at once.
//
// attention_decode_tma.cu gives every pair a block of its own (or several): with 512 pairs and 296
// resident blocks the second wave is three quarters empty, and every block pays its start-up and
// its merge.  Here the grid is fixed (as many blocks as are resident at once) and the *tiles* of
// all pairs, laid end to end, are dealt out evenly: block b takes the tiles
// [b * total / blocks, (b + 1) * total / blocks), whatever pairs they belong to.  A block walks its
// range pair by pair ("segments"); its producer warp keeps the TMA ring full across segment
// borders, so the next pair's first tiles arrive while the consumers finish the previous pair.
//
//   * A segment that covers a whole pair is normalised and written out by its block.
//   * A pair cut by a block border is finished by whichever of its blocks comes last (a ticket per
//     pair): each block leaves its (max, sum, unnormalised output) in scratch memory, in one of
//     two slots of its own (its first and its last segment are the only ones that can be cut), and
//     the last one adds the pieces in block order.  No block ever waits for another.
//   * The schedule is computed in the kernel from the step's positions (a prefix sum over the
//     requests' tile counts in shared memory), so a captured launch can be replayed with other
//     lengths.
//
//   * The next pair's queries are fetched into registers while the current pair is computed; the
//     ring has three stages where two blocks of them still share an SM, else two.
//   * With early_fetch the schedule and the first tiles (those that lie wholly below a query's
//     position) do not wait for the preceding kernel (see the entry point for what the caller
//     promises).
//   * The same kernel takes batches that are long or uneven in length at any size (the host
//     decides), and the decoding requests of a step that also holds prompt portions (only_single).
//
// Tile handling, masking and the arithmetic are those of decode_attention_tma_kernel; limits are
// the same (bfloat16, head_dim 64/128/192/256, pages of 8..64 tokens, no window, at most 16 query
// heads per KV head, one token per request), and at most 4096 requests.  Every mbarrier wait is
// bounded; on a timeout the block raises the error word, drains its copies and returns.
#include "decode_tiles.cuh"

namespace {

constexpr int kMaxRequests = 4096;

struct LeanParams {
  const __nv_bfloat16* q;      // [N, q_stride]
  int q_stride;
  __nv_bfloat16* out;          // [N, out_stride]
  int out_stride;
  const int32_t* positions;    // [N]
  const int32_t* q_start;      // [R+1]
  const int32_t* block_table;  // [R, table_width]
  int table_width, page_size, num_pages;
  int n_requests, nh, g, per;
  float scale_log2;
  int early_fetch;             // 1: index arrays and keys below the queries' positions are settled (see the kernel)
  int only_single;             // 1: requests that bring more than one token are left to another kernel
  float* part_o;               // [blocks, 2, 16, HS]
  float* part_ml;              // [blocks, 2, 16, 2]
  int32_t* tickets;            // [R * g], zero before and after
  int32_t* error;
};

// First tile of block b when `total` tiles are dealt to `blocks` blocks.
__device__ __forceinline__ long long first_tile_of(int b, long long total, int blocks) { return (long long)b * total / blocks; }
// The block that holds tile t: the largest b with first_tile_of(b) <= t.
__device__ __forceinline__ int block_of_tile(long long t, long long total, int blocks) {
  return (int)(((t + 1) * blocks + total - 1) / total) - 1;
}

// One stretch of a block's range inside one (request, KV head).
struct Segment {
  int req, kvh;
  int tile_lo, tile_hi;        // tiles [tile_lo, tile_hi) of the pair
  int tiles;                   // tiles of the whole pair
  long long first;             // index of the pair's first tile among all tiles
};

// Walks the segments of the tile range [t, end): `cum` holds the requests' tile counts as a prefix
// sum ([R+1]), every request's tiles g times over (KV head after KV head).
struct Walker {
  const int* cum;
  int n_requests, g;
  long long t, end;
  int req;
  __device__ void start(const int* cum_, int n_requests_, int g_, long long t_, long long end_) {
    cum = cum_; n_requests = n_requests_; g = g_; t = t_; end = end_;
    // the last request whose first tile is at or before t (requests without tiles share their successor's start)
    int lo = 0, hi = n_requests - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if ((long long)cum[mid] * g <= t) lo = mid; else hi = mid - 1;
    }
    req = lo;
  }
  __device__ bool next(Segment* s) {
    if (t >= end) return false;
    while (req + 1 < n_requests && (long long)cum[req + 1] * g <= t) ++req;
    const int tiles = cum[req + 1] - cum[req];
    const long long base = (long long)cum[req] * g;
    const int kvh = (int)((t - base) / tiles);
    const int a = (int)((t - base) - (long long)kvh * tiles);
    const int n = (int)min((long long)(tiles - a), end - t);
    s->req = req; s->kvh = kvh; s->tile_lo = a; s->tile_hi = a + n; s->tiles = tiles;
    s->first = base + (long long)kvh * tiles;
    t += n;
    return true;
  }
};

// Registers: two blocks of five warps share an SM only up to 168 a thread (the register file is dealt out
// to warps in groups), which head sizes up to 128 keep to; larger ones run one block per SM.
template <int HS, int NST>
__global__ void __maxnreg__(HS <= 128 ? 168 : 255)
decode_attention_lean_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                             const LeanParams p) {
  constexpr int H2 = HS / 64;                  // 64-column halves of a row
  constexpr int TILE_BYTES = BN * HS * 2;      // one K (or V) tile
  constexpr int LDQ = HS + 8;                  // padded Q rows
  constexpr int KSTEPS = HS / 16, DT = HS / 8;
  constexpr int WKEYS = BN / CWARPS;           // 16 keys of a tile per consumer warp
  constexpr int VEC = HS / 4;                  // float4 groups of a row
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int n_rows = p.per;                    // rows that count = query heads of a KV head
  unsigned char* k_s = base;                                 // [NST][TILE_BYTES]
  unsigned char* v_s = base + NST * TILE_BYTES;              // [NST][TILE_BYTES]
  float* mo = reinterpret_cast<float*>(v_s + NST * TILE_BYTES);             // [CWARPS][n_rows][HS] the warps' outputs
  float* mml = mo + CWARPS * n_rows * HS;                                    // [CWARPS][n_rows][2] their max and sum
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(mml + CWARPS * n_rows * 2);   // [16][LDQ]
  uint64_t* full = reinterpret_cast<uint64_t*>(q_s + 16 * LDQ);
  uint64_t* empty = full + NST;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + NST);
  int* s_last = const_cast<int*>(abort_flag) + 1;
  int* cum = s_last + 3;                                                     // [R+1] prefix sum of tile counts

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x;
  if (threadIdx.x == CWARPS * 32) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], CWARPS);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  for (int c = threadIdx.x; c < 16 * LDQ / 8; c += kThreads)          // the rows of Q beyond n_rows stay zero
    reinterpret_cast<uint4*>(q_s)[c] = make_uint4(0u, 0u, 0u, 0u);
  // With early_fetch the caller promises that positions, q_start, the block table and every key and value below
  // the queries' positions were complete before the preceding kernel began: the schedule and the first tiles
  // then do not wait for that kernel (which writes this step's queries, keys and values).
  if (!p.early_fetch) pdl_wait();

  // ---- the schedule: tiles per request, their prefix sum, this block's range ---------------------
  for (int r = threadIdx.x; r < p.n_requests; r += kThreads) {
    const int tok = p.q_start[r];
    const int n_tok = p.q_start[r + 1] - tok;
    cum[r + 1] = (p.only_single ? n_tok == 1 : n_tok > 0) ? p.positions[tok] / BN + 1 : 0;
  }
  if (threadIdx.x == 0) cum[0] = 0;
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int r0 = 0; r0 < p.n_requests; r0 += 32) {
      const int r = r0 + lane;
      int v = r < p.n_requests ? cum[r + 1] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
      }
      if (r < p.n_requests) cum[r + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
  const long long total = (long long)cum[p.n_requests] * p.g;
  const int blocks = (int)min((long long)gridDim.x, total);     // every block that works has at least one tile
  const long long t_lo = b < blocks ? first_tile_of(b, total, blocks) : 0;
  const long long t_hi = b < blocks ? first_tile_of(b + 1, total, blocks) : 0;

  int armed = 0;                               // tiles this block has asked for (producer) / used (consumers)
  if (warp == CWARPS) {
    // ---- producer: the block's tiles in order, segment after segment ----------------------------
    const int pages_per_tile = BN / p.page_size;
    const uint32_t page_bytes = (uint32_t)p.page_size * HS * 2;
    Walker w;
    w.start(cum, p.n_requests, p.g, t_lo, t_hi);
    Segment sg;
    bool alive = true;
    bool waited = !p.early_fetch;              // whether this warp has waited for the preceding kernel
    while (alive && w.next(&sg)) {
      const int hi_key = p.positions[p.q_start[sg.req]];
      const int32_t* bt = p.block_table + (size_t)sg.req * p.table_width;
      for (int tile = sg.tile_lo; tile < sg.tile_hi; ++tile) {
        if (!waited && (tile == sg.tiles - 1 || armed >= NST)) {
          // a pair's last tile holds the key written in this step; and the ring is full until the consumers start
          pdl_wait();
          waited = true;
        }
        const int s = armed % NST;
        const uint32_t ph = (armed / NST) & 1;
        const int key0 = tile * BN;
        const int n_pages = min(pages_per_tile, (hi_key - key0) / p.page_size + 1);
        int ok = 1;
        if (lane == 0) {
          ok = mbar_wait(&empty[s], ph ^ 1, abort_flag) ? 1 : 0;
          if (ok) mbar_expect_tx(&full[s], 2u * page_bytes * (uint32_t)n_pages);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) { alive = false; break; }
        for (int c = lane; c < n_pages * 2 * H2; c += 32) {
          const int i = c / (2 * H2), kv = (c / H2) & 1, h = c % H2;
          const int pi = key0 / p.page_size + i;
          int page = pi < p.table_width ? bt[pi] : -1;
          if (page < 0 || page >= p.num_pages) {   // a visible key without a page: a caller's bug
            if (p.error) atomicOr(p.error, YALIS_FLAG_BAD_PAGE);
            page = 0;
          }
          const int y = (page * p.g + sg.kvh) * p.page_size;
          const int off = h * (BN * 128) + i * p.page_size * 128;
          tma_load_2d((kv ? v_s : k_s) + s * TILE_BYTES + off, kv ? &map_v : &map_k, h * 64, y, &full[s]);
        }
        __syncwarp();
        ++armed;
      }
    }
    if (!waited) pdl_wait();
    if (lane == 0) pdl_launch_dependents();     // the last tile is on its way
    __syncwarp();
  } else {
    // ---- consumers ---------------------------------------------------------------------------------
    if (p.early_fetch) pdl_wait();
    const int gid = lane >> 2, tig = lane & 3;
    const int wkey = warp * WKEYS;
    const bool row_ok[2] = {gid < n_rows, gid + 8 < n_rows};
    constexpr int CHUNKS = HS / 8;             // 16-byte pieces of a query row
    constexpr int QLOADS = (16 * CHUNKS + CWARPS * 32 - 1) / (CWARPS * 32);
    Walker w;
    w.start(cum, p.n_requests, p.g, t_lo, t_hi);
    Segment sg, nx;
    // The queries of a segment are fetched into registers while the segment before it is computed.
    uint4 q_next[QLOADS];
    int tok_next = 0, hi_next = 0;
    auto fetch_q = [&](const Segment& to) {
      tok_next = p.q_start[to.req];
      hi_next = p.positions[tok_next];
#pragma unroll
      for (int j = 0; j < QLOADS; ++j) {
        const int c = threadIdx.x + j * CWARPS * 32;
        const int r = c / CHUNKS, ch = c - r * CHUNKS;
        if (r < n_rows)
          q_next[j] = *reinterpret_cast<const uint4*>(p.q + (size_t)tok_next * p.q_stride + (size_t)(to.kvh * p.per + r) * HS + ch * 8);
      }
    };
    bool more = w.next(&nx);
    if (more) fetch_q(nx);
    for (int seg_index = 0; more; ++seg_index) {
      sg = nx;
      const int tok = tok_next;
      const int hi_key = hi_next;
      consumer_sync();                         // the previous segment's merge has been read, its queries are in registers
#pragma unroll
      for (int j = 0; j < QLOADS; ++j) {
        const int c = threadIdx.x + j * CWARPS * 32;
        const int r = c / CHUNKS, ch = c - r * CHUNKS;
        if (r < n_rows) *reinterpret_cast<uint4*>(q_s + r * LDQ + ch * 8) = q_next[j];
      }
      consumer_sync();
      more = w.next(&nx);
      if (more) fetch_q(nx);
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

      for (int tile = sg.tile_lo; tile < sg.tile_hi; ++tile, ++armed) {
        const int s = armed % NST;
        const uint32_t ph = (armed / NST) & 1;
        int ok = 1;
        if (lane == 0) ok = mbar_wait(&full[s], ph, abort_flag) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;                        // timed out: the block stops after this segment
        const int key0 = tile * BN;
        const uint32_t kt = smem_u32(k_s + s * TILE_BYTES), vt = smem_u32(v_s + s * TILE_BYTES);
        const bool last = key0 + BN - 1 > hi_key;
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

      // ---- merge the four warps ------------------------------------------------------------------
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = gid + i * 8;
        if (r < n_rows) {
#pragma unroll
          for (int d = 0; d < DT; ++d)
            *reinterpret_cast<float2*>(mo + ((size_t)warp * n_rows + r) * HS + d * 8 + tig * 2) = make_float2(o[d][i * 2], o[d][i * 2 + 1]);
          if (tig == 0) {
            mml[(warp * n_rows + r) * 2] = m_run[i];
            mml[(warp * n_rows + r) * 2 + 1] = l_run[i];
          }
        }
      }
      if (threadIdx.x == 0) s_last[1] = *abort_flag;      // one reading of the flag for all consumers
      consumer_sync();
      if (s_last[1]) break;
      const bool whole = sg.tile_lo == 0 && sg.tile_hi == sg.tiles;
      const int slot = b * 2 + (seg_index == 0 ? 0 : 1);    // only a block's first and last segment can be cut
      for (int e = threadIdx.x; e < n_rows * VEC; e += CWARPS * 32) {
        const int r = e / VEC, d = (e - r * VEC) * 4;
        float mw[CWARPS], mm = -INFINITY;
#pragma unroll
        for (int wi = 0; wi < CWARPS; ++wi) {
          mw[wi] = mml[(wi * n_rows + r) * 2];
          mm = fmaxf(mm, mw[wi]);
        }
        float ll = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int wi = 0; wi < CWARPS; ++wi) {
          const float f = (mw[wi] == -INFINITY) ? 0.f : exp2f(mw[wi] - mm);
          ll += mml[(wi * n_rows + r) * 2 + 1] * f;
          const float4 v = *reinterpret_cast<const float4*>(mo + ((size_t)wi * n_rows + r) * HS + d);
          acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
        }
        if (whole) {
          store_bf16x4(p.out + (size_t)tok * p.out_stride + (size_t)(sg.kvh * p.per + r) * HS + d, acc, ll > 0.f ? 1.0f / ll : 0.f);
        } else {
          *reinterpret_cast<float4*>(p.part_o + ((size_t)slot * 16 + r) * HS + d) = acc;
          if (d == 0) *reinterpret_cast<float2*>(p.part_ml + ((size_t)slot * 16 + r) * 2) = make_float2(mm, ll);
        }
      }
      if (!whole) {
        // ---- a pair cut by block borders: the last of its blocks to arrive adds the pieces ----------
        const int b_first = block_of_tile(sg.first, total, blocks);
        const int n_parts = block_of_tile(sg.first + sg.tiles - 1, total, blocks) - b_first + 1;
        const int pair = sg.req * p.g + sg.kvh;
        __threadfence();
        consumer_sync();
        if (threadIdx.x == 0) s_last[0] = (atomicAdd(&p.tickets[pair], 1) == n_parts - 1) ? 1 : 0;
        consumer_sync();
        if (s_last[0]) {
          __threadfence();
          // Piece j lies in block b_first + j: in its second slot if the pair is not that block's first
          // segment, which can only be so for the first of them.  Read past the L1, four loads in flight.
          const int slot0 = b_first * 2 + (first_tile_of(b_first, total, blocks) >= sg.first ? 0 : 1);
          auto slot_of = [&](int j) { return j == 0 ? slot0 : (b_first + j) * 2; };
          for (int e = threadIdx.x; e < n_rows * VEC; e += CWARPS * 32) {
            const int r = e / VEC, d = (e - r * VEC) * 4;
            float mm = -INFINITY;
            for (int j0 = 0; j0 < n_parts; j0 += 4) {
              float2 ml[4];
#pragma unroll
              for (int j = 0; j < 4; ++j)
                ml[j] = j0 + j < n_parts ? __ldcg(reinterpret_cast<const float2*>(p.part_ml + ((size_t)slot_of(j0 + j) * 16 + r) * 2))
                                         : make_float2(-INFINITY, 0.f);
#pragma unroll
              for (int j = 0; j < 4; ++j) mm = fmaxf(mm, ml[j].x);
            }
            float ll = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int j0 = 0; j0 < n_parts; j0 += 4) {
              float2 ml[4];
              float4 v[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const bool in = j0 + j < n_parts;
                const size_t at = (size_t)slot_of(in ? j0 + j : 0) * 16 + r;
                ml[j] = in ? __ldcg(reinterpret_cast<const float2*>(p.part_ml + at * 2)) : make_float2(-INFINITY, 0.f);
                v[j] = in ? __ldcg(reinterpret_cast<const float4*>(p.part_o + at * HS + d)) : make_float4(0.f, 0.f, 0.f, 0.f);
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float f = (ml[j].x == -INFINITY) ? 0.f : exp2f(ml[j].x - mm);
                ll += ml[j].y * f;
                acc.x += v[j].x * f; acc.y += v[j].y * f; acc.z += v[j].z * f; acc.w += v[j].w * f;
              }
            }
            store_bf16x4(p.out + (size_t)tok * p.out_stride + (size_t)(sg.kvh * p.per + r) * HS + d, acc, ll > 0.f ? 1.0f / ll : 0.f);
          }
          if (threadIdx.x == 0) p.tickets[pair] = 0;
        }
      }
    }
  }

  // ---- exit: on an abort wait (bounded) for copies in flight so none lands after the block ---
  __syncthreads();
  if (*abort_flag && threadIdx.x == CWARPS * 32) {
    if (p.error) atomicOr(p.error, YALIS_FLAG_WAIT_ATTENTION);
    for (int it = max(0, armed - NST); it < armed; ++it) {
      const int s = it % NST;
      const uint32_t ph = (it / NST) & 1;
      for (uint32_t i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(&full[s], ph)) break;
    }
  }
  __syncthreads();
}

size_t lean_smem_bytes(int hs, int stages, int per, int n_requests) {
  return 1024 + (size_t)2 * stages * BN * hs * 2 + (size_t)CWARPS * per * (hs + 2) * 4 + (size_t)16 * (hs + 8) * 2 +
         2 * stages * 8 + 16 + (size_t)(n_requests + 1) * 4 + 16;
}

template <int HS, int NST>
int launch_lean_stages(const CUtensorMap& mk, const CUtensorMap& mv, const LeanParams& p, int n_blocks, cudaStream_t stream) {
  const size_t smem = lean_smem_bytes(HS, NST, p.per, p.n_requests);
  static size_t configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(decode_attention_lean_kernel<HS, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return YALIS_ERR_LAUNCH;
    configured = smem;
  }
  return yalis_launch(decode_attention_lean_kernel<HS, NST>, dim3(n_blocks), dim3(kThreads), smem, stream, mk, mv, p);
}

// Three ring stages where two blocks of them still share an SM (or one block holds them at all), else two.
template <int HS>
int launch_lean(const CUtensorMap& mk, const CUtensorMap& mv, const LeanParams& p, int n_blocks, cudaStream_t stream) {
  const size_t three = lean_smem_bytes(HS, 3, p.per, p.n_requests), two = lean_smem_bytes(HS, 2, p.per, p.n_requests);
  const size_t half_sm = 113 * 1024, whole_sm = 226 * 1024;
  const bool use_three = three <= half_sm || (two > half_sm && three <= whole_sm);
  if (use_three) return launch_lean_stages<HS, 3>(mk, mv, p, n_blocks, stream);
  if (two > whole_sm) return YALIS_ERR_SHAPE;
  return launch_lean_stages<HS, 2>(mk, mv, p, n_blocks, stream);
}

}  // namespace

// Floats of scratch memory for a launch of n_blocks blocks.
YALIS_API long long yalis_decode_attention_lean_scratch_floats(int n_blocks, int hs) {
  return (long long)n_blocks * 2 * 16 * (hs + 2);
}

// One query token per request; the same result as yalis_decode_attention_tma up to the order in which the
// pieces of a cut (request, KV head) are added.  n_blocks: the grid (the number of blocks resident at once is
// the intended value; any positive number is correct).  scratch: yalis_decode_attention_lean_scratch_floats
// floats; tickets: n_requests * g int32, zero before the call and left zero.  error: device int32 raised on a
// timed-out wait or an unmapped page.  early_fetch as for yalis_decode_attention_tma.  A request's token is the
// first of its range in q_start; with only_single = 1 requests that bring more than one token are skipped (their
// rows of out are not written: a step that mixes prompt portions and decoding requests gives those to the
// prompt kernel).
YALIS_API int yalis_decode_attention_lean(const void* q, int q_stride, void* out, int out_stride, const void* k_pool,
                                          const void* v_pool, const int32_t* positions, const int32_t* q_start,
                                          const int32_t* block_table, int table_width, int page_size, int num_pages,
                                          int n_tokens, int n_requests, int nh, int g, int hs, float scale, int n_blocks,
                                          int early_fetch, int only_single, float* scratch, int32_t* tickets, int32_t* error, cudaStream_t stream) {
  if (n_tokens <= 0 || n_requests <= 0) return YALIS_OK;
  if (g <= 0 || nh % g != 0 || n_blocks < 1 || n_requests > kMaxRequests) return YALIS_ERR_SHAPE;
  const bool hs_ok = hs == 64 || hs == 128 || hs == 192 || hs == 256;
  const bool page_ok = page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64;
  if (!hs_ok || !page_ok || nh / g > 16) return YALIS_ERR_SHAPE;
  if (scratch == nullptr || tickets == nullptr) return YALIS_ERR_SHAPE;
  if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out | (uintptr_t)scratch) & 15) return YALIS_ERR_ALIGN;
  if ((q_stride % 8) || (out_stride % 4)) return YALIS_ERR_ALIGN;
  CUtensorMap mk, mv;
  const long long rows = (long long)num_pages * g * page_size;
  if (!make_pool_map(&mk, k_pool, rows, hs, page_size) || !make_pool_map(&mv, v_pool, rows, hs, page_size))
    return YALIS_ERR_LAUNCH;
  LeanParams p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride;
  p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.positions = positions; p.q_start = q_start; p.block_table = block_table;
  p.table_width = table_width; p.page_size = page_size; p.num_pages = num_pages;
  p.n_requests = n_requests; p.nh = nh; p.g = g; p.per = nh / g;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.early_fetch = early_fetch ? 1 : 0;
  p.only_single = only_single ? 1 : 0;
  p.part_o = scratch;
  p.part_ml = scratch + (size_t)n_blocks * 2 * 16 * hs;
  p.tickets = tickets;
  p.error = error;
  switch (hs) {
    case 64: return launch_lean<64>(mk, mv, p, n_blocks, stream);
    case 128: return launch_lean<128>(mk, mv, p, n_blocks, stream);
    case 192: return launch_lean<192>(mk, mv, p, n_blocks, stream);
    default: return launch_lean<256>(mk, mv, p, n_blocks, stream);
  }
}
