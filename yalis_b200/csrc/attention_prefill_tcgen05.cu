// Paged causal attention for prompt portions on the 5th-generation tensor cores.
//
// One block owns up to 128 rows of one (request, KV head) -- row = token * heads_per_group +
// head_in_group, so the whole GQA group of a token shares the K/V tiles -- and walks the visible
// keys in tiles of 64 (two blocks share an SM: while one computes a softmax the other's products run):
//
//   S = Q K^T      tcgen05.mma (cta_group::1, kind::f16), Q and K tiles in 128B-swizzled shared
//                  memory (fed by TMA: Q through a 3-D map [head_dim, heads_per_group, tokens],
//                  K and V one box per cache page or part of a page), S in tensor memory, double buffered;
//   P = softmax    four warps, one thread per row: tcgen05.ld of its S row into registers, mask
//                  by absolute position, running max and sum in float32 (exp2 domain), P packed
//                  to bfloat16 and written back to tensor memory over the S it came from (tcgen05.st);
//   O += P V       tcgen05.mma with A = P from tensor memory and B = the V tile read as an
//                  MN-major operand (V is stored [key][dim]); O stays in tensor memory for the
//                  whole key loop.  When a row's maximum grows by more than 2^8 the softmax
//                  threads rescale O in place (tcgen05.ld / st); smaller growth is absorbed by
//                  keeping the older maximum, which is exact as long as exp2 stays in range.
//
// One warp issues all TMA copies and one warp all MMAs; completion travels over mbarriers
// (tcgen05.commit for the MMAs); QK^T of tile j+1 runs while the softmax of tile j is computed.
// The MMA warp runs its loop converged, waits included, and an elected lane issues: the operands
// of tcgen05.mma are warp-uniform values, and computing them in a branch that a single lane takes
// made each issue cost about a hundred cycles (measured: 410 against 70 cycles for the four
// products and two commits of a P V).  The copy warp looks the pages of a tile up one tile ahead
// (a block-table entry is a global load whose latency would otherwise stand between a freed buffer
// and the copy into it) and asks for K one tile ahead of V, the order in which their buffers come
// free, so that a wait for one never holds up the other.  The grid is (tiles of queries of the step x KV heads, 1,
// shares of the keys); a block finds the request of its tile from the requests' token ranges.
// Same semantics as paged_attention_generic (mask by absolute position,
// yalis/attention/backend_impl/sdpa_and_flex.py:15-19, 301-307) without a window.
//
// Limits (else the caller uses the mma.sync kernel): bfloat16, head_dim 64 or 128, page_size 8,
// 16, 32, 64 or 128, at most 128 heads per KV head, no window.
// Rows of V past a tile's last visible key may hold anything; they are zeroed in shared memory
// before they are multiplied.  All mbarrier waits are bounded (error word, tensor memory freed).
#include <cuda.h>

#include <algorithm>

#include "common.cuh"

namespace {

constexpr int BM = 128;           // rows (tensor-memory lanes) per block
constexpr int BN = 64;            // keys per tile
constexpr int kThreads = 192;     // warps 0-3 softmax, warp 4 TMA, warp 5 MMA + tensor memory
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr int kBarriers = 21;     // mbarriers of a block (see the kernel)
// Two blocks share an SM (one's softmax runs while the other's products do), so each takes half the tensor
// memory: S0, S1 (BN columns each) and O (up to 128).  P(j) is written over the first half of S(j): by then S(j)
// is in registers, and the product that next writes that buffer is issued after the one that reads P(j).
constexpr int TMEM_COLS = 256;
constexpr int COL_S = 0, COL_O = 2 * BN;

struct PrefillParams {
  __nv_bfloat16* out;
  int out_stride;
  const int32_t* positions;    // [N]
  const int32_t* q_start;      // [R+1]
  const int32_t* block_table;  // [R, table_width]
  int table_width, page_size, num_pages;
  int nh, g, per;
  int n_requests;
  int n_items;                 // work items: items_per_share * n_z
  int items_per_share;         // tiles of queries of the step (an upper bound) * KV heads
  int n_z;                     // shares of the keys that a tile of queries may be divided into
  int32_t* work;               // [2] zero between launches: the next item, blocks that are done
  int tokens_per_tile;         // 128 / per
  float scale_log2;
  // With key splits (n_z > 1) a tile of queries whose visible keys fill more than tiles_per_split key tiles
  // is shared by several work items (at most n_z): item z takes its share of the keys and leaves the
  // unnormalised output with its (max, sum) here; a second kernel adds the shares.  Tiles of queries with fewer
  // keys are finished by block 0 alone, which marks their rows (max = +inf in share 0) for the second kernel.
  int tiles_per_split;
  int skip_single;             // 1: requests that bring one token are left to another kernel
  float* part_o;               // [N, nh, n_splits, HS]
  float* part_ml;              // [N, nh, n_splits, 2]
  int32_t* error;
#ifdef YALIS_TRACE_CLOCKS
  long long* trace;            // [blocks][64 tiles][32 stamps] of clock64(), for timeline probes (compiled out by default)
#endif
};

#ifdef YALIS_TRACE_CLOCKS
#define STAMP(j, k)                                                                                             \
  do {                                                                                                          \
    if (p.trace && (j) < 64) p.trace[((size_t)trace_row * 64 + (j)) * 32 + (k)] = clock64(); \
  } while (0)
// Wall-clock stamps (nanoseconds, comparable between blocks) in row 62 of a block's record, and its SM.
#define GSTAMP(k)                                                                                               \
  do {                                                                                                          \
    if (p.trace) {                                                                                              \
      unsigned long long t_;                                                                                    \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                                    \
      p.trace[((size_t)trace_row * 64 + 62) * 32 + (k)] = (long long)t_;            \
    }                                                                                                           \
  } while (0)
#else
#define STAMP(j, k) do { } while (0)
#define GSTAMP(k) do { } while (0)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
#ifdef YALIS_TRACE_CLOCKS
__device__ unsigned long long g_gave_up[8];      // the first wait that ran out: block, thread, barrier address, parity
#endif
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
#ifdef YALIS_TRACE_CLOCKS
  if (atomicCAS(&g_gave_up[0], 0ull, 1ull) == 0ull) {
    g_gave_up[1] = blockIdx.x; g_gave_up[2] = blockIdx.y; g_gave_up[3] = threadIdx.x;
    g_gave_up[4] = smem_u32(bar); g_gave_up[5] = parity;
  }
#endif
  *abort_flag = 1;
  return false;
}
// One lane polls, the warp stays convergent.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int lane) {
  int ok = 1;
  if (lane == 0) ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}
// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
  return ((uint64_t)(saddr >> 4) & 0x3FFFull) | (1ull << 16) | ((1024ull >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand (V stored [key][dim]), 128-byte swizzle: 64 dims (128 bytes) contiguous per key,
// 8-key groups 1024 bytes apart (stride byte offset), the next 64 dims `lbo_bytes` further (leading byte offset).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr, uint32_t lbo_bytes) {
  return ((uint64_t)(saddr >> 4) & 0x3FFFull) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
         ((1024ull >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16, D float32, A/B bfloat16, M = 128; b_mn selects an MN-major B.
__device__ __forceinline__ uint32_t idesc_f16(int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
// 1 in one lane of a converged warp, 0 in the others.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
  return pred;
}
// The products and commits below are executed by every lane of the converged MMA warp and take effect in the
// elected one: all lanes compute the (identical) operands, so these stay warp-uniform values.
__device__ __forceinline__ void umma_ss(uint32_t elected, uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(elected) : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t elected, uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d), "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc), "r"(elected) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t elected, uint64_t* bar) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
               "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
               ::"r"(smem_u32(bar)), "r"(elected) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
// 2^x in one instruction; the softmax arguments are <= 8 and -inf gives 0.
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two float32 operations in one instruction (sm_100): d = a * b + c and d = a + b on pairs held in 64-bit registers
// (each half rounded as the single operation is).  The softmax warps are bound by their own instruction streams:
// pairs took 2 % off the kernel, a share of the exponentials as a polynomial on the FMA pipe added 16 to 24 %.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// What a work item is, as the copy warp hands it to the others through shared memory.
struct ItemDesc {
  int n_tiles;      // key tiles of the item (> 0), or -1: no more items
  int tile_base;    // its first key tile among the tiles its queries see
  int n_splits;     // shares that the tile of queries is divided into (1: finished here)
  int split;        // which of them this item is
  int kvh;
  int tok_first;    // row of the first query token in the step
  int n_rows;       // rows of the tile in use: tokens * heads_per_group
  int pos_first;    // absolute position of the first query token
  int hi_key;       // absolute position of the last one = the last visible key
  int trace_row;
};

template <int HS>
__global__ void __launch_bounds__(kThreads, 2)
prefill_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v, const PrefillParams p) {
  constexpr int H2 = HS / 64;
  constexpr int Q_BYTES = BM * HS * 2;
  constexpr int KV_BYTES = BN * HS * 2;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* q_s = base;                       // [H2][128 rows][128 B]
  unsigned char* k_s = q_s + Q_BYTES;              // [2][H2][128 keys][128 B]
  unsigned char* v_s = k_s + 2 * KV_BYTES;         // [2][H2][128 keys][128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + 2 * KV_BYTES);
  uint64_t* q_full = bars;                         // 1
  uint64_t* k_full = bars + 1;                     // 2
  uint64_t* k_empty = bars + 3;                    // 2
  uint64_t* v_full = bars + 5;                     // 2
  uint64_t* v_empty = bars + 7;                    // 2
  uint64_t* s_full = bars + 9;                     // 2
  uint64_t* q_empty = bars + 11;                   // 1
  uint64_t* p_full = bars + 13;                    // 2
  uint64_t* o_full = bars + 15;                    // 1
  uint64_t* o_done = bars + 16;                    // 1
  uint64_t* desc_full = bars + 17;                 // 2
  uint64_t* desc_empty = bars + 19;                // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kBarriers);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  ItemDesc* descs = reinterpret_cast<ItemDesc*>(tmem_slot + 2);     // [2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The blocks stay for the whole launch, two to an SM, and draw work items (a tile of queries of one KV head,
  // one share of its keys) from a counter.  The hardware would hand out a block per item as well, but not onto
  // an SM where another block of this kernel is at work: while a resident block writes tensor memory
  // (tcgen05.st: P, and O when it is rescaled), the SM is given no new block until that one has ended (measured
  // with variants of this kernel that left out the copies, the products, the loads or the stores of tensor
  // memory: only without the stores did a block start as soon as one of the two before it had ended).  With a
  // block per item every pair of blocks therefore ran as long as its longer one.
  //
  // The copy warp draws the items, works out what each is (request, tokens, keys) and hands that to the other
  // warps through a ring of two descriptors; since it runs up to two key tiles ahead of them, it draws the next
  // item while the current one is at its last tiles, and has that item's queries and first keys in shared
  // memory by the time the softmax warps have written the current one's output.  Barriers are initialised
  // once: buffers and phases are counted on from item to item (every warp keeps the same counts).
  //
  // Set-up that needs nothing of the step's data comes before the wait for the kernel in front.
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_q)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&k_full[b], 1); mbar_init(&k_empty[b], 1);
      mbar_init(&v_full[b], 1); mbar_init(&v_empty[b], 1);
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], 4);
      mbar_init(&desc_full[b], 1);
      mbar_init(&desc_empty[b], 5);                 // the product warp and the four softmax warps
    }
    mbar_init(o_full, 1);
    mbar_init(o_done, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  pdl_launch_dependents();
  pdl_wait();             // the counter is read only after this: the launch before this one has left it at zero
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  const int slots = p.n_z;                                  // shares that the scratch memory has room for

  int q_armed = 0, k_armed = 0, v_armed = 0;                // copies the copy warp has asked for (for the drain)
  if (warp == 4) {
    // ---------------------------------- items and TMA copies -----------------------------------
    // Lane 0 waits for free buffers and arms the barriers; lane c issues box c of a tile (with small pages one
    // thread would spend longer issuing them than they take).  A tile is fetched in boxes of min(page, BN) keys:
    // several pages, or a part of one.
    const int page_shift = 31 - __clz(p.page_size);                 // pages are powers of two
    const int box_shift = min(page_shift, 6);
    const int my_box = lane / (HS / 64), my_half = lane - my_box * (HS / 64);
    const int box_rows = 1 << box_shift;
    const int boxes_per_tile = BN >> box_shift;
    const uint32_t box_bytes = (uint32_t)box_rows * HS * 2;         // my_box, my_half: boxes_per_tile * H2 <= 16 lanes have a box
    const bool count_single = !(p.skip_single && slots == 1);
    uint32_t T = 0;                                         // key tiles handed on so far
    int n = 0;                                              // items handed on so far
    bool ok = true;
    while (ok) {
      int item = 0;
      if (lane == 0) item = atomicAdd(p.work, 1);
      item = __shfl_sync(0xffffffffu, item, 0);
      if (item >= p.n_items) break;
      // Items are numbered share by share, within a share tile by tile with the KV heads of a tile of queries as
      // neighbours, and later tiles, which see more keys, first, so that the light ones fill the tail.  The
      // request of the item's tile is found by adding up the requests' tiles, 32 requests at a time (the launch
      // counts tiles of the whole step, an upper bound that the host can give without the requests' lengths).
      const int split = item / p.items_per_share, in_share = item - split * p.items_per_share;
      const int kvh = in_share % p.g;
      const int flat = p.items_per_share / p.g - 1 - in_share / p.g;
      int req = -1, tile_in_req = 0;
      for (int c = 0, seen = 0; c < p.n_requests; c += 32) {
        int tiles = 0;
        if (c + lane < p.n_requests) {
          const int q = p.q_start[c + lane + 1] - p.q_start[c + lane];
          tiles = (q == 1 && !count_single) ? 0 : (q + p.tokens_per_tile - 1) / p.tokens_per_tile;
        }
        int upto = tiles;                                     // tiles of requests c .. c + lane
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int below = __shfl_up_sync(0xffffffffu, upto, o);
          if (lane >= o) upto += below;
        }
        const int total = __shfl_sync(0xffffffffu, upto, 31);
        if (flat < seen + total) {                            // uniform: flat, seen and total are
          const int owner = __ffs(__ballot_sync(0xffffffffu, seen + upto > flat)) - 1;
          req = c + owner;
          tile_in_req = flat - seen - __shfl_sync(0xffffffffu, upto - tiles, owner);
          break;
        }
        seen += total;
      }
      if (req < 0) continue;                                  // past the step's last tile
      const int32_t* bt = p.block_table + (size_t)req * p.table_width;
      // The loads below are issued back to back: two round trips to memory (token range and first pages; then
      // positions) stand between the draw of an item and its first copy, not four.
      int early_page = -2;                                    // this lane's page of tile 0 (known before the positions are)
      if (slots == 1) {
        const int pi = (my_box << box_shift) >> page_shift;
        early_page = (my_box < boxes_per_tile && pi < p.table_width) ? bt[pi] : -1;
      }
      const int tok0 = p.q_start[req], q_len = p.q_start[req + 1] - tok0;
      const int t0 = tile_in_req * p.tokens_per_tile;         // first token of this item within the request
      if (p.skip_single && q_len == 1) {
        // Another kernel writes this request's row; with key splits the second kernel must leave it alone.
        if (slots > 1 && split == 0)
          for (int h = lane; h < p.per; h += 32)
            *reinterpret_cast<float2*>(p.part_ml + (((size_t)tok0 * p.nh + kvh * p.per + h) * slots) * 2) =
                make_float2(INFINITY, 0.f);
        continue;
      }
      const int n_tok = min(p.tokens_per_tile, q_len - t0);
      const int n_rows = n_tok * p.per;
      const int pos_first = p.positions[tok0 + t0];
      const int hi_key = p.positions[tok0 + t0 + n_tok - 1];
      // This item's share of the key tiles (all of them without splits).
      const int all_tiles = hi_key / BN + 1;
      const int wanted = slots > 1 ? min(slots, (all_tiles + p.tiles_per_split - 1) / p.tiles_per_split) : 1;
      const int per_split = (all_tiles + wanted - 1) / wanted;
      const int n_splits = (all_tiles + per_split - 1) / per_split;   // shares that get a tile (7 tiles in 5 shares: 4 of 2)
      if (split >= n_splits) {
        if (n_splits > 1)                                     // an unused share of a divided tile: nothing to add
          for (int r = lane; r < n_rows; r += 32) {
            const int t_in = r / p.per, head = r - t_in * p.per;
            const size_t slot = ((size_t)(tok0 + t0 + t_in) * p.nh + kvh * p.per + head) * slots + split;
            *reinterpret_cast<float2*>(p.part_ml + slot * 2) = make_float2(-INFINITY, 0.f);
          }
        continue;
      }
      const int tile_base = split * per_split;
      const int n_tiles = min(all_tiles, tile_base + per_split) - tile_base;     // >= 1
#ifdef YALIS_TRACE_CLOCKS
      const int trace_row = in_share;
#endif

      // Hand the item on: the others are through with the item before the one before.
      const int d = n & 1;
      if (!warp_wait(&desc_empty[d], ((n >> 1) & 1) ^ 1, abort_flag, lane)) { ok = false; break; }
      if (lane == 0) {
        ItemDesc& it = descs[d];
        it.n_tiles = n_tiles; it.tile_base = tile_base; it.n_splits = n_splits; it.split = split; it.kvh = kvh;
        it.tok_first = tok0 + t0; it.n_rows = n_rows; it.pos_first = pos_first; it.hi_key = hi_key;
        it.trace_row = in_share;
        mbar_arrive(&desc_full[d]);
        // Q, once the products of the item before, which read it, are done.
        ok = mbar_wait(q_empty, (n & 1) ^ 1, abort_flag);
        if (ok) {
          mbar_expect_tx(q_full, (uint32_t)(p.tokens_per_tile * p.per) * HS * 2);
#pragma unroll
          for (int h = 0; h < H2; ++h)
            tma_load_3d(q_s + h * (BM * 128), &map_q, h * 64, kvh * p.per, tok0 + t0, q_full);
          q_armed = n + 1;
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      // Row of this lane's box of tile j in the pool seen as a matrix (K and V pools are laid out alike), or -1.
      auto box_row = [&](int j) -> int {
        const int key = ((tile_base + j) << 6) + (my_box << box_shift);
        if (j >= n_tiles || my_box >= boxes_per_tile || key > hi_key) return -1;
        const int pi = key >> page_shift;
        int page = (j == 0 && early_page != -2) ? early_page : (pi < p.table_width ? bt[pi] : -1);
        if (page < 0 || page >= p.num_pages) {
          if (p.error) atomicOr(p.error, YALIS_FLAG_BAD_PAGE);
          page = 0;
        }
        return ((page * p.g + kvh) << page_shift) + (key & (p.page_size - 1));
      };
      auto fetch = [&](int j, int kv, int y) {
        const int b = (T + j) & 1;
        const uint32_t ph = ((T + j) >> 1) & 1;
        const int n_boxes = min(boxes_per_tile, ((hi_key - ((tile_base + j) << 6)) >> box_shift) + 1);
        uint64_t* full = kv == 0 ? &k_full[b] : &v_full[b];
        uint64_t* empty = kv == 0 ? &k_empty[b] : &v_empty[b];
        int go = 1;
        if (lane == 0) {
          go = mbar_wait(empty, ph ^ 1, abort_flag) ? 1 : 0;
          if (go) mbar_expect_tx(full, box_bytes * (uint32_t)n_boxes);
        }
        go = __shfl_sync(0xffffffffu, go, 0);
        if (!go) { ok = false; return; }
        if (lane == 0) STAMP(j, 30 + kv);
        if (y >= 0)
          tma_load_2d((kv == 0 ? k_s : v_s) + b * KV_BYTES + my_half * (BN * 128) + my_box * box_rows * 128,
                      kv == 0 ? &map_k : &map_v, my_half * 64, y, full);
        __syncwarp();
        if (kv == 0) k_armed = (int)T + j + 1; else v_armed = (int)T + j + 1;
      };
      // K runs one tile ahead of V (their buffers come free in that order: QK(j-1), then PV(j-2)); the pages of
      // a tile are looked up a tile before its K is asked for.
      int y_v = box_row(0);
      fetch(0, 0, y_v);                                       // the first keys are on their way before anything else is looked up
      int y_k = box_row(1), y_ahead = box_row(2);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) fetch(j + 1, 0, y_k);
        if (ok) fetch(j, 1, y_v);
        y_v = y_k;
        y_k = y_ahead;
        y_ahead = box_row(j + 3);
      }
      T += (uint32_t)n_tiles;
      ++n;
    }
    // No more items: tell the others (unless something gave up; then they find out from the flag).
    if (ok) {
      const int d = n & 1;
      if (warp_wait(&desc_empty[d], ((n >> 1) & 1) ^ 1, abort_flag, lane) && lane == 0) {
        descs[d].n_tiles = -1;
        mbar_arrive(&desc_full[d]);
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ---------------------------------- MMA issuer --------------------------------------------
    // The whole warp runs the loop and every lane waits on the barriers itself; the elected lane issues.  (With
    // one lane polling for the warp, blocks of four and more key tiles ran into their bounded waits.)
    const uint32_t elected = elect_one();
    const uint32_t idesc_qk = idesc_f16(BN, false), idesc_pv = idesc_f16(HS, true);
    const uint64_t q_desc = desc_kmajor(smem_u32(q_s));
    const uint64_t k_desc0 = desc_kmajor(smem_u32(k_s));
    const uint64_t v_desc0 = desc_mnmajor(smem_u32(v_s), BN * 128);
    uint32_t T = 0;
    bool ok = true;
    for (int n = 0; ok; ++n) {
      const int d = n & 1;
      if (!mbar_wait(&desc_full[d], (n >> 1) & 1, abort_flag)) break;
      const int n_tiles = descs[d].n_tiles;
      if (n_tiles < 0) break;
#ifdef YALIS_TRACE_CLOCKS
      const int trace_row = descs[d].trace_row;
#endif
      ok = mbar_wait(q_full, n & 1, abort_flag);
      if (lane == 0) STAMP(63, 3);
      auto issue_qk = [&](int j) -> bool {
        const int b = (T + j) & 1;
        const uint32_t ph = ((T + j) >> 1) & 1;
        // The S buffer is free: the wait for P(j-2), which lay in it, came after every softmax thread had read
        // S(j-2), and the product that read P(j-2) was issued before this one (products run in issue order).
        if (!mbar_wait(&k_full[b], ph, abort_flag)) return false;
        if (lane == 0 && j > 0) STAMP(j - 1, 11);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t k_desc = k_desc0 + (uint64_t)((b * KV_BYTES) >> 4);
#pragma unroll
        for (int ks = 0; ks < HS / 16; ++ks) {
          // 64-dim half (BM rows of Q, BN rows of K, 128 bytes each), then 32 bytes per 16 dims; the address
          // field of a descriptor counts 16-byte units
          const uint32_t q_off = (ks >> 2) * (BM * 128) + (ks & 3) * 32, k_off = (ks >> 2) * (BN * 128) + (ks & 3) * 32;
          umma_ss(elected, tmem + COL_S + b * BN, q_desc + (q_off >> 4), k_desc + (k_off >> 4), idesc_qk, ks > 0);
        }
        umma_commit(elected, &s_full[b]);
        umma_commit(elected, &k_empty[b]);
        if (j == n_tiles - 1) umma_commit(elected, q_empty);     // the item's last reader of Q
        return true;
      };
      if (ok) ok = issue_qk(0);
      if (lane == 0) STAMP(63, 4);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int b = (T + j) & 1;
        const uint32_t ph = ((T + j) >> 1) & 1;
        if (lane == 0) STAMP(j, 6);
        if (j + 1 < n_tiles) ok = issue_qk(j + 1);
        if (!ok) break;
        if (lane == 0) STAMP(j, 7);
        if (!mbar_wait(&v_full[b], ph, abort_flag)) { ok = false; break; }
        if (lane == 0) STAMP(j, 8);
        // P(j) written, O rescaled if needed.  For the item's first tile this also says that every softmax warp
        // has read the O of the item before: a warp arrives here only after its part of that output is written.
        if (!mbar_wait(&p_full[b], ph, abort_flag)) { ok = false; break; }
        if (lane == 0) STAMP(j, 9);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t v_desc = v_desc0 + (uint64_t)((b * KV_BYTES) >> 4);
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
          // 16 keys = two 8-key swizzle groups = 2048 bytes further; P: 16 bfloat16 = 8 columns further
          umma_ts(elected, tmem + COL_O, tmem + COL_S + b * BN + ks * 8, v_desc + ((ks * 2048) >> 4), idesc_pv,
                  (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(elected, o_full);
        umma_commit(elected, &v_empty[b]);
        if (lane == 0) STAMP(j, 10);
      }
      if (!ok) break;
      umma_commit(elected, o_done);
      T += (uint32_t)n_tiles;
      __syncwarp();
      if (lane == 0) mbar_arrive(&desc_empty[d]);
    }
    __syncwarp();
  } else {
    // ---------------------------------- softmax, one thread per row ----------------------------
    const int r = threadIdx.x;                        // row of the tile = tensor-memory lane
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    uint32_t T = 0;
    bool ok = true;
    for (int n = 0; ok; ++n) {
      const int d = n & 1;
      if (!warp_wait(&desc_full[d], (n >> 1) & 1, abort_flag, lane)) break;
      const int n_tiles = descs[d].n_tiles;
      if (n_tiles < 0) break;
      const int tile_base = descs[d].tile_base, n_splits = descs[d].n_splits, split = descs[d].split;
      const int kvh = descs[d].kvh, tok_first = descs[d].tok_first, n_rows = descs[d].n_rows;
      const int pos_first = descs[d].pos_first, hi_key = descs[d].hi_key;
#ifdef YALIS_TRACE_CLOCKS
      const int trace_row = descs[d].trace_row;
      if (threadIdx.x == 0) { STAMP(63, 0); GSTAMP(0); }
#endif
      const bool valid = r < n_rows;
      const int t_in = r / p.per, head = r - t_in * p.per;
      const int pos_row = valid ? p.positions[tok_first + t_in] : -1;
      float m_run = -INFINITY, l_run = 0.f;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int b = (T + j) & 1;
        const uint32_t ph = ((T + j) >> 1) & 1;
        const int key0 = (tile_base + j) * BN;
        if (lane == 0) STAMP(j, 0 + (warp ? 6 + warp * 6 : 0));
        if (!warp_wait(&s_full[b], ph, abort_flag, lane)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (lane == 0) STAMP(j, 1 + (warp ? 6 + warp * 6 : 0));
        float sv[BN];
        {
          const uint32_t s_addr = lane_base + COL_S + b * BN;
#pragma unroll
          for (int c0 = 0; c0 < BN; c0 += 32) tmem_ld32(s_addr + c0, *reinterpret_cast<uint32_t(*)[32]>(&sv[c0]));
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        }
        // S is in registers now; its buffer is written again only after P(j), which takes its place, has been used.
        if (lane == 0) STAMP(j, 2 + (warp ? 6 + warp * 6 : 0));
        if (key0 + BN - 1 > pos_first || !valid) {           // some key of the tile is hidden from this row
#pragma unroll
          for (int c = 0; c < BN; ++c)
            if (!valid || key0 + c > pos_row) sv[c] = -INFINITY;
        }
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < BN; c += 8) {                    // four chains of three-input maxima
          mx[0] = max3(mx[0], sv[c], sv[c + 1]); mx[1] = max3(mx[1], sv[c + 2], sv[c + 3]);
          mx[2] = max3(mx[2], sv[c + 4], sv[c + 5]); mx[3] = max3(mx[3], sv[c + 6], sv[c + 7]);
        }
        const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
        const float m_new = fmaxf(m_run, m_tile);
        if (lane == 0) STAMP(j, 3 + (warp ? 6 + warp * 6 : 0));
        // Keep the older maximum unless the new one is more than 2^8 larger: exp2 of at most 8 is
        // harmless in float32 and bfloat16, and O then needs no rescaling.
        const bool grow = (m_new - m_run > 8.0f) || (m_run == -INFINITY && m_new != -INFINITY);
        const float m_use = grow ? m_new : m_run;
        const float mb = (m_use == -INFINITY) ? 0.f : m_use;
        const float corr = grow ? ((m_run == -INFINITY) ? 0.f : ex2(m_run - mb)) : 1.f;
        uint64_t ls2[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
        const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), nmb2 = pack2(-mb, -mb);
        const uint32_t p_addr = lane_base + COL_S + b * BN;          // over the first half of S(j)
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            // scale and shift, and the row sums, two values to an instruction
            float x0, x1, x2, x3;
            unpack2(fma2(pack2(sv[c0 + c], sv[c0 + c + 1]), scale2, nmb2), x0, x1);
            unpack2(fma2(pack2(sv[c0 + c + 2], sv[c0 + c + 3]), scale2, nmb2), x2, x3);
            const float p0 = ex2(x0), p1 = ex2(x1), p2 = ex2(x2), p3 = ex2(x3);
            ls2[0] = add2(ls2[0], pack2(p0, p1));
            ls2[1] = add2(ls2[1], pack2(p2, p3));
            pk[c >> 1] = pack_bf16(p0, p1);
            pk[(c >> 1) + 1] = pack_bf16(p2, p3);
          }
          tmem_st16(p_addr + (c0 >> 1), pk);
        }
        float ls[4];
        unpack2(ls2[0], ls[0], ls[1]);
        unpack2(ls2[1], ls[2], ls[3]);
        l_run = l_run * corr + ((ls[0] + ls[1]) + (ls[2] + ls[3]));
        if (lane == 0) STAMP(j, 4 + (warp ? 6 + warp * 6 : 0));
        m_run = m_use;
        // Rescale O in place if some row of this warp moved its maximum (never for the first tile).
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          if (!warp_wait(o_full, (T + j - 1) & 1, abort_flag, lane)) { ok = false; break; }     // P V of tile j-1 is done
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
          for (int c0 = 0; c0 < HS; c0 += 16) {
            uint32_t o[16];
            tmem_ld16(lane_base + COL_O + c0, o);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int c = 0; c < 16; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * corr);
            tmem_st16(lane_base + COL_O + c0, o);
          }
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        if (key0 + BN - 1 > hi_key) {
          // Last tile: rows of V past the last visible key may hold anything (even NaN); zero them
          // once the tile has landed, and make the writes visible to the tensor core's reads.
          if (!warp_wait(&v_full[b], ph, abort_flag, lane)) { ok = false; break; }
          if (r < BN && key0 + r > hi_key) {
            unsigned char* vt = v_s + b * KV_BYTES;
#pragma unroll
            for (int h = 0; h < H2; ++h)
#pragma unroll
              for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(vt + h * (BN * 128) + r * 128 + c * 16) = make_uint4(0u, 0u, 0u, 0u);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[b]);
        if (lane == 0) STAMP(j, 5 + (warp ? 6 + warp * 6 : 0));
      }
      // ---- O / l -> global --------------------------------------------------------------------
      if (ok) ok = warp_wait(o_done, n & 1, abort_flag, lane);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (n_splits > 1) {
        // a share: unnormalised, with the maximum it is relative to and its sum
        const size_t slot = ((size_t)(tok_first + (valid ? t_in : 0)) * p.nh + kvh * p.per + (valid ? head : 0)) * slots + split;
        float* dst = p.part_o + slot * HS;
        if (valid) *reinterpret_cast<float2*>(p.part_ml + slot * 2) = make_float2(m_run, l_run);
#pragma unroll 1
        for (int c0 = 0; c0 < HS; c0 += 16) {
          uint32_t o[16];
          tmem_ld16(lane_base + COL_O + c0, o);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (valid) {
#pragma unroll
            for (int c = 0; c < 16; c += 4)
              *reinterpret_cast<uint4*>(dst + c0 + c) = make_uint4(o[c], o[c + 1], o[c + 2], o[c + 3]);
          }
        }
      } else {
        if (slots > 1 && valid) {                             // finished here: the second kernel leaves these rows alone
          const size_t slot = ((size_t)(tok_first + t_in) * p.nh + kvh * p.per + head) * slots;
          *reinterpret_cast<float2*>(p.part_ml + slot * 2) = make_float2(INFINITY, 0.f);
        }
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
        __nv_bfloat16* dst = p.out + (size_t)(tok_first + (valid ? t_in : 0)) * p.out_stride +
                             (size_t)(kvh * p.per + (valid ? head : 0)) * HS;
#pragma unroll 1
        for (int c0 = 0; c0 < HS; c0 += 16) {
          uint32_t o[16];
          tmem_ld16(lane_base + COL_O + c0, o);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (valid) {
            uint4 v0, v1;
            v0.x = pack_bf16(__uint_as_float(o[0]) * inv, __uint_as_float(o[1]) * inv);
            v0.y = pack_bf16(__uint_as_float(o[2]) * inv, __uint_as_float(o[3]) * inv);
            v0.z = pack_bf16(__uint_as_float(o[4]) * inv, __uint_as_float(o[5]) * inv);
            v0.w = pack_bf16(__uint_as_float(o[6]) * inv, __uint_as_float(o[7]) * inv);
            v1.x = pack_bf16(__uint_as_float(o[8]) * inv, __uint_as_float(o[9]) * inv);
            v1.y = pack_bf16(__uint_as_float(o[10]) * inv, __uint_as_float(o[11]) * inv);
            v1.z = pack_bf16(__uint_as_float(o[12]) * inv, __uint_as_float(o[13]) * inv);
            v1.w = pack_bf16(__uint_as_float(o[14]) * inv, __uint_as_float(o[15]) * inv);
            *reinterpret_cast<uint4*>(dst + c0) = v0;
            *reinterpret_cast<uint4*>(dst + c0 + 8) = v1;
          }
        }
      }
#ifdef YALIS_TRACE_CLOCKS
      if (threadIdx.x == 0) {
        GSTAMP(1);
        unsigned sm_;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(sm_));
        if (p.trace) p.trace[((size_t)trace_row * 64 + 62) * 32 + 2] = sm_ + 1;
      }
#endif
      T += (uint32_t)n_tiles;
      // The O of this item is in registers or written: the next item's first P V may overwrite it (it waits for
      // this warp's next arrival at p_full, which comes after this point).
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&desc_empty[d]);
    }
  }

  // ---- exit: drain on abort, hand the counter back, free tensor memory -------------------------------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 4 * 32) {
      if (p.error) atomicOr(p.error, YALIS_FLAG_WAIT_ATTENTION);
      // copies that were asked for and may not have been waited for
      if (q_armed > 0)
        for (uint32_t i = 0; i < kSpinLimit; ++i)
          if (mbar_try_wait(q_full, (q_armed - 1) & 1)) break;
      for (int j = max(0, k_armed - 2); j < k_armed; ++j)
        for (uint32_t i = 0; i < kSpinLimit; ++i)
          if (mbar_try_wait(&k_full[j & 1], (j >> 1) & 1)) break;
      for (int j = max(0, v_armed - 2); j < v_armed; ++j)
        for (uint32_t i = 0; i < kSpinLimit; ++i)
          if (mbar_try_wait(&v_full[j & 1], (j >> 1) & 1)) break;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    // Every block comes here once, after it has drawn a number past the last item or given up; the last to do
    // so leaves both counters at zero for the next launch.
    __threadfence();
    if (atomicAdd(p.work + 1, 1) == (int)gridDim.x - 1) {
      p.work[0] = 0;
      p.work[1] = 0;
      __threadfence();
    }
  }
  if (warp == 5) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// The pool [pages, g, page_size, hs] as a matrix [pages*g*page_size, hs]; boxes of [page_size rows, 64 columns].
bool make_pool_map(CUtensorMap* map, const void* pool, long long rows, int hs, int page_size) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {(cuuint64_t)hs, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)hs * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)(page_size < BN ? page_size : BN)};   // a page, or the part of one that a tile covers
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// q [N, q_stride] with head h at column h*hs, seen as [tokens][heads][hs]; a box is
// [tokens_per_tile][heads_per_group][64 columns], i.e. the rows of a tile in (token, head) order.
bool make_q_map(CUtensorMap* map, const void* q, long long n_tokens, int q_stride, int nh, int hs, int per,
                int tokens_per_tile) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[3] = {(cuuint64_t)hs, (cuuint64_t)nh, (cuuint64_t)n_tokens};
  cuuint64_t strides[2] = {(cuuint64_t)hs * 2, (cuuint64_t)q_stride * 2};
  cuuint32_t box[3] = {64u, (cuuint32_t)per, (cuuint32_t)tokens_per_tile};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Adds the shares of every (token, head) that was divided: one block per token, a thread per four output columns.
__global__ void prefill_merge_splits_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                            __nv_bfloat16* __restrict__ out, int out_stride, int nh, int hs, int n_splits) {
  pdl_launch_dependents();
  pdl_wait();
  const int tok = blockIdx.x, vec = hs / 4;
  for (int e = threadIdx.x; e < nh * vec; e += blockDim.x) {
    const int head = e / vec, d = (e - head * vec) * 4;
    const size_t slot0 = ((size_t)tok * nh + head) * n_splits;
    if (part_ml[slot0 * 2] == INFINITY) continue;        // written by the first kernel itself
    float mm = -INFINITY;
    for (int sp = 0; sp < n_splits; ++sp) mm = fmaxf(mm, part_ml[(slot0 + sp) * 2]);
    float ll = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sp = 0; sp < n_splits; ++sp) {              // in split order
      const float2 ml = *reinterpret_cast<const float2*>(part_ml + (slot0 + sp) * 2);
      if (ml.x == -INFINITY) continue;                   // a split without visible keys wrote no output
      const float f = exp2f(ml.x - mm);
      const float4 v = *reinterpret_cast<const float4*>(part_o + (slot0 + sp) * hs + d);
      ll += ml.y * f;
      acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
    }
    const float inv = ll > 0.f ? 1.0f / ll : 0.f;
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv), hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    uint2 w;
    w.x = *reinterpret_cast<unsigned*>(&lo);
    w.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(out + (size_t)tok * out_stride + (size_t)head * hs + d) = w;
  }
}

template <int HS>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const PrefillParams& p, int n_splits,
           int n_tokens, cudaStream_t stream) {
  const size_t smem = 1024 + (size_t)BM * HS * 2 + (size_t)4 * BN * HS * 2 + kBarriers * 8 + 8 + 2 * sizeof(ItemDesc);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(prefill_attention_tcgen05_kernel<HS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return YALIS_ERR_LAUNCH;
    configured = true;
  }
  // Two blocks to an SM for the whole launch (fewer if the step has fewer items).
  dim3 grid((unsigned)std::min<long long>(p.n_items, 2LL * yalis_sm_count()), 1, 1);
  int st = yalis_launch(prefill_attention_tcgen05_kernel<HS>, grid, dim3(kThreads), smem, stream, mq, mk, mv, p);
  if (st != YALIS_OK || n_splits == 1) return st;
  return yalis_launch(prefill_merge_splits_kernel, dim3(n_tokens), dim3(256), 0, stream, (const float*)p.part_o,
                      (const float*)p.part_ml, p.out, p.out_stride, p.nh, HS, n_splits);
}

}  // namespace

#ifdef YALIS_TRACE_CLOCKS
YALIS_API int yalis_prefill_gave_up(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, g_gave_up, sizeof(g_gave_up)) == cudaSuccess ? 0 : -1;
}
#endif

YALIS_API int yalis_prefill_attention_tcgen05_supports(int hs, int page_size, int per) {
  const bool page_ok = page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128;
  return ((hs == 64 || hs == 128) && page_ok && per >= 1 && per <= 128) ? 1 : 0;
}

// Floats of scratch memory for n_splits > 1.
YALIS_API long long yalis_prefill_attention_tcgen05_scratch_floats(int n_tokens, int nh, int hs, int n_splits) {
  return (long long)n_tokens * nh * n_splits * (hs + 2);
}

// q: [N, q_stride] (head h at column h*hs); out [N, out_stride].  error: device int32 raised on a timed-out
// wait or an unmapped page.  No window.  With n_splits > 1 a tile of queries that sees more than tiles_per_split
// tiles of 64 keys has them divided among ceil(tiles / tiles_per_split) blocks, at most n_splits (long contexts:
// too few tiles of queries to fill the GPU evenly, or a few of them with far more keys than the rest); it needs
// scratch: yalis_prefill_attention_tcgen05_scratch_floats floats, and every token row of [0, n_tokens) must then
// belong to a request.  skip_single = 1 leaves the rows of requests that bring one token unwritten (a decode
// kernel takes them).  work: two int32 that are zero and that no other launch uses at the same time (the kernel
// counts its work items in them and leaves them at zero).
YALIS_API int yalis_prefill_attention_tcgen05(const void* q, int q_stride, void* out, int out_stride, const void* k_pool,
                                              const void* v_pool, const int32_t* positions, const int32_t* q_start,
                                              const int32_t* block_table, int table_width, int page_size,
                                              int num_pages, int n_tokens, int n_requests, int max_q_len, int nh,
                                              int g, int hs, float scale, int n_splits, int tiles_per_split, int skip_single,
                                              float* scratch, int32_t* work, int32_t* error, cudaStream_t stream
#ifdef YALIS_TRACE_CLOCKS
                                              , long long* trace
#endif
) {
  if (n_tokens <= 0 || n_requests <= 0) return YALIS_OK;
  if (g <= 0 || nh % g != 0 || max_q_len < 1 || n_splits < 1 || n_splits > 64) return YALIS_ERR_SHAPE;
  if (n_splits > 1 && (scratch == nullptr || ((uintptr_t)scratch & 15))) return YALIS_ERR_ALIGN;
  if (n_splits > 1 && tiles_per_split < 1) return YALIS_ERR_SHAPE;
  if (work == nullptr) return YALIS_ERR_ALIGN;
  if (!yalis_prefill_attention_tcgen05_supports(hs, page_size, nh / g)) return YALIS_ERR_SHAPE;
  if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15) return YALIS_ERR_ALIGN;
  if ((q_stride % 8) || (out_stride % 8)) return YALIS_ERR_ALIGN;
  PrefillParams p;
  p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.positions = positions; p.q_start = q_start; p.block_table = block_table;
  p.table_width = table_width; p.page_size = page_size; p.num_pages = num_pages;
  p.nh = nh; p.g = g; p.per = nh / g;
  p.n_requests = n_requests;
  p.tokens_per_tile = BM / p.per;
  {
    // Tiles of queries in the step: sum of ceil(q / tokens_per_tile) over the requests, bounded from their
    // number, the step's tokens and the longest request.
    const long long tpt = p.tokens_per_tile;
    const long long tiles = std::min(((long long)n_tokens + (long long)n_requests * (tpt - 1)) / tpt,
                                     (long long)n_requests * ((max_q_len + tpt - 1) / tpt));
    if (tiles * g * n_splits > 0x7fffffffLL) return YALIS_ERR_SHAPE;
    p.items_per_share = (int)(tiles * g);
    p.n_z = n_splits;
    p.n_items = p.items_per_share * n_splits;
  }
  p.work = work;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.tiles_per_split = tiles_per_split > 0 ? tiles_per_split : 1;
  p.skip_single = skip_single ? 1 : 0;
  p.part_o = scratch;
  p.part_ml = scratch ? scratch + (size_t)n_tokens * nh * n_splits * hs : nullptr;
  p.error = error;
#ifdef YALIS_TRACE_CLOCKS
  p.trace = trace;
#endif
  CUtensorMap mq, mk, mv;
  const long long rows = (long long)num_pages * g * page_size;
  if (!make_q_map(&mq, q, n_tokens, q_stride, nh, hs, p.per, p.tokens_per_tile) ||
      !make_pool_map(&mk, k_pool, rows, hs, page_size) || !make_pool_map(&mv, v_pool, rows, hs, page_size))
    return YALIS_ERR_LAUNCH;
  return hs == 64 ? launch<64>(mq, mk, mv, p, n_splits, n_tokens, stream)
                  : launch<128>(mq, mk, mv, p, n_splits, n_tokens, stream);
}
