// y = x W^T for few tokens (1..256) on the 5th-generation tensor cores: the
// weight-streaming product of decode steps.
//
// The product is computed transposed ("swap-AB"): a block owns 128 rows of W
// [N, K] as the M side of tcgen05.mma (cta_group::1, kind::f16, bfloat16 in,
// float32 accumulation in tensor memory) and the tokens, padded to NTOK in
// {16, 32, 64, 128, 256}, are the N side.  W is read from HBM exactly once:
// one elected thread streams 128x64 tiles of it (and the matching NTOKx64 tiles
// of x, which stay in L2) with TMA (cp.async.bulk.tensor, 128-byte swizzle) into
// a ring of shared-memory stages guarded by mbarriers; a second elected thread
// issues four K=16 MMAs per stage and releases the stage with tcgen05.commit;
// four epilogue warps read the 128 x NTOK accumulator from tensor memory with
// tcgen05.ld and store it transposed, so that a warp writes 32 consecutive
// outputs of one token.
//
// Outputs with few 128-row tiles (N = 4096 gives 32) cannot fill 148 SMs, so the
// K range is divided among `splits` blocks per tile; with splits > 1 each block
// writes a float32 partial [split, M, N] and the consumer (the fused residual
// add + norm, or the rotary kernel) sums the partials in split order, which
// keeps the result deterministic.
//
// Every wait on an mbarrier is bounded: after kSpinLimit failed polls a thread
// raises the block's abort flag and the global error word, all roles leave
// their loops, outstanding TMA transactions are waited for (bounded again),
// tensor memory is freed and the block returns.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace {

constexpr int TILE_N = 128;      // weight rows per block (MMA M)
constexpr int TILE_K = 64;       // bfloat16 elements per stage along K: one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;    // warp 0: TMA, warp 1: MMA + tensor memory, warps 2-5: epilogue
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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
// Bounded wait; false (and the abort flag raised) if the phase never completed.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// The same with an L2 eviction policy (weights are read once: evict first; the x tile is read by every block: keep).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes,
// groups of 8 rows 1024 bytes apart, descriptor version 1 (Blackwell).
__device__ __forceinline__ uint64_t umma_desc_sw128(const void* smem) {
  const uint64_t addr = smem_u32(smem);
  return ((addr >> 4) & 0x3FFFull) | (1ull << 16) | ((1024ull >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor of kind::f16: D float32, A and B bfloat16, both K-major, M = 128, N = ntok.
__device__ __forceinline__ uint32_t umma_idesc(int ntok) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ntok >> 3) << 17) | ((uint32_t)(TILE_N >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}


struct GemmParams {
  void* out;            // splits == 1: [M, N] of out_dtype; splits > 1: float32 [splits, M, N]
  int out_dtype;
  long long ldo;        // row stride of out in elements
  int M, N, K;
  int splits;
  int kt_per_split;     // stage steps (of 64 or 128 columns of K) per split
  int silu_inter;       // 0, or I: w is [gate (I rows); up (I rows)] and out[m, i] = silu(gate_i) * up_i, [M, I] bfloat16
  int32_t* error;       // YALIS_FLAG_WAIT_PRODUCT is raised in it if a wait ran out
};

// Ring depth. A stage is 16 KB of W plus NTOK * 128 bytes of x.  Two blocks fit an SM with ~95 KB each, so that
// grids between one and two blocks per SM run as one wave.  (A ring of a whole SM for grids of at most one block
// per SM is faster for a product alone, but slower inside a decode step: the next kernel's blocks then find no
// room beside it and cannot fetch ahead.  Measured 3.28 against 3.33 ms for a batch-8 step of Llama-3-8B.)
// K blocks of 64 per stage: two for up to 16 tokens (32 KB of W per stage and barrier round trip), else one.
template <int NTOK>
__host__ __device__ constexpr int kblocks_for() { return NTOK <= 16 ? 2 : 1; }
template <int NTOK>
__host__ __device__ constexpr int stages_for() {
  return NTOK <= 16 ? 3 : NTOK <= 32 ? 5 : NTOK <= 64 ? 4 : NTOK <= 128 ? 3 : 4;
}

// SILU: the gated-activation epilogue (p.silu_inter > 0).  A variant of its own: its extra registers would also
// be charged to the plain kernel, which then fits once instead of twice beside the attention blocks it follows.
template <int NTOK, bool SILU>
__global__ void __launch_bounds__(kThreads, NTOK > 128 ? 1 : 2)
gemm_wstream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const GemmParams p) {
  constexpr int STAGES = stages_for<NTOK>();
  constexpr int KB = kblocks_for<NTOK>();
  constexpr int A_SUB = TILE_N * TILE_K * 2, B_SUB = NTOK * TILE_K * 2;     // one K block of 64
  constexpr int A_BYTES = KB * A_SUB;
  constexpr int B_BYTES = KB * B_SUB;
  constexpr int TMEM_COLS = NTOK < 32 ? 32 : NTOK;
  extern __shared__ __align__(1024) unsigned char smem[];
  // The dynamic window is only guaranteed 16-byte aligned: round up to 1024 for the swizzled tiles.
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~uintptr_t(1023));
  unsigned char* a_s = base;                          // [STAGES][128][64] bf16, swizzled
  unsigned char* b_s = base + STAGES * A_BYTES;       // [STAGES][NTOK][64] bf16, swizzled
  uint64_t* full = reinterpret_cast<uint64_t*>(b_s + STAGES * B_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Plain: 128 rows of w from n0.  SiLU mode: 64 gate rows from n0 (tensor-memory lanes 0-63) and the 64
  // up rows of the same outputs, I further down (lanes 64-127); the map's box is 64 rows then.
  const int n0 = blockIdx.x * (SILU ? TILE_N / 2 : TILE_N);
  const int split = blockIdx.y;
  const int kt_total = (p.K + KB * TILE_K - 1) / (KB * TILE_K);      // stage steps of KB * 64 columns
  const int kt_begin = split * p.kt_per_split;
  const int kt_end = min(kt_total, kt_begin + p.kt_per_split);
  const int n_kt = max(0, kt_end - kt_begin);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = *tmem_slot;

  int armed = 0;   // producer: stages armed so far (for the drain on abort)
  if (warp == 0) {
    if (lane == 0) {
      // Weights do not depend on the kernel before this one: fill the ring with W tiles at once,
      // and only then wait for that kernel before the first read of x.
      const uint64_t pol_w = l2_policy_evict_first(), pol_x = l2_policy_evict_last();
      // K blocks past the end of K are filled with zeros by the copy (and still count their bytes).
      auto load_w = [&](int s, int kt) {
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
          const int k = ((kt_begin + kt) * KB + kb) * TILE_K;
          unsigned char* dst = a_s + s * A_BYTES + kb * A_SUB;
          if constexpr (SILU) {
            tma_load_2d_hint(dst, &map_w, k, n0, &full[s], pol_w);
            tma_load_2d_hint(dst + A_SUB / 2, &map_w, k, p.silu_inter + n0, &full[s], pol_w);
          } else {
            tma_load_2d_hint(dst, &map_w, k, n0, &full[s], pol_w);
          }
        }
      };
      auto load_x = [&](int s, int kt) {
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_2d_hint(b_s + s * B_BYTES + kb * B_SUB, &map_x, ((kt_begin + kt) * KB + kb) * TILE_K, 0, &full[s], pol_x);
      };
      const int n_pre = min(n_kt, STAGES);
      for (int kt = 0; kt < n_pre; ++kt) {
        mbar_expect_tx(&full[kt], A_BYTES + B_BYTES);
        load_w(kt, kt);
      }
      armed = n_pre;
      pdl_wait();
      for (int kt = 0; kt < n_pre; ++kt) load_x(kt, kt);
      // When this block is about to ask for its last tiles, the next kernel's blocks may be scheduled and fill
      // their own rings: earlier they would take bandwidth from tiles this kernel still waits for (and
      // registers and shared memory from its later blocks); later the hand-over shows.  Measured on a decode
      // step of the Llama-3-8B shape: 4 tiles ahead is best with 8 tokens, 0 to 2 with 64.
      constexpr int kTriggerAhead = NTOK <= 32 ? 4 / KB : 1;      // in stage steps
      bool released = false;
      if (n_kt - 1 - kTriggerAhead < n_pre) {        // a short K range: the steps that are left are already on their way
        pdl_launch_dependents();
        released = true;
      }
      for (int kt = n_pre; kt < n_kt; ++kt) {
        const int s = kt % STAGES;
        const uint32_t ph = (kt / STAGES) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, abort_flag)) break;
        mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
        load_w(s, kt);
        load_x(s, kt);
        armed = kt + 1;
        if (kt == n_kt - 1 - kTriggerAhead) {
          pdl_launch_dependents();
          released = true;
        }
      }
      if (!released) pdl_launch_dependents();
    }
    else pdl_wait();
    __syncwarp();
  } else if (warp == 1) {
    pdl_wait();
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(NTOK);
      int kt = 0;
      for (; kt < n_kt; ++kt) {
        const int s = kt % STAGES;
        const uint32_t ph = (kt / STAGES) & 1;
        if (!mbar_wait(&full[s], ph, abort_flag)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
          const uint64_t da = umma_desc_sw128(a_s + s * A_BYTES + kb * A_SUB);
          const uint64_t db = umma_desc_sw128(b_s + s * B_BYTES + kb * B_SUB);
#pragma unroll
          for (int j = 0; j < TILE_K / UMMA_K; ++j) {
            // 16 bfloat16 = 32 bytes further along K inside the swizzled row: +2 in the address field
            umma(tmem_d, da + 2 * j, db + 2 * j, idesc, (kt > 0 || kb > 0 || j > 0) ? 1u : 0u);
          }
        }
        umma_commit(&empty[s]);
      }
      if (kt == n_kt) umma_commit(acc_full);
    }
    __syncwarp();
  } else {
    // Epilogue: warp w may touch the 32 tensor-memory lanes of its quarter (w % 4).
    pdl_wait();
    const int q = warp & 3;
    int ok = 1;
    if (n_kt > 0 && lane == 0) ok = mbar_wait(acc_full, 0, abort_flag) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);      // one poller per warp, so the warp stays convergent
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if constexpr (SILU) {
      // the four warps meet at barriers below: they must agree on whether the accumulator is there
      uint32_t all_ok;
      asm volatile(
          "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, 2, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(all_ok) : "r"((uint32_t)ok) : "memory");
      ok = (int)all_ok;
    }
    if (SILU && ok) {
      // Warps 0 and 1 of the epilogue hold the gate rows, warps 2 and 3 the up rows of the same 64 outputs:
      // the up values cross through shared memory (the ring is free by now), 16 tokens at a time, two buffers.
      float* ex = reinterpret_cast<float*>(a_s);            // [2][16 tokens][64 outputs]
      const int col = (q & 1) * 32 + lane;                   // output within the tile
      const int n = n0 + col;
#pragma unroll
      for (int c0 = 0; c0 < NTOK; c0 += 16) {
        uint32_t r[16];
        tmem_ld16(tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        float* buf = ex + ((c0 >> 4) & 1) * (16 * 64);
        if (q >= 2) {
#pragma unroll
          for (int i = 0; i < 16; ++i) buf[i * 64 + col] = __uint_as_float(r[i]);
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (q < 2 && n < p.silu_inter) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int m = c0 + i;
            if (m < p.M) {
              // both factors rounded to bfloat16 first: the same bits as the unfused product followed by the
              // activation kernel
              const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[i])));
              const float u = __bfloat162float(__float2bfloat16_rn(buf[i * 64 + col]));
              reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + n] = __float2bfloat16_rn(silu_bf16_path(g) * u);
            }
          }
        }
      }
    } else if (!SILU && ok) {
      const int n = n0 + q * 32 + lane;
#pragma unroll
      for (int c0 = 0; c0 < NTOK; c0 += 16) {
        uint32_t r[16];
        if (n_kt > 0) {
          tmem_ld16(tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = 0u;
        }
        if (n < p.N) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int m = c0 + i;
            if (m < p.M) {
              const float v = __uint_as_float(r[i]);
              if (p.splits > 1) {
                reinterpret_cast<float*>(p.out)[((size_t)split * p.M + m) * (size_t)p.ldo + n] = v;
              } else if (p.out_dtype == YALIS_F32) {
                reinterpret_cast<float*>(p.out)[(size_t)m * p.ldo + n] = v;
              } else {
                reinterpret_cast<__nv_bfloat16*>(p.out)[(size_t)m * p.ldo + n] = __float2bfloat16_rn(v);
              }
            }
          }
        }
      }
    }
  }

  // ---- common exit: drain on abort, free tensor memory ---------------------------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) {
      atomicOr(p.error, YALIS_FLAG_WAIT_PRODUCT);
      // Wait (bounded) for every TMA transaction this block started, so none lands after exit.
      for (int kt = max(0, armed - STAGES); kt < armed; ++kt) {
        const int s = kt % STAGES;
        const uint32_t ph = (kt / STAGES) & 1;
        for (uint32_t i = 0; i < kSpinLimit; ++i)
          if (mbar_try_wait(&full[s], ph)) break;
      }
    }
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(TMEM_COLS));
  }
}

// ---- host side ------------------------------------------------------------------------------

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

// A 2-D bfloat16 matrix [rows, K] with row stride ld (elements), boxes of [box_rows, 64], 128-byte swizzle,
// out-of-range elements read as zero.
// Encoded maps are kept by what they describe: a step asks for the same few hundred (matrix, box) pairs again and
// again (weights never move, and the allocator hands activations the same addresses step after step), and one
// encoding costs the host more than the launch it serves.  A map describes addresses and shapes only, never
// contents, so a kept one stays valid while its key repeats.
struct MapKey {
  const void* ptr;
  long long rows, K, ld;
  int box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && K == o.K && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
    h ^= (size_t)k.rows * 0xC2B2AE3D27D4EB4Full + (size_t)k.K * 0x165667B19E3779F9ull + (size_t)k.ld * 31 + (size_t)k.box_rows;
    return h;
  }
};

bool make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, long long ld, int box_rows) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> kept;
  const MapKey key{ptr, rows, K, ld, box_rows};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = kept.find(key);
    if (it != kept.end()) {
      *map = it->second;
      return true;
    }
  }
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)TILE_K, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  if (fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  std::lock_guard<std::mutex> lock(mu);
  if (kept.size() >= 8192) kept.clear();
  kept.emplace(key, *map);
  return true;
}

template <int NTOK, bool SILU>
int launch_cfg(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, cudaStream_t stream) {
  constexpr int STAGES = stages_for<NTOK>();
  const size_t smem = 1024 + (size_t)STAGES * kblocks_for<NTOK>() * (TILE_N * TILE_K * 2 + NTOK * TILE_K * 2) +
                      (2 * STAGES + 1) * 8 + 16;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_wstream_kernel<NTOK, SILU>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return YALIS_ERR_LAUNCH;
    configured = true;
  }
  const int tile_rows = p.silu_inter ? TILE_N / 2 : TILE_N;
  const int rows = p.silu_inter ? p.silu_inter : p.N;
  dim3 grid((rows + tile_rows - 1) / tile_rows, p.splits);
  return yalis_launch(gemm_wstream_kernel<NTOK, SILU>, grid, dim3(kThreads), smem, stream, mw, mx, p);
}

template <int NTOK>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, cudaStream_t stream) {
  return p.silu_inter ? launch_cfg<NTOK, true>(mw, mx, p, stream) : launch_cfg<NTOK, false>(mw, mx, p, stream);
}

}  // namespace

// How many K splits the launcher would use for this shape (so callers can size `out`).
// Chosen so that the grid fills the GPU without a mostly empty last wave: grids of up to two
// blocks per SM run as one wave; every split costs a little (a partial output to write and add).
YALIS_API int yalis_gemm_wstream_splits(int N, int K) {
  const int tiles = (N + TILE_N - 1) / TILE_N;
  const int kt = (K + TILE_K - 1) / TILE_K;
  int best = 1;
  double best_cost = 1e30;
  const int sms = yalis_sm_count();
  for (int s = 1; s <= 16; ++s) {
    if (s > 1 && kt / s < 8) break;
    const int blocks = tiles * s;
    double cost;
    if (blocks <= 2 * sms) {
      // A grid keeps HBM busy from about one and a half blocks per SM on (a block alone on an SM has only its own
      // five tiles in flight); measured on the decode shapes of Llama-3-8B, where 7 / 5 / 7 splits for the down, QKV
      // and attention-output products beat 5 / 3 / 5 by 2 % of a step.
      const int full = sms + sms / 2;
      cost = blocks >= full ? 1.0 : (double)full / blocks;
    } else {
      const int waves = (blocks + 2 * sms - 1) / (2 * sms);
      cost = (double)waves * 2 * sms / blocks;
    }
    cost += 0.02 * s;
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}

// out = x[M, K] . w[N, K]^T, bfloat16 operands.  splits must be yalis_gemm_wstream_splits(N, K) or 1;
// with splits > 1, out is float32 [splits, M, N] (ldo = N).  error: device int32 raised on a timed-out wait.
namespace {
int gemm_wstream_impl(const void* x, long long ldx, const void* w, long long ldw, void* out, int out_dtype, long long ldo,
                      int M, int N, int K, int splits, int silu_inter, int32_t* error, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return YALIS_OK;
  if (M > 256 || K <= 0 || splits < 1) return YALIS_ERR_SHAPE;
  if ((K % 8) || (ldx % 8) || (ldw % 8)) return YALIS_ERR_ALIGN;          // TMA: 16-byte strides
  if (((uintptr_t)x | (uintptr_t)w) & 15) return YALIS_ERR_ALIGN;
  if (out_dtype != YALIS_F32 && out_dtype != YALIS_BF16) return YALIS_ERR_DTYPE;
  if (splits > 1 && out_dtype != YALIS_F32) return YALIS_ERR_DTYPE;
  const int ntok = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  CUtensorMap mw, mx;
  if (!make_map(&mw, w, N, K, ldw, silu_inter ? TILE_N / 2 : TILE_N) || !make_map(&mx, x, M, K, ldx, ntok))
    return YALIS_ERR_LAUNCH;
  GemmParams p;
  p.out = out; p.out_dtype = out_dtype; p.ldo = ldo; p.M = M; p.N = N; p.K = K; p.splits = splits;
  const int step_k = (ntok <= 16 ? 2 : 1) * TILE_K;            // kblocks_for<ntok>() columns per stage step
  const int kt = (K + step_k - 1) / step_k;
  p.kt_per_split = (kt + splits - 1) / splits;
  p.silu_inter = silu_inter;
  p.error = error;
  switch (ntok) {
    case 16: return launch<16>(mw, mx, p, stream);
    case 32: return launch<32>(mw, mx, p, stream);
    case 64: return launch<64>(mw, mx, p, stream);
    case 128: return launch<128>(mw, mx, p, stream);
    default: return launch<256>(mw, mx, p, stream);
  }
}
}  // namespace

YALIS_API int yalis_gemm_wstream(const void* x, long long ldx, const void* w, long long ldw, void* out, int out_dtype,
                                 long long ldo, int M, int N, int K, int splits, int32_t* error,
                                 cudaStream_t stream) {
  return gemm_wstream_impl(x, ldx, w, ldw, out, out_dtype, ldo, M, N, K, splits, 0, error, stream);
}

// The gated activation fused into the product: w is [2 * inter, K] with the gate rows first and the up rows
// after them; out[m, i] = silu(x . gate_i) * (x . up_i), bfloat16 [M, inter] with row stride ldo.  Both products
// are rounded to bfloat16 before the activation, so the result has the bits of yalis_gemm_wstream followed by
// yalis_silu_mul.  The K range is never split.
YALIS_API int yalis_gemm_wstream_silu(const void* x, long long ldx, const void* w, long long ldw, void* out,
                                      long long ldo, int M, int inter, int K, int32_t* error, cudaStream_t stream) {
  if (inter <= 0) return YALIS_ERR_SHAPE;
  return gemm_wstream_impl(x, ldx, w, ldw, out, YALIS_BF16, ldo, M, 2 * inter, K, 1, inter, error, stream);
}
