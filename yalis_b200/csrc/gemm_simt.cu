// y = x W^T on the CUDA cores: the matrix product of the float32 path.
//
// x [M, K] and W [N, K] are both K-contiguous (a Linear layer's weight as it
// is stored).  Products and sums are float32 FMAs; there is no tensor-core
// instruction and no reduced-precision mode anywhere in this file, so with
// float32 operands the result is a true 32-bit product.  Each output element
// is accumulated over k = 0..K-1 in ascending order by one thread, so it does
// not depend on M, N or the tile a row falls into: a token's result is the
// same bits whatever batch it is computed in.
//
// Operand and output types are independent (float or bfloat16), which lets the
// same kernel serve as the twin of the tensor-core kernels in tests.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16;
constexpr int TM = 4, TN = 4;  // per-thread tile; 16 x 16 threads

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_tn_simt_kernel(const TA* __restrict__ A, long long lda, const TW* __restrict__ W, long long ldw,
                    TO* __restrict__ O, long long ldo, int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  const int lr = tid >> 2;        // 0..63: row of the tile this thread loads
  const int lk = (tid & 3) * 4;   // 0,4,8,12: first k of its four elements
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + lk + u;
      const int am = m0 + lr, wn = n0 + lr;
      As[lk + u][lr] = (am < M && k < K) ? to_f32<TA>(A[(size_t)am * lda + k]) : 0.f;
      Ws[lk + u][lr] = (wn < N && k < K) ? to_f32<TW>(W[(size_t)wn * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) O[(size_t)m * ldo + n] = from_f32<TO>(acc[i][j]);
    }
  }
}

template <typename TA, typename TW, typename TO>
int launch(const void* A, long long lda, const void* W, long long ldw, void* O, long long ldo, int M, int N, int K,
           cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return YALIS_ERR_SHAPE;
  return yalis_launch(gemm_tn_simt_kernel<TA, TW, TO>, grid, dim3(256), 0, stream, (const TA*)A, lda, (const TW*)W, ldw,
                      (TO*)O, ldo, M, N, K);
}

}  // namespace

// O[M, N] = A[M, K] . W[N, K]^T with float32 accumulation.
YALIS_API int yalis_gemm_tn_simt(const void* A, int a_dtype, long long lda, const void* W, int w_dtype, long long ldw,
                                 void* O, int o_dtype, long long ldo, int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return YALIS_OK;
  if (K <= 0) return YALIS_ERR_SHAPE;
  using bf16 = __nv_bfloat16;
  const int code = a_dtype * 4 + w_dtype * 2 + o_dtype;
  switch (code) {
    case 0: return launch<float, float, float>(A, lda, W, ldw, O, ldo, M, N, K, stream);
    case 1: return launch<float, float, bf16>(A, lda, W, ldw, O, ldo, M, N, K, stream);
    case 2: return launch<float, bf16, float>(A, lda, W, ldw, O, ldo, M, N, K, stream);
    case 3: return launch<float, bf16, bf16>(A, lda, W, ldw, O, ldo, M, N, K, stream);
    case 4: return launch<bf16, float, float>(A, lda, W, ldw, O, ldo, M, N, K, stream);
    case 5: return launch<bf16, float, bf16>(A, lda, W, ldw, O, ldo, M, N, K, stream);
    case 6: return launch<bf16, bf16, float>(A, lda, W, ldw, O, ldo, M, N, K, stream);
    case 7: return launch<bf16, bf16, bf16>(A, lda, W, ldw, O, ldo, M, N, K, stream);
    default: return YALIS_ERR_DTYPE;
  }
}
