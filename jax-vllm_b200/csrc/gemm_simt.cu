// C[M, N] = A[M, K] * W[N, K]^T on CUDA cores, accumulating in 32-bit with FFMA: the
// matrix product of the 32-bit path (no reduced-precision tensor mode), also used where
// a result must leave in 32-bit (logits) from 16-bit operands.  Every output element is
// the sum over k in ascending order whatever M and N are, so a row's result does not
// depend on which other rows are in the batch.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) gemm_tn_simt_kernel(const TA* __restrict__ A, int lda,
                                                           const TW* __restrict__ W, int ldw,
                                                           TC* __restrict__ C, int ldc, int M, int N,
                                                           int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256;
      const int row = idx >> 4, kk = idx & 15;
      const int k = k0 + kk;
      float a = 0.f, w = 0.f;
      if (k < K) {
        if (m0 + row < M) a = to_f32(A[(size_t)(m0 + row) * lda + k]);
        if (n0 + row < N) w = to_f32(W[(size_t)(n0 + row) * ldw + k]);
      }
      As[kk][row] = a;
      Ws[kk][row] = w;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * ldc + n] = from_f32<TC>(acc[i][j]);
    }
  }
}
}  // namespace

// A: [M, K] rows of lda elements; W: [N, K] rows of ldw elements; C: [M, N] rows of ldc.
JV_EXPORT int jv_gemm_tn_simt(const void* A, int a_dtype, int lda, const void* W, int w_dtype, int ldw,
                              void* C, int c_dtype, int ldc, int M, int N, int K,
                              cudaStream_t stream) {
  if (M == 0 || N == 0) return JV_OK;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return JV_ERR_UNSUPPORTED;
  JV_DISPATCH_DTYPE(a_dtype, TA, JV_DISPATCH_DTYPE(w_dtype, TW, JV_DISPATCH_DTYPE(c_dtype, TC,
      (gemm_tn_simt_kernel<TA, TW, TC><<<grid, 256, 0, stream>>>(
          (const TA*)A, lda, (const TW*)W, ldw, (TC*)C, ldc, M, N, K)))));
  return jv_check_launch();
}
