// y[M, N] = x[M, K] * W[N, K]^T for a few rows of x (decoded tokens): bfloat16 operands,
// 32-bit accumulation, bound by reading W once from HBM.
//
// The weight is the 16-row operand of mma.sync m16n8k16 and the batch is its 8-column operand
// (y^T = W x^T), so no tensor-core rows are wasted on padding the batch.  Operand fragments come
// straight from global memory with 16-byte loads, without shared memory: a sum over k does not
// care about the order of k, so within a 64-wide chunk of k thread c of a row takes elements
// [8c, 8c+8) and [32+8c, 32+8c+8) and uses pair j of each as the two k-halves of step j, for W and
// for x alike.  Every load instruction of a warp then covers 8 rows x 64 contiguous bytes.
//
// A block owns 16 rows of W (16 columns of y); its 8 warps split k into 8 contiguous slices and
// are summed in shared memory in warp order.  The slicing depends on K only, so a row of y is
// the same whatever other rows are in the batch.
#include "common.cuh"

namespace {
constexpr int WARPS = 8;
constexpr int KC = 64;   // k elements per chunk

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_w(const __nv_bfloat16* p, bool ok) {
  return ok ? __ldcs(reinterpret_cast<const uint4*>(p)) : make_uint4(0, 0, 0, 0);   // streamed: read once
}
__device__ __forceinline__ uint4 load_x(const __nv_bfloat16* p, bool ok) {
  return ok ? __ldg(reinterpret_cast<const uint4*>(p)) : make_uint4(0, 0, 0, 0);    // reused by every block
}
__device__ __forceinline__ uint32_t pick(const uint4& v, int j) {
  return j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w));
}

template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <int NB, typename TOut>
__global__ void __launch_bounds__(WARPS * 32) skinny_kernel(const __nv_bfloat16* __restrict__ X, int ldx,
                                                            const __nv_bfloat16* __restrict__ W, int ldw,
                                                            TOut* __restrict__ Y, int ldy, int M, int N, int K) {
  __shared__ float red[WARPS][16][NB * 8 + 1];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int chunks = (K + KC - 1) / KC;
  const int per_warp = (chunks + WARPS - 1) / WARPS;
  const int k_begin = warp * per_warp * KC;
  const int k_end = min(K, k_begin + per_warp * KC);

  // rows of W this thread reads (clamped: rows beyond N are read from the last row and dropped later)
  const __nv_bfloat16* w0 = W + (size_t)min(n0 + r, N - 1) * ldw;
  const __nv_bfloat16* w1 = W + (size_t)min(n0 + r + 8, N - 1) * ldw;
  const __nv_bfloat16* xr[NB];
  bool xok[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    const int m = nb * 8 + r;
    xok[nb] = m < M;
    xr[nb] = X + (size_t)(xok[nb] ? m : 0) * ldx;
  }
  float acc[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nb][i] = 0.f;

#pragma unroll 4
  for (int k0 = k_begin; k0 < k_end; k0 += KC) {
    const int ka = k0 + c * 8, kb = k0 + 32 + c * 8;
    const bool oka = ka + 8 <= K, okb = kb + 8 <= K;
    const uint4 a_lo0 = load_w(w0 + ka, oka), a_hi0 = load_w(w0 + kb, okb);
    const uint4 a_lo1 = load_w(w1 + ka, oka), a_hi1 = load_w(w1 + kb, okb);
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const uint4 x_lo = load_x(xr[nb] + ka, oka && xok[nb]), x_hi = load_x(xr[nb] + kb, okb && xok[nb]);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        mma_bf16(acc[nb], pick(a_lo0, j), pick(a_lo1, j), pick(a_hi0, j), pick(a_hi1, j), pick(x_lo, j), pick(x_hi, j));
    }
  }

  // ---- sum the k slices in warp order
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    red[warp][r][nb * 8 + c * 2] = acc[nb][0];
    red[warp][r][nb * 8 + c * 2 + 1] = acc[nb][1];
    red[warp][r + 8][nb * 8 + c * 2] = acc[nb][2];
    red[warp][r + 8][nb * 8 + c * 2 + 1] = acc[nb][3];
  }
  __syncthreads();
  for (int idx = tid; idx < 16 * NB * 8; idx += WARPS * 32) {
    const int row = idx & 15, m = idx >> 4;
    if (m >= M || n0 + row >= N) continue;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) s += red[w][row][m];
    store_out<TOut>(Y + (size_t)m * ldy + n0 + row, s);
  }
}

template <typename TOut>
int launch(const void* X, int ldx, const void* W, int ldw, void* Y, int ldy, int M, int N, int K, cudaStream_t stream) {
  const int blocks = (N + 15) / 16;
  const __nv_bfloat16* x = (const __nv_bfloat16*)X;
  const __nv_bfloat16* w = (const __nv_bfloat16*)W;
  TOut* y = (TOut*)Y;
  if (M <= 8) skinny_kernel<1, TOut><<<blocks, WARPS * 32, 0, stream>>>(x, ldx, w, ldw, y, ldy, M, N, K);
  else if (M <= 16) skinny_kernel<2, TOut><<<blocks, WARPS * 32, 0, stream>>>(x, ldx, w, ldw, y, ldy, M, N, K);
  else if (M <= 32) skinny_kernel<4, TOut><<<blocks, WARPS * 32, 0, stream>>>(x, ldx, w, ldw, y, ldy, M, N, K);
  else if (M <= 64) skinny_kernel<8, TOut><<<blocks, WARPS * 32, 0, stream>>>(x, ldx, w, ldw, y, ldy, M, N, K);
  else return JV_ERR_UNSUPPORTED;
  return jv_check_launch();
}
}  // namespace

// Largest number of rows of x the kernel takes.
JV_EXPORT int jv_linear_skinny_max_rows() { return 64; }

// X: [M, K] bfloat16 rows of ldx elements; W: [N, K] bfloat16 rows of ldw; Y: [M, N] rows of ldy, bfloat16
// (out_dtype 1) or float (0).  K, ldx and ldw must be multiples of 8 and X, W 16-byte aligned.
JV_EXPORT int jv_linear_skinny(const void* X, int ldx, const void* W, int ldw, void* Y, int out_dtype, int ldy, int M,
                               int N, int K, cudaStream_t stream) {
  if (M == 0 || N == 0) return JV_OK;
  if (M > 64 || K < 8 || (K % 8) || (ldx % 8) || (ldw % 8) || ((uintptr_t)X % 16) || ((uintptr_t)W % 16))
    return JV_ERR_UNSUPPORTED;
  if (out_dtype == 0) return launch<float>(X, ldx, W, ldw, Y, ldy, M, N, K, stream);
  if (out_dtype == 1) return launch<__nv_bfloat16>(X, ldx, W, ldw, Y, ldy, M, N, K, stream);
  return JV_ERR_UNSUPPORTED;
}
