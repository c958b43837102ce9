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
// A strip is 16 rows of W (16 columns of y); the 8 warps of a block split k into 8 contiguous slices
// and are summed in shared memory in warp order.  The slicing depends on K only, so a row of y is
// the same whatever other rows are in the batch.  Up to 16 rows of x; larger batches go to the
// library product, which is faster there.
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

__device__ __forceinline__ uint4 load_x(const __nv_bfloat16* p, bool ok) {
  return ok ? __ldg(reinterpret_cast<const uint4*>(p)) : make_uint4(0, 0, 0, 0);    // reused by every block
}
__device__ __forceinline__ uint32_t pick(const uint4& v, int j) {
  return j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w));
}

template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int STAGES = 4;          // 64-wide chunks of k in flight per warp
constexpr int CTAS_PER_SM = 3;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;   // 0 bytes read: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src), "r"(n));
}

// Persistent blocks: block b takes the 16-row strips b, b + gridDim.x, ...; warp w takes the w-th
// slice of k of every strip.  A warp's stream of chunks (over all its strips) runs through a ring of
// STAGES chunk buffers in shared memory filled by cp.async, each lane owning the 4 x 16 bytes it will
// consume itself, so a chunk needs no synchronisation between threads and the next strip's first
// chunks are already under way while this strip is summed up.
template <int NB, typename TOut>
__global__ void __launch_bounds__(WARPS * 32, CTAS_PER_SM) skinny_kernel(const __nv_bfloat16* __restrict__ X, int ldx,
                                                                         const __nv_bfloat16* __restrict__ W, int ldw,
                                                                         TOut* __restrict__ Y, int ldy, int M, int N,
                                                                         int K, int n_strips) {
  extern __shared__ uint4 dyn_smem[];
  uint4 (*ring)[STAGES][4][32] = reinterpret_cast<uint4 (*)[STAGES][4][32]>(dyn_smem);                 // [WARPS]
  float (*red)[16][NB * 8 + 1] = reinterpret_cast<float (*)[16][NB * 8 + 1]>(dyn_smem + WARPS * STAGES * 4 * 32);  // [WARPS]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int chunks = (K + KC - 1) / KC;
  const int per_warp = (chunks + WARPS - 1) / WARPS;      // chunks of one strip that this warp takes
  const int k_begin = warp * per_warp * KC;
  const int n_my = ((int)blockIdx.x < n_strips) ? (n_strips - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const int total = n_my * per_warp;

  const __nv_bfloat16* xr[NB];
  bool xok[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    const int m = nb * 8 + r;
    xok[nb] = m < M;
    xr[nb] = X + (size_t)(xok[nb] ? m : 0) * ldx;
  }

  // producer state: the next chunk to request
  int p_strip = blockIdx.x, p_chunk = 0, p_count = 0;
  auto issue = [&]() {
    if (p_count < total) {
      const int n0 = p_strip * 16;
      const int k0 = k_begin + p_chunk * KC;
      const int ka = k0 + c * 8, kb = k0 + 32 + c * 8;
      const bool oka = ka + 8 <= K, okb = kb + 8 <= K;
      const int r0 = n0 + r, r1 = n0 + r + 8;
      const bool ok0 = r0 < N, ok1 = r1 < N;
      const __nv_bfloat16* w0 = W + (size_t)(ok0 ? r0 : 0) * ldw;
      const __nv_bfloat16* w1 = W + (size_t)(ok1 ? r1 : 0) * ldw;
      uint4* slot = &ring[warp][p_count % STAGES][0][lane];
      cp_async16(slot, w0 + (oka ? ka : 0), ok0 && oka);
      cp_async16(slot + 32, w0 + (okb ? kb : 0), ok0 && okb);
      cp_async16(slot + 64, w1 + (oka ? ka : 0), ok1 && oka);
      cp_async16(slot + 96, w1 + (okb ? kb : 0), ok1 && okb);
      ++p_count;
      if (++p_chunk == per_warp) { p_chunk = 0; p_strip += gridDim.x; }
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  pdl_trigger();
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) issue();   // weights: nobody writes them, so they are requested
  pdl_wait();                                     // before the kernels that produce x have finished

  float acc[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nb][i] = 0.f;

  int strip = blockIdx.x, chunk = 0;
  for (int i = 0; i < total; ++i) {
    issue();
    asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 1));
    const uint4* slot = &ring[warp][i % STAGES][0][lane];
    const uint4 a_lo0 = slot[0], a_hi0 = slot[32], a_lo1 = slot[64], a_hi1 = slot[96];
    const int k0 = k_begin + chunk * KC;
    const int ka = k0 + c * 8, kb = k0 + 32 + c * 8;
    const bool oka = ka + 8 <= K, okb = kb + 8 <= K;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const uint4 x_lo = load_x(xr[nb] + ka, oka && xok[nb]), x_hi = load_x(xr[nb] + kb, okb && xok[nb]);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        mma_bf16(acc[nb], pick(a_lo0, j), pick(a_lo1, j), pick(a_hi0, j), pick(a_hi1, j), pick(x_lo, j), pick(x_hi, j));
    }
    if (++chunk == per_warp) {
      // ---- the strip is complete in this warp: sum the k slices in warp order
      chunk = 0;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        red[warp][r][nb * 8 + c * 2] = acc[nb][0];
        red[warp][r][nb * 8 + c * 2 + 1] = acc[nb][1];
        red[warp][r + 8][nb * 8 + c * 2] = acc[nb][2];
        red[warp][r + 8][nb * 8 + c * 2 + 1] = acc[nb][3];
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[nb][q] = 0.f;
      }
      __syncthreads();
      const int n0 = strip * 16;
      for (int idx = tid; idx < 16 * NB * 8; idx += WARPS * 32) {
        const int row = idx & 15, m = idx >> 4;
        if (m >= M || n0 + row >= N) continue;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) s += red[w][row][m];
        store_out<TOut>(Y + (size_t)m * ldy + n0 + row, s);
      }
      __syncthreads();
      strip += gridDim.x;
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
}

template <int NB> constexpr size_t smem_bytes() {
  return sizeof(uint4) * WARPS * STAGES * 4 * 32 + sizeof(float) * WARPS * 16 * (NB * 8 + 1);
}

template <typename TOut>
int launch(const void* X, int ldx, const void* W, int ldw, void* Y, int ldy, int M, int N, int K, cudaStream_t stream) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  const int n_strips = (N + 15) / 16;
  const int blocks = n_strips < sms * CTAS_PER_SM ? n_strips : sms * CTAS_PER_SM;
  const __nv_bfloat16* x = (const __nv_bfloat16*)X;
  const __nv_bfloat16* w = (const __nv_bfloat16*)W;
  TOut* y = (TOut*)Y;
  static bool ready = false;   // set once: the attribute calls are kept out of stream captures
  if (!ready) {
    if (cudaFuncSetAttribute(skinny_kernel<1, TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<1>()) != cudaSuccess ||
        cudaFuncSetAttribute(skinny_kernel<2, TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<2>()) != cudaSuccess)
      return JV_ERR_UNSUPPORTED;
    ready = true;
  }
  if (M <= 8)
    return jv_launch(skinny_kernel<1, TOut>, dim3(blocks), dim3(WARPS * 32), smem_bytes<1>(), stream, x, ldx, w, ldw, y,
                     ldy, M, N, K, n_strips);
  if (M <= 16)
    return jv_launch(skinny_kernel<2, TOut>, dim3(blocks), dim3(WARPS * 32), smem_bytes<2>(), stream, x, ldx, w, ldw, y,
                     ldy, M, N, K, n_strips);
  return JV_ERR_UNSUPPORTED;
}
}  // namespace

// Largest number of rows of x the kernel takes.
JV_EXPORT int jv_linear_skinny_max_rows() { return 16; }

// X: [M, K] bfloat16 rows of ldx elements; W: [N, K] bfloat16 rows of ldw; Y: [M, N] rows of ldy, bfloat16
// (out_dtype 1) or float (0).  K, ldx and ldw must be multiples of 8 and X, W 16-byte aligned.
JV_EXPORT int jv_linear_skinny(const void* X, int ldx, const void* W, int ldw, void* Y, int out_dtype, int ldy, int M,
                               int N, int K, cudaStream_t stream) {
  if (M == 0 || N == 0) return JV_OK;
  if (M > 16 || K < 8 || (K % 8) || (ldx % 8) || (ldw % 8) || ((uintptr_t)X % 16) || ((uintptr_t)W % 16))
    return JV_ERR_UNSUPPORTED;
  if (out_dtype == 0) return launch<float>(X, ldx, W, ldw, Y, ldy, M, N, K, stream);
  if (out_dtype == 1) return launch<__nv_bfloat16>(X, ldx, W, ldw, Y, ldy, M, N, K, stream);
  return JV_ERR_UNSUPPORTED;
}
