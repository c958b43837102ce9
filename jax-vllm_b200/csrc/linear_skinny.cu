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
// the same whatever other rows are in the batch.  Up to 16 rows of x (the second 8 cost a fifth of the
// speed: from 9 rows on the caller prefers the tcgen05 kernel of linear_stream.cu).
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

// Persistent blocks.  A unit of work is a 16-row strip of W, or one of `splits` equal parts of its k when
// strips alone would leave multiprocessors idle (few strips) or unevenly loaded; block b takes the units
// b, b + gridDim.x, ... and warp w the w-th eighth of every unit's k.  A warp's stream of chunks (over all its
// units) runs through a ring of STAGES chunk buffers in shared memory filled by cp.async, each lane owning the
// 4 x 16 bytes it will consume itself, so a chunk needs no synchronisation between threads and the next
// unit's first chunks are already under way while this unit is summed up.  With splits, part s of every
// strip goes to parts[s] ([splits, M, N], 32-bit) and the kernel that reads the result adds the parts in the
// order of s as it loads them: nobody waits and no block sums up after another.  The partition depends on
// N, K and the number of multiprocessors only, never on the batch.
template <int NB, typename TOut>
__global__ void __launch_bounds__(WARPS * 32, CTAS_PER_SM) skinny_kernel(const __nv_bfloat16* __restrict__ X, int ldx,
                                                                         const __nv_bfloat16* __restrict__ W, int ldw,
                                                                         TOut* __restrict__ Y, int ldy, int M, int N,
                                                                         int K, int n_strips, int splits, int per_warp,
                                                                         float* __restrict__ parts) {
  // all shared memory is dynamic and begins on a 128-byte line: a warp's 512 bytes of a ring slot then lie in
  // four lines (a static variable before it once shifted the ring by 16 bytes, which cost a fifth of the speed)
  extern __shared__ __align__(128) uint4 dyn_smem[];
  uint4 (*ring)[STAGES][4][32] = reinterpret_cast<uint4 (*)[STAGES][4][32]>(dyn_smem);                 // [WARPS]
  float (*red)[16][NB * 8 + 1] = reinterpret_cast<float (*)[16][NB * 8 + 1]>(dyn_smem + WARPS * STAGES * 4 * 32);  // [WARPS]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int n_units = n_strips * splits;
  const int n_my = ((int)blockIdx.x < n_units) ? (n_units - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const int total = n_my * per_warp;
  // unit u is part u % splits of strip u / splits; this warp's chunks of it begin at k_of(u)
  auto k_of = [&](int unit) { return ((unit % splits) * WARPS + warp) * per_warp * KC; };

  const __nv_bfloat16* xr[NB];
  bool xok[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    const int m = nb * 8 + r;
    xok[nb] = m < M;
    xr[nb] = X + (size_t)(xok[nb] ? m : 0) * ldx;
  }

  // producer state: the next chunk to request
  int p_unit = blockIdx.x, p_chunk = 0, p_count = 0;
  int p_n0 = (p_unit / splits) * 16, p_k = k_of(p_unit);          // kept up to date at unit ends: no division per chunk
  auto issue = [&]() {
    if (p_count < total) {
      const int n0 = p_n0;
      const int k0 = p_k;
      uint4* slot = &ring[warp][p_count % STAGES][0][lane];
      const int ka = k0 + c * 8, kb = k0 + 32 + c * 8;
      const bool oka = ka + 8 <= K, okb = kb + 8 <= K;
      const int r0 = n0 + r, r1 = n0 + r + 8;
      const bool ok0 = r0 < N, ok1 = r1 < N;
      const __nv_bfloat16* w0 = W + (size_t)(ok0 ? r0 : 0) * ldw;
      const __nv_bfloat16* w1 = W + (size_t)(ok1 ? r1 : 0) * ldw;
      cp_async16(slot, w0 + (oka ? ka : 0), ok0 && oka);
      cp_async16(slot + 32, w0 + (okb ? kb : 0), ok0 && okb);
      cp_async16(slot + 64, w1 + (oka ? ka : 0), ok1 && oka);
      cp_async16(slot + 96, w1 + (okb ? kb : 0), ok1 && okb);
      ++p_count;
      p_k += KC;
      if (++p_chunk == per_warp) { p_chunk = 0; p_unit += gridDim.x; p_n0 = (p_unit / splits) * 16; p_k = k_of(p_unit); }
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

  // x of the chunk after this one is asked for before this chunk's products, so its way from the L2 is hidden
  auto fetch_x = [&](int k0, uint4 (&lo)[NB], uint4 (&hi)[NB]) {
    const int ka = k0 + c * 8, kb = k0 + 32 + c * 8;
    const bool oka = ka + 8 <= K, okb = kb + 8 <= K;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      lo[nb] = load_x(xr[nb] + ka, oka && xok[nb]);
      hi[nb] = load_x(xr[nb] + kb, okb && xok[nb]);
    }
  };
  uint4 x_lo[NB], x_hi[NB];
  int unit = blockIdx.x, chunk = 0;
  int k_now = k_of(unit), k_next_unit = k_of(unit + gridDim.x);
  if (total > 0) fetch_x(k_now, x_lo, x_hi);
  for (int i = 0; i < total; ++i) {
    issue();
    uint4 nx_lo[NB], nx_hi[NB];
    k_now = (chunk + 1 == per_warp) ? k_next_unit : k_now + KC;
    fetch_x(k_now, nx_lo, nx_hi);
    asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 1));
    const uint4* slot = &ring[warp][i % STAGES][0][lane];
    const uint4 a_lo0 = slot[0], a_hi0 = slot[32], a_lo1 = slot[64], a_hi1 = slot[96];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        mma_bf16(acc[nb], pick(a_lo0, j), pick(a_lo1, j), pick(a_hi0, j), pick(a_hi1, j), pick(x_lo[nb], j), pick(x_hi[nb], j));
      x_lo[nb] = nx_lo[nb]; x_hi[nb] = nx_hi[nb];
    }
    if (++chunk == per_warp) {
      // ---- the unit is complete in this warp: sum the k slices in warp order
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
      const int strip = unit / splits;
      const int n0 = strip * 16;
      constexpr int CELLS = 16 * NB * 8;             // (row of the strip, row of x) pairs, at most one per thread
      static_assert(CELLS <= WARPS * 32, "one cell per thread");
      const int row = tid & 15, m = tid >> 4;
      const bool mine = tid < CELLS && m < M && n0 + row < N;
      float sum = 0.f;
      if (mine) {
#pragma unroll
        for (int w = 0; w < WARPS; ++w) sum += red[w][row][m];
      }
      if (splits == 1) {
        if (mine) store_out<TOut>(Y + (size_t)m * ldy + n0 + row, sum);
      } else if (mine) {
        parts[((size_t)(unit - strip * splits) * M + m) * N + n0 + row] = sum;
      }
      __syncthreads();
      unit += gridDim.x;
      k_next_unit = k_of(unit + gridDim.x);
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
}

template <int NB> constexpr size_t smem_bytes() {
  return sizeof(uint4) * WARPS * STAGES * 4 * 32 + sizeof(float) * WARPS * 16 * (NB * 8 + 1);
}

int multiprocessors() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  return sms;
}

// How evenly `n_strips` strips cut into `s` parts of k load the device, between 0 and 1: the useful share of the
// busiest multiprocessor's time (blocks go to multiprocessors in turn; a multiprocessor's load is the units of its
// blocks).
double load_evenness(int n_strips, int K, int sms, int s) {
  const int chunks = (K + KC - 1) / KC;
  const long long units = (long long)n_strips * s, slots = (long long)sms * CTAS_PER_SM;
  const long long blocks = units < slots ? units : slots;
  long long worst = 0;
  for (int sm = 0; sm < sms && sm < blocks; ++sm) {
    long long load = 0;
    for (long long b = sm; b < blocks; b += sms) load += (units - 1 - b) / blocks + 1;
    if (load > worst) worst = load;
  }
  const int per_warp = (chunks + WARPS * s - 1) / (WARPS * s);
  const double used = (double)chunks / ((double)per_warp * WARPS * s);   // the last part may reach past K
  return used * (double)units / ((double)worst * sms);
}

// The useful share of the busiest block's time when the strips are not cut: 1 while every strip has a block of its
// own; with a few strips more than resident blocks, the blocks that take a second strip run on alone when the
// others are done (448 strips for 444 blocks: 0.50).
double rounds_evenness(int n_strips, int sms) {
  const long long units = n_strips, slots = (long long)sms * CTAS_PER_SM;
  const long long blocks = units < slots ? units : slots;
  return (double)units / ((double)((units + blocks - 1) / blocks) * blocks);
}

// Into how many parts the k of a strip is cut: the smallest number, up to 8, that loads the multiprocessors
// evenly (each unit keeps at least two 64-wide chunks per warp), if that gains a tenth or more over uncut strips.
int choose_splits(int n_strips, int K, int sms) {
  const int chunks = (K + KC - 1) / KC;
  auto efficiency = [&](int s) { return load_evenness(n_strips, K, sms, s); };
  int best = 1;
  double best_eff = efficiency(1);
  const double floor_gain = best_eff * 1.03;
  for (int s = 2; s <= 8; ++s) {
    if (chunks < s * WARPS * 2) break;
    const double e = efficiency(s);
    if (e >= floor_gain && e > best_eff + 0.02) { best = s; best_eff = e; }
  }
  return best;
}

template <typename TOut>
int launch(const void* X, int ldx, const void* W, int ldw, void* Y, int ldy, int M, int N, int K, int splits, float* parts,
           cudaStream_t stream) {
  const int sms = multiprocessors();
  const int n_strips = (N + 15) / 16;
  const int chunks = (K + KC - 1) / KC;
  const int per_warp = (chunks + WARPS * splits - 1) / (WARPS * splits);     // chunks of one unit that a warp takes
  const long long units = (long long)n_strips * splits;
  const int blocks = units < (long long)sms * CTAS_PER_SM ? (int)units : sms * CTAS_PER_SM;
  const __nv_bfloat16* x = (const __nv_bfloat16*)X;
  const __nv_bfloat16* w = (const __nv_bfloat16*)W;
  TOut* y = (TOut*)Y;
  static bool ready[JV_MAX_DEVICES];
  if (!jv_once_per_device(ready, [&] {
        return cudaFuncSetAttribute(skinny_kernel<1, TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<1>()) == cudaSuccess &&
               cudaFuncSetAttribute(skinny_kernel<2, TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes<2>()) == cudaSuccess;
      }))
    return JV_ERR_UNSUPPORTED;
  if (M <= 8)
    return jv_launch(skinny_kernel<1, TOut>, dim3(blocks), dim3(WARPS * 32), smem_bytes<1>(), stream, x, ldx, w, ldw, y,
                     ldy, M, N, K, n_strips, splits, per_warp, parts);
  if (M <= 16)
    return jv_launch(skinny_kernel<2, TOut>, dim3(blocks), dim3(WARPS * 32), smem_bytes<2>(), stream, x, ldx, w, ldw, y,
                     ldy, M, N, K, n_strips, splits, per_warp, parts);
  return JV_ERR_UNSUPPORTED;
}
}  // namespace

// Largest number of rows of x the kernel takes.
JV_EXPORT int jv_linear_skinny_max_rows() { return 16; }

// Into how many parts the kernel would best cut the k of a strip for an [N, K] weight on this device (1: not at all).
JV_EXPORT int jv_linear_skinny_plan(int N, int K) { return choose_splits((N + 15) / 16, K, multiprocessors()); }

// How evenly the uncut strips of a weight of N rows fill the rounds of this device's resident blocks, in thousandths
// (see `rounds_evenness`): what a caller that wants one tensor gets.
JV_EXPORT int jv_linear_skinny_fill(int N) { return (int)(1000.0 * rounds_evenness((N + 15) / 16, multiprocessors())); }

// X: [M, K] bfloat16 rows of ldx elements; W: [N, K] bfloat16 rows of ldw.  splits == 1: Y [M, N] rows of ldy,
// bfloat16 (out_dtype 1) or float (0).  splits > 1 (at most 8, each part at least 8 chunks of 64): Y is not
// written; parts [splits, M, N] float gets the sums over the parts of k, to be added by the reader.
// K, ldx and ldw must be multiples of 8 and X, W 16-byte aligned.
JV_EXPORT int jv_linear_skinny(const void* X, int ldx, const void* W, int ldw, void* Y, int out_dtype, int ldy, int M,
                               int N, int K, float* parts, int splits, cudaStream_t stream) {
  if (M == 0 || N == 0) return JV_OK;
  if (M > 16 || K < 8 || (K % 8) || (ldx % 8) || (ldw % 8) || ((uintptr_t)X % 16) || ((uintptr_t)W % 16))
    return JV_ERR_UNSUPPORTED;
  if (splits < 1 || splits > 8 || (splits > 1 && (parts == nullptr || (K + KC - 1) / KC < splits * WARPS)))
    return JV_ERR_UNSUPPORTED;
  if (out_dtype == 0) return launch<float>(X, ldx, W, ldw, Y, ldy, M, N, K, splits, parts, stream);
  if (out_dtype == 1) return launch<__nv_bfloat16>(X, ldx, W, ldw, Y, ldy, M, N, K, splits, parts, stream);
  return JV_ERR_UNSUPPORTED;
}
