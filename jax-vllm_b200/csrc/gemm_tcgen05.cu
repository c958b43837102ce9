// C[M, N] = A[M, K] * B[N, K]^T for bfloat16 on the 5th-generation tensor cores: tcgen05.mma with
// the accumulator in tensor memory (TMEM), operands brought into shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle), a persistent block per SM.
//
// Roles in a block of 6 warps:
//   warp 0, one thread   producer: waits for a free stage, announces the bytes of an A tile (128 x 64) and a
//                        B tile (256 x 64) on the stage's mbarrier and issues the two TMA loads;
//   warp 1, one thread   issues four tcgen05.mma (128 x 256 x 16 each) per stage into one of two TMEM
//                        accumulators (2 x 256 columns of 32-bit), frees the stage with tcgen05.commit, and
//                        hands the finished accumulator to the epilogue with another commit;
//   warp 1               allocates and frees the 512 TMEM columns;
//   warps 2..5           epilogue: each reads its 32 TMEM lanes (= rows of the tile) with tcgen05.ld, 32
//                        columns at a time, and writes C; meanwhile the other accumulator is being filled.
// Epilogues: bfloat16, float, and the gated activation silu(g) * u where the 256 columns of a tile are
// 128 gate columns followed by the 128 up columns of the same indices (the weight rows are stored so).
// Rows and columns beyond M, N, K are zero-filled by TMA on the way in and skipped on the way out.
// Every wait on an mbarrier is bounded by a clock deadline; a wait that runs out sets a bit in the
// status word and the block goes to its tear-down (TMEM is freed) instead of spinning.
#include "common.cuh"
#include "mbarrier.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

namespace {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 512;
constexpr int THREADS = 192;

enum : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_SWIGLU = 2 };


__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
               ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile in the 128-byte-swizzle layout that TMA writes: rows of
// 128 bytes, groups of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1, swizzle mode 2.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);          // start address
  d |= (uint64_t)1 << 16;                           // leading byte offset (not used with this swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;                 // stride byte offset
  d |= (uint64_t)1 << 46;                           // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                           // 128-byte swizzle
  return d;
}
// Instruction descriptor: bfloat16 x bfloat16 -> float, both operands K-major, M = 128, N = 256.
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(IDESC), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

struct Shared {
  uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
  uint64_t drain;                 // used only after a wait ran out (see the tear-down)
  uint32_t tmem_base;
  int failed;
  int armed[STAGES];              // parity of the phase that the producer armed last on full[s]; -1: never
};

template <int EPI>
__global__ void __launch_bounds__(THREADS, 1) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap a_map,
                                                                  const __grid_constant__ CUtensorMap b_map, void* C,
                                                                  int ldc, int M, int N, int K, int* status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  Shared* sh = reinterpret_cast<Shared*>(tiles + STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int n_tiles = tiles_m * tiles_n;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&sh->full[s], 1); mbar_init(&sh->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&sh->acc_full[a], 1); mbar_init(&sh->acc_empty[a], 128); }
    mbar_init(&sh->drain, 1);
    sh->failed = 0;
    for (int s = 0; s < STAGES; ++s) sh->armed[s] = -1;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {   // TMEM: all 512 columns (one block per SM)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh->tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = sh->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int s = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&sh->empty[s], phase ^ 1)) { ok = false; break; }
          sh->armed[s] = phase;
          mbar_expect_tx(&sh->full[s], STAGE_BYTES);
          tma_load_2d(tiles + s * STAGE_BYTES, &a_map, kb * BK, m0, &sh->full[s]);
          tma_load_2d(tiles + s * STAGE_BYTES + A_BYTES, &b_map, kb * BK, n0, &sh->full[s]);
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
      }
      if (!ok) { atomicOr(status, JV_STATUS_WAIT_EXPIRED); sh->failed = 1; }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- mma issuer
    if (lane == 0) {
      int s = 0, phase = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
        const int acc = it & 1, acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&sh->acc_empty[acc], acc_phase ^ 1)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(&sh->full[s], phase)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint64_t a_desc = smem_desc(smem_u32(tiles + s * STAGE_BYTES));
          const uint64_t b_desc = smem_desc(smem_u32(tiles + s * STAGE_BYTES + A_BYTES));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)   // 32 bytes further along k inside the swizzled row: +2 in the address field
            umma(tmem_d, a_desc + 2 * k, b_desc + 2 * k, (kb | k) != 0);
          umma_commit(&sh->empty[s]);
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&sh->acc_full[acc]);
      }
      if (!ok) { atomicOr(status, JV_STATUS_WAIT_EXPIRED); sh->failed = 1; }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;                     // the 32 TMEM lanes this warp may read
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
      const int acc = it & 1, acc_phase = (it >> 1) & 1;
      const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
      if (!mbar_wait(&sh->acc_full[acc], acc_phase)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const int row = m0 + quad * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
      if (EPI == EPI_SWIGLU) {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(C);
        const int o0 = (n0 / 2);                   // 128 outputs per tile
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          float g[32], u[32];
          tmem_ld32(taddr + c * 32, g);
          tmem_ld32(taddr + 128 + c * 32, u);
          if (row < M) {
            __nv_bfloat16* dst = out + (size_t)row * ldc + o0 + c * 32;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 pk;
              __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float g0 = g[v * 8 + 2 * e], g1 = g[v * 8 + 2 * e + 1];
                h[e] = __floats2bfloat162_rn(g0 / (1.f + expf(-g0)) * u[v * 8 + 2 * e],
                                             g1 / (1.f + expf(-g1)) * u[v * 8 + 2 * e + 1]);
              }
              if (o0 + c * 32 + v * 8 + 8 <= N / 2) *reinterpret_cast<uint4*>(dst + v * 8) = pk;
              else
                for (int e = 0; e < 8; ++e)
                  if (o0 + c * 32 + v * 8 + e < N / 2) dst[v * 8 + e] = reinterpret_cast<__nv_bfloat16*>(&pk)[e];
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          float v[32];
          tmem_ld32(taddr + c * 32, v);
          const int col = n0 + c * 32;
          if (row < M && col < N) {
            if (EPI == EPI_F32) {
              float* dst = reinterpret_cast<float*>(C) + (size_t)row * ldc + col;
              if (col + 32 <= N && (ldc & 3) == 0) {
#pragma unroll
                for (int q = 0; q < 8; ++q) *reinterpret_cast<float4*>(dst + q * 4) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
              } else {
                for (int e = 0; e < 32; ++e) if (col + e < N) dst[e] = v[e];
              }
            } else {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(C) + (size_t)row * ldc + col;
              if (col + 32 <= N && (ldc & 7) == 0) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  uint4 pk;
                  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                  for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(v[q * 8 + 2 * e], v[q * 8 + 2 * e + 1]);
                  *reinterpret_cast<uint4*>(dst + q * 8) = pk;
                }
              } else {
                for (int e = 0; e < 32; ++e) if (col + e < N) dst[e] = __float2bfloat16_rn(v[e]);
              }
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      mbar_arrive(&sh->acc_empty[acc]);
    }
    if (!ok && lane == 0) { atomicOr(status, JV_STATUS_WAIT_EXPIRED); sh->failed = 1; }
  }

  // ---- tear-down: everybody is done with TMEM (or gave up); the allocating warp frees it
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (sh->failed) {
    // a wait ran out: products already issued may still write tensor memory and copies already asked for still land
    // in this block's shared memory; both get a bounded time to finish before tensor memory is freed and the block ends
    if (warp == 1 && lane == 0) drain_products_after_failure(&sh->drain);
    if (warp == 0 && lane == 0)
      for (int s = 0; s < STAGES; ++s)
        if (sh->armed[s] >= 0) drain_copies_after_failure(&sh->full[s], sh->armed[s]);
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

// A 2-D map over a row-major [rows, k] bfloat16 matrix with rows of `ld` elements; boxes of box_rows x 64.
bool make_map(CUtensorMap* map, const void* base, int rows, int k, int ld, int box_rows) {
  auto fn = encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int EPI>
int launch(const CUtensorMap& a, const CUtensorMap& b, void* C, int ldc, int M, int N, int K, int* status,
           cudaStream_t stream) {
  constexpr size_t smem = STAGES * STAGE_BYTES + sizeof(Shared) + 1024;
  static bool ready[JV_MAX_DEVICES];
  static int sm_count[JV_MAX_DEVICES];
  int dev = 0;
  if (!jv_once_per_device(ready, [&] {
        int d = 0, n = 0;
        if (cudaFuncSetAttribute(gemm_tcgen05_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
            cudaGetDevice(&d) != cudaSuccess)
          return false;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || n <= 0) n = 148;
        sm_count[d] = n;
        return true;
      }) || cudaGetDevice(&dev) != cudaSuccess)
    return JV_ERR_UNSUPPORTED;
  const int sms = sm_count[dev];
  const int n_tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int blocks = n_tiles < sms ? n_tiles : sms;
  gemm_tcgen05_kernel<EPI><<<blocks, THREADS, smem, stream>>>(a, b, C, ldc, M, N, K, status);
  return jv_check_launch();
}
}  // namespace

// A: [M, K] bfloat16 rows of lda; B: [N, K] bfloat16 rows of ldb; C: [M, N] rows of ldc, bfloat16 (epilogue 0)
// or float (1); epilogue 2: C is [M, N/2] bfloat16 = silu(gate) * up, where every 256 rows of B are 128
// gate rows followed by the 128 up rows of the same indices (N a multiple of 256).  K, lda, ldb multiples
// of 8; A and B 16-byte aligned.
JV_EXPORT int jv_gemm_tcgen05(const void* A, int lda, const void* B, int ldb, void* C, int ldc, int M, int N, int K,
                              int epilogue, int* status, cudaStream_t stream) {
  if (M == 0 || N == 0) return JV_OK;
  if (K < 8 || (K % 8) || (lda % 8) || (ldb % 8) || ((uintptr_t)A % 16) || ((uintptr_t)B % 16)) return JV_ERR_UNSUPPORTED;
  if (epilogue == EPI_SWIGLU && ((N % 256) || (ldc % 8) || ((uintptr_t)C % 16))) return JV_ERR_UNSUPPORTED;
  CUtensorMap a_map, b_map;
  if (!make_map(&a_map, A, M, K, lda, BM) || !make_map(&b_map, B, N, K, ldb, BN)) return JV_ERR_UNSUPPORTED;
  switch (epilogue) {
    case EPI_BF16: return launch<EPI_BF16>(a_map, b_map, C, ldc, M, N, K, status, stream);
    case EPI_F32: return launch<EPI_F32>(a_map, b_map, C, ldc, M, N, K, status, stream);
    case EPI_SWIGLU: return launch<EPI_SWIGLU>(a_map, b_map, C, ldc, M, N, K, status, stream);
  }
  return JV_ERR_UNSUPPORTED;
}
