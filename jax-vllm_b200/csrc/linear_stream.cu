// y[M, N] = x[M, K] * W[N, K]^T for 9 to 128 rows of x (a batch of decoded tokens): bfloat16 operands,
// 32-bit accumulation, bound by reading W once from HBM.  On the 5th-generation tensor cores with the
// roles turned round: the weight is the 128-row operand (a strip of 128 rows of W = 128 columns of y per
// product), the batch is the narrow one (N of the instruction = rows of x rounded up to 16), so
// y^T[128, rows] = W_strip * x^T accumulates in tensor memory and no tensor-core rows are spent on padding
// the batch.
//
// A block (one per multiprocessor, persistent) has a TMA producer thread that keeps STAGES chunks of 128 k in
// flight as two boxes each (2 x 16 KB of W, 256 bytes of every row, and the matching rows x 256 bytes of x, which every
// block reads again from the L2), one thread that issues eight tcgen05.mma 128 x rows x 16 per chunk into one of two accumulators, and four
// epilogue warps that read the other accumulator out of tensor memory (a lane = a row of W = a column of y)
// and write y, 32 consecutive columns per store instruction.
//
// A unit of work is a strip, or one of `splits` parts of its k when strips alone would leave multiprocessors
// idle or unevenly loaded; block b takes units b, b + grid, ...  With splits, part s of every strip goes to
// parts[s] ([splits, M, N], 32-bit) and the kernel that reads the result adds the parts in the order of s:
// nobody waits and no block sums up after another.  The partition depends on N, K and the number of
// multiprocessors only, never on the batch, and the sum over a part's k runs in ascending order.
// Weights are asked for before the wait on the kernel that produces x (nobody writes them).  Every wait on an
// mbarrier is bounded by a clock deadline; a wait that runs out sets a bit in the status word and the block
// goes to its tear-down (tensor memory is freed) instead of spinning.
#include "common.cuh"
#include "mbarrier.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>

namespace {

constexpr int BM = 128, BOX_K = 64, BOXES = 2, BK = BOX_K * BOXES, UMMA_K = 16;   // a chunk: two boxes of 64 k, 256 bytes of every row
constexpr int W_BOX_BYTES = BM * BOX_K * 2, W_BYTES = W_BOX_BYTES * BOXES;
constexpr int THREADS = 192;
constexpr int MAX_ROWS = 128;
constexpr int SMEM_TILES = 192 * 1024;            // for the stages; 3 to 5 of them depending on the rows of x
constexpr int MAX_STAGES = 8;

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
               ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// Shared-memory matrix descriptor of a K-major tile in the 128-byte-swizzle layout that TMA writes: rows of
// 128 bytes, groups of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1, swizzle mode 2.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

struct Shared {
  uint64_t full[MAX_STAGES], empty[MAX_STAGES], acc_full[2], acc_empty[2];
  uint64_t drain;                 // used only after a wait ran out (see the tear-down)
  uint32_t tmem_base;
  int failed;                     // a role gave up on a wait
  int armed[MAX_STAGES];          // parity of the phase that the producer armed last on full[s]; -1: never
};

struct Params {
  void* y; int ldy; int out_bf16;
  float* parts;
  int M, N, K, rows16;               // rows16: rows of x rounded up to a multiple of 16 (N of the instruction)
  int n_strips, splits, chunks, chunks_per_part, stages, stage_bytes, tmem_cols;
  int* status;
};

__global__ void __launch_bounds__(THREADS, 1) linear_stream_kernel(const __grid_constant__ CUtensorMap w_map,
                                                                   const __grid_constant__ CUtensorMap x_map,
                                                                   const Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  Shared* sh = reinterpret_cast<Shared*>(tiles + p.stages * p.stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_units = p.n_strips * p.splits;
  pdl_trigger();

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&sh->full[s], 1); mbar_init(&sh->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&sh->acc_full[a], 1); mbar_init(&sh->acc_empty[a], 128); }
    mbar_init(&sh->drain, 1);
    sh->failed = 0;
    for (int s = 0; s < MAX_STAGES; ++s) sh->armed[s] = -1;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh->tmem_base)), "r"(p.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = sh->tmem_base;
  const int acc_cols = p.tmem_cols / 2;

  // the chunks of this block, unit after unit: (unit, chunk index, end, first row of the strip)
  struct Cursor { int u, c, c1, n0; };
  auto open_unit = [&](Cursor& it) {
    if (it.u < n_units) {
      const int part = it.u % p.splits;
      it.n0 = (it.u / p.splits) * BM;
      it.c = part * p.chunks_per_part;
      it.c1 = min(p.chunks, it.c + p.chunks_per_part);
    }
  };
  auto advance = [&](Cursor& it) {
    if (++it.c >= it.c1) { it.u += gridDim.x; open_unit(it); }
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      const int x_box = p.rows16 * 128, x_bytes = x_box * BOXES;
      auto load_w = [&](int s, int c, int n0) {
#pragma unroll
        for (int b = 0; b < BOXES; ++b)
          tma_load_2d(tiles + s * p.stage_bytes + b * W_BOX_BYTES, &w_map, c * BK + b * BOX_K, n0, &sh->full[s]);
      };
      auto load_x = [&](int s, int c) {
#pragma unroll
        for (int b = 0; b < BOXES; ++b)
          tma_load_2d(tiles + s * p.stage_bytes + W_BYTES + b * x_box, &x_map, c * BK + b * BOX_K, 0, &sh->full[s]);
      };
      Cursor it{(int)blockIdx.x, 0, 0, 0};
      open_unit(it);
      // the weights of the first chunks are asked for before the kernel that makes x has finished
      Cursor ahead = it;
      int n_ahead = 0;
      for (; n_ahead < p.stages && ahead.u < n_units; ++n_ahead, advance(ahead)) {
        sh->armed[n_ahead] = 0;
        mbar_expect_tx(&sh->full[n_ahead], W_BYTES + x_bytes);
        load_w(n_ahead, ahead.c, ahead.n0);
      }
      pdl_wait();
      for (int s = 0; s < n_ahead; ++s, advance(it))
        load_x(s, it.c);
      int s = n_ahead == p.stages ? 0 : n_ahead, phase = n_ahead == p.stages ? 1 : 0;
      bool ok = true;
      for (; it.u < n_units && ok; advance(it)) {
        if (!mbar_wait(&sh->empty[s], phase ^ 1)) { ok = false; break; }
        sh->armed[s] = phase;
        mbar_expect_tx(&sh->full[s], W_BYTES + x_bytes);
        load_w(s, it.c, it.n0);
        load_x(s, it.c);
        if (++s == p.stages) { s = 0; phase ^= 1; }
      }
      if (!ok) { atomicOr(p.status, JV_STATUS_WAIT_EXPIRED); sh->failed = 1; }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- mma issuer
    if (lane == 0) {
      // bfloat16 x bfloat16 -> float, both operands K-major, M = 128, N = rows of x rounded up to 16
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.rows16 >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      int s = 0, phase = 0, n = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++n) {
        const int acc = n & 1, acc_phase = (n >> 1) & 1;
        const int part = u % p.splits;
        const int c0 = part * p.chunks_per_part, c1 = min(p.chunks, c0 + p.chunks_per_part);
        if (!mbar_wait(&sh->acc_empty[acc], acc_phase ^ 1)) { ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t tmem_d = tmem_base + acc * acc_cols;
        for (int c = c0; c < c1; ++c) {
          if (!mbar_wait(&sh->full[s], phase)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
          for (int b = 0; b < BOXES; ++b) {
            const uint64_t a_desc = smem_desc(smem_u32(tiles + s * p.stage_bytes + b * W_BOX_BYTES));
            const uint64_t b_desc = smem_desc(smem_u32(tiles + s * p.stage_bytes + W_BYTES + b * p.rows16 * 128));
#pragma unroll
            for (int k = 0; k < BOX_K / UMMA_K; ++k)   // 32 bytes further along k inside the swizzled row: +2 in the address field
              umma(tmem_d, a_desc + 2 * k, b_desc + 2 * k, idesc, (c > c0 || b > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&sh->empty[s]);
          if (++s == p.stages) { s = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&sh->acc_full[acc]);
      }
      if (!ok) { atomicOr(p.status, JV_STATUS_WAIT_EXPIRED); sh->failed = 1; }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;                     // the 32 TMEM lanes this warp may read
    int n = 0;
    bool ok = true;
    pdl_wait();                                    // nothing is written before the kernels before this one are done
    for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++n) {
      const int acc = n & 1, acc_phase = (n >> 1) & 1;
      const int part = u % p.splits;
      const int col = (u / p.splits) * BM + quad * 32 + lane;      // column of y = row of W
      if (!mbar_wait(&sh->acc_full[acc], acc_phase)) { ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * acc_cols;
#pragma unroll 1
      for (int m0 = 0; m0 < p.rows16; m0 += 16) {
        float v[16];
        tmem_ld16(taddr + m0, v);
        if (col < p.N) {
          if (p.splits > 1) {
            float* dst = p.parts + ((size_t)part * p.M + m0) * p.N + col;
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (m0 + i < p.M) dst[(size_t)i * p.N] = v[i];
          } else if (p.out_bf16) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.y) + (size_t)m0 * p.ldy + col;
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (m0 + i < p.M) dst[(size_t)i * p.ldy] = __float2bfloat16_rn(v[i]);
          } else {
            float* dst = reinterpret_cast<float*>(p.y) + (size_t)m0 * p.ldy + col;
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (m0 + i < p.M) dst[(size_t)i * p.ldy] = v[i];
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      mbar_arrive(&sh->acc_empty[acc]);
    }
    if (!ok && lane == 0) { atomicOr(p.status, JV_STATUS_WAIT_EXPIRED); sh->failed = 1; }
  }

  // ---- tear-down: everybody is done with tensor memory (or gave up); the allocating warp frees it
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (sh->failed) {
    // a wait ran out: products already issued may still write tensor memory and copies already asked for still land
    // in this block's shared memory; both get a bounded time to finish before tensor memory is freed and the block ends
    if (warp == 1 && lane == 0) drain_products_after_failure(&sh->drain);
    if (warp == 0 && lane == 0)
      for (int s = 0; s < p.stages; ++s)
        if (sh->armed[s] >= 0) drain_copies_after_failure(&sh->full[s], sh->armed[s]);
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
  }
}

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  }
  return fn;
}

// A 2-D map over a row-major [rows, k] bfloat16 matrix with rows of `ld` elements; boxes of box_rows x 64.
bool make_map(CUtensorMap* map, const void* base, int rows, int k, int ld, int box_rows) {
  auto fn = encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BOX_K, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int multiprocessors() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  return sms;
}

// Into how many parts the k of a strip is cut: blocks take units in turn, so a launch takes as long as the
// most loaded block, (units / blocks rounded up) x chunks of a part.  The parts cost their own bytes (written
// in 32 bits and read again), counted here for 64 rows whatever the batch is.  At most 8 parts of at least 4
// chunks; cut only if that gains a twentieth.
int choose_splits(int n_strips, int K, int sms) {
  const int chunks = (K + BK - 1) / BK;
  auto cost = [&](int s) {
    const int cpp = (chunks + s - 1) / s;
    const long long units = (long long)n_strips * s;
    const long long rounds = (units + sms - 1) / sms;
    const double extra = s > 1 ? 1.0 + (double)s * 128.0 / (double)K : 1.0;
    return (double)rounds * cpp * extra;
  };
  int best = 1;
  double best_cost = cost(1);
  for (int s = 2; s <= 8; ++s) {
    const int cpp = (chunks + s - 1) / s;
    if (cpp < 4 || (long long)(s - 1) * cpp >= chunks) continue;     // every part has chunks of its own
    const double c = cost(s);
    if (c < best_cost) { best = s; best_cost = c; }
  }
  if (best_cost > cost(1) * 0.95) best = 1;
  return best;
}
}  // namespace

// Largest number of rows of x the kernel takes.
JV_EXPORT int jv_linear_stream_max_rows() { return MAX_ROWS; }

// Into how many parts the kernel would best cut the k of a strip for an [N, K] weight on this device (1: not at all).
JV_EXPORT int jv_linear_stream_plan(int N, int K) { return choose_splits((N + BM - 1) / BM, K, multiprocessors()); }

// X: [M, K] bfloat16 rows of ldx elements, M up to 128; W: [N, K] bfloat16 rows of ldw.  splits == 1: Y [M, N] rows of
// ldy, bfloat16 (out_dtype 1) or float (0).  splits > 1 (at most 8, every part with chunks of its own): Y is not
// written; parts [splits, M, N] float gets the sums over the parts of k, to be added by the reader.
// K, ldx and ldw must be multiples of 8 and X, W 16-byte aligned.
JV_EXPORT int jv_linear_stream(const void* X, int ldx, const void* W, int ldw, void* Y, int out_dtype, int ldy, int M,
                               int N, int K, float* parts, int splits, int* status, cudaStream_t stream) {
  if (M == 0 || N == 0) return JV_OK;
  if (M > MAX_ROWS || K < 8 || (K % 8) || (ldx % 8) || (ldw % 8) || ((uintptr_t)X % 16) || ((uintptr_t)W % 16))
    return JV_ERR_UNSUPPORTED;
  if (out_dtype != 0 && out_dtype != 1) return JV_ERR_UNSUPPORTED;
  const int chunks = (K + BK - 1) / BK;
  if (splits < 1 || splits > 8 || (splits > 1 && parts == nullptr)) return JV_ERR_UNSUPPORTED;
  const int cpp = (chunks + splits - 1) / splits;
  if ((long long)(splits - 1) * cpp >= chunks) return JV_ERR_UNSUPPORTED;
  Params p;
  p.y = Y; p.ldy = ldy; p.out_bf16 = out_dtype == 1; p.parts = parts;
  p.M = M; p.N = N; p.K = K; p.rows16 = (M + 15) / 16 * 16;
  p.n_strips = (N + BM - 1) / BM; p.splits = splits; p.chunks = chunks; p.chunks_per_part = cpp;
  p.stage_bytes = W_BYTES + BOXES * p.rows16 * 128;          // a multiple of 1 KB: rows16 is a multiple of 16
  p.stages = SMEM_TILES / p.stage_bytes < MAX_STAGES ? SMEM_TILES / p.stage_bytes : MAX_STAGES;
  p.tmem_cols = 32;
  while (p.tmem_cols < 2 * p.rows16) p.tmem_cols *= 2;
  p.status = status;
  CUtensorMap w_map, x_map;
  if (!make_map(&w_map, W, N, K, ldw, BM) || !make_map(&x_map, X, M, K, ldx, p.rows16)) return JV_ERR_UNSUPPORTED;
  constexpr size_t smem = SMEM_TILES + sizeof(Shared) + 1024;
  static bool ready[JV_MAX_DEVICES];
  if (!jv_once_per_device(ready, [&] {
        return cudaFuncSetAttribute(linear_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
      }))
    return JV_ERR_UNSUPPORTED;
  const long long units = (long long)p.n_strips * splits;
  const int sms = multiprocessors();
  const int blocks = units < sms ? (int)units : sms;
  return jv_launch(linear_stream_kernel, dim3(blocks), dim3(THREADS), smem, stream, w_map, x_map, p);
}
