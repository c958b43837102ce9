// Decode attention on the 5th-generation tensor cores, for head size 128 and up to 16 query heads per
// kv head.  One query token has too few rows for a 128-row tensor-core tile, so the products are taken
// the other way round: the 128 KEYS of a tile are the rows,
//     S^T[key, head] = K[key, :] . Q[head, :]       A = K tile (K-major), B = Q (16 rows, K-major)
//     O^T[d, head]  += V[key, d]^T P^T[key, head]   A = V tile (MN-major), B = P^T (16 rows, K-major)
// with S^T (2 x 16 columns) and O^T (2 x 16 columns) in tensor memory.  Keys and values stream from the
// pages by TMA (one box per page and half of the head) through a 3-stage ring; nothing but the 4-byte
// score and the probability of each (key, head) passes through registers: a softmax thread owns one key row.
//
// The softmax is kept against a reference maximum per head that only moves when some score exceeds it by
// more than 2^8; the per-key sums are kept per thread and added up once per segment.  So the usual tile
// costs a thread: one TMEM load, G exponentials, G two-byte stores, one named barrier.
//
// The launch is persistent: the key tiles of all (request, kv head) pairs form one list, and block b of B
// takes the tiles [b T / B, (b+1) T / B) of it, whatever the batch and the lengths are.  The run of a block's
// tiles that belong to one pair is a segment; the loads, the products and the softmax of the next segment
// follow the last tile of this one without a gap (two query buffers, two O^T buffers).  A pair that lies
// within one block is normalised and written at once; otherwise each segment leaves its unnormalised O^T and
// (reference, sum) in scratch memory and the block that finishes a pair last merges its segments in
// ascending order (nobody waits).  Every mbarrier wait is bounded by a clock deadline and reports to the
// status word.
//
// Two ways in: after a kernel that has normed and rotated the queries and written the new token's key and value
// into the cache (csrc/rope_kv.cu: steps that mix prompt portions and single tokens), or, for steps of single
// tokens only, straight after the product q|k|v: a warp of this kernel then norms and rotates the segment's
// queries into the operand tile, and the block that holds a pair's last tile does the same for the new key,
// writes key and value to the cache, and adds the new token to the softmax as one more key at the pair's end.
// Nothing that this kernel streams depends on the kernel before it then: only that warp waits for it.
//
// Restrictions (the caller falls back to the mma.sync kernel): bfloat16, head size 128, no window, at most
// 16 query heads per kv head, page size a power of two from 8 to 128, at most 512 requests.
#include "common.cuh"
#include "mbarrier.cuh"
#include "qk_prepare.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>
#include <math.h>

namespace {

constexpr int D = 128, BN = 128, NH = 16;        // head size, keys per tile, columns (query heads, padded)
constexpr int TILE_BYTES = 128 * 128 * 2;        // a 128 x 128 bfloat16 tile: two halves of [128 rows][128 bytes]
constexpr int HALF_BYTES = 128 * 128;
constexpr int SMALL_BYTES = NH * 128 * 2;        // a 16 x 128 tile (Q, P^T): two halves of [16 rows][128 bytes]
constexpr int SMALL_HALF = NH * 128;
// Key and value tiles in flight: two of each.  Three fit and were slower at every size (64 requests x 2,048 keys:
// 98.3 us with three, 91.7 us with two; one: 127.8 us).
constexpr int STAGES = 2;
constexpr int THREADS = 256;                      // warps: keys producer, mma issuer, 4 x softmax, values producer, query producer
constexpr int TMEM_COLS = 64;                    // S^T buffers at columns 0 and 16, O^T buffers at 32 and 48
constexpr int MAX_WORK = 512;                    // requests in one launch
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LAZY = 8.f;

struct Params {
  __nv_bfloat16* out; int out_stride;
  float* part_o; float* part_ml; int* counters;
  const int* block_table; int table_width;
  const int* cu_seqlens; const int* start_pos; const int* work;
  int n_work, n_q_heads, n_kv_heads, page_size, num_pages;
  float scale_log2;
  int* status;
  // with the preparation of queries, keys and values in this kernel (FUSED): the product q|k|v as it comes
  // (rows of qkv_stride elements: query heads, key heads, value heads), the tables and weights of the per-head
  // norm and the rotation, and the caches to write the new token's key and value to
  const __nv_bfloat16* qkv; int qkv_stride;
  const float* inv_freq;                      // [64] or null (no rotation)
  const void* q_norm_w; const void* k_norm_w; int norm_w_f32; float eps;    // null: no norm
  __nv_bfloat16* k_cache; __nv_bfloat16* v_cache;
};

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
               ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, int x, int y, int z, int w, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n"
               ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar)) : "memory");
}
// K-major operand tile: rows of 128 bytes along k, 8-row groups 1024 bytes apart, 128-byte swizzle.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// MN-major operand tile: rows of 128 bytes run along m (64 elements), consecutive rows are consecutive k, 8 rows =
// 1024 bytes (stride byte offset); the next 64 m are HALF_BYTES further (leading byte offset).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(HALF_BYTES >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// bfloat16 x bfloat16 -> float, M = 128, N = 16; A K-major (S^T = K Q^T) or MN-major (O^T = V^T P^T); B K-major.
constexpr uint32_t IDESC_QK = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NH >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
constexpr uint32_t IDESC_PV = IDESC_QK | (1u << 15);

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// One row (TMEM lane) per thread, N consecutive 32-bit columns.
template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, float (&v)[N]) {
  static_assert(N == 4 || N == 8 || N == 16, "columns per load");
  uint32_t r[N];
  if constexpr (N == 4) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr));
  } else if constexpr (N == 8) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr));
  } else {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
  }
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = __uint_as_float(r[i]);
}
template <int N>
__device__ __forceinline__ void tmem_st(uint32_t taddr, const float (&v)[N]) {
  static_assert(N == 4 || N == 8 || N == 16, "columns per store");
#define JV_U(i) "r"(__float_as_uint(v[i]))
  if constexpr (N == 4) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(taddr), JV_U(0), JV_U(1), JV_U(2), JV_U(3) : "memory");
  } else if constexpr (N == 8) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n"
                 ::"r"(taddr), JV_U(0), JV_U(1), JV_U(2), JV_U(3), JV_U(4), JV_U(5), JV_U(6), JV_U(7) : "memory");
  } else {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
                 ::"r"(taddr), JV_U(0), JV_U(1), JV_U(2), JV_U(3), JV_U(4), JV_U(5), JV_U(6), JV_U(7), JV_U(8), JV_U(9), JV_U(10),
                   JV_U(11), JV_U(12), JV_U(13), JV_U(14), JV_U(15) : "memory");
  }
#undef JV_U
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
#define TC_FENCE_BEFORE() asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory")
#define TC_FENCE_AFTER() asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory")
#define PROXY_FENCE() asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory")
#define SOFTMAX_BARRIER() asm volatile("bar.sync 1, 128;\n" ::: "memory")
// Barrier of the 128 softmax threads that also tells every one of them whether any had `flag` set.
__device__ __forceinline__ bool softmax_barrier_or(bool flag) {
  uint32_t any;
  asm volatile("{\n.reg .pred p, q;\nsetp.ne.b32 q, %1, 0;\nbar.red.or.pred p, 1, 128, q;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(any) : "r"((uint32_t)flag) : "memory");
  return any != 0;
}

struct Shared {
  uint64_t q_full[2], q_empty[2], k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
  uint64_t s_full[2], p_full[2], o_done[2], o_free[2];
  uint64_t drain;                // used only after a wait ran out (see the tear-down)
  uint32_t tmem_base;
  int is_last;
  int failed;                    // a role gave up on a wait
  int armed[2][STAGES];          // parity of the phase that the key (0) / value (1) producer armed last on a stage; -1: never
  int armed_q[2];                // the same for the two query buffers
  float m_ref[NH];               // reference maxima of the running segment (raw score units)
  float alpha[NH];
  float red[4][NH];              // per-warp partial maxima / sums
  float s_new[2][NH];            // FUSED: raw scores of the new token's key, per segment buffer
  float v_new[2][D];             // FUSED: the new token's value
  int entry[MAX_WORK];           // request of work item i
  int pos[MAX_WORK];             // its query position (= number of keys before it)
  int token[MAX_WORK];           // its row in q and out
  int pre[MAX_WORK + 1];         // key tiles (per kv head) of the work items before i
};

// Where a role stands in the list of tiles: work item, kv head, tile of the pair, tiles of the pair, segment number.
struct Cursor { int i, head, j, nt, seg; };

// FUSED: the kernel takes q|k|v as the product leaves it and does the per-head norm, the rotation and the write
// of the new token's key and value itself; the new token (not in the cache while the kernel streams it) joins
// the softmax as one more key at the end of the pair's last tile.  Otherwise a kernel before this one has done
// all that, and the new token's key and value are read from the cache like the others.
template <int GP, bool FUSED>     // GP: query heads per kv head, rounded up to 4, 8 or 16
__global__ void __launch_bounds__(THREADS, 1) attn_decode_tcgen05_kernel(const __grid_constant__ CUtensorMap q_map,
                                                                         const __grid_constant__ CUtensorMap k_map,
                                                                         const __grid_constant__ CUtensorMap v_map,
                                                                         const Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* k_s = base;                                   // [stages][2 halves of d][128 keys][128 B]
  unsigned char* v_s = k_s + STAGES * TILE_BYTES;              // [stages][2 halves of d][128 keys][128 B]
  unsigned char* q_s = v_s + STAGES * TILE_BYTES;              // [2 buffers][2 halves of d][16 rows][128 B]
  unsigned char* p_s = q_s + 2 * SMALL_BYTES;                  // [2 buffers][2 halves of keys][16 rows][128 B]
  Shared* sh = reinterpret_cast<Shared*>(p_s + 2 * SMALL_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int Hkv = p.n_kv_heads, G = p.n_q_heads / p.n_kv_heads;

  pdl_trigger();
  // ---- the requests' lengths are on their way while the barriers and the tensor memory are set up
  const int my_entry = (int)threadIdx.x < p.n_work ? p.work[2 * threadIdx.x] : 0;
  int my_pos = 0, my_token = 0;
  if ((int)threadIdx.x < p.n_work) { my_pos = p.start_pos[my_entry]; my_token = p.cu_seqlens[my_entry]; }
  if (threadIdx.x == 32) {
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&q_map) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&k_map) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(&v_map) : "memory");
  }
  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->q_full[b], 1); mbar_init(&sh->q_empty[b], 1);
      mbar_init(&sh->s_full[b], 1); mbar_init(&sh->p_full[b], 128); mbar_init(&sh->o_done[b], 1); mbar_init(&sh->o_free[b], 128);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sh->k_full[s], 1); mbar_init(&sh->k_empty[s], 1);
      mbar_init(&sh->v_full[s], 1); mbar_init(&sh->v_empty[s], 1);
      sh->armed[0][s] = sh->armed[1][s] = -1;
    }
    mbar_init(&sh->drain, 1);
    sh->failed = 0;
    sh->armed_q[0] = sh->armed_q[1] = -1;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  // zeros where no copy will write: the unused rows of Q (heads G..15) and of P^T, in both buffers of each
  for (int i = threadIdx.x; i < 4 * SMALL_BYTES / 16; i += THREADS) reinterpret_cast<uint4*>(q_s)[i] = make_uint4(0, 0, 0, 0);
  PROXY_FENCE();
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh->tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  // ---- the list of tiles: work item i has pos/128 + 1 tiles for each kv head
  for (int i = threadIdx.x; i < p.n_work; i += THREADS) {
    int e = my_entry, pos = my_pos, token = my_token;
    if (i >= THREADS) { e = p.work[2 * i]; pos = p.start_pos[e]; token = p.cu_seqlens[e]; }
    if (pos < 0 || pos / p.page_size >= p.table_width) {        // a length that the block table cannot hold
      atomicOr(p.status, JV_STATUS_BAD_ROW);
      pos = 0;
    }
    sh->entry[i] = e; sh->pos[i] = pos; sh->token[i] = token; sh->pre[i + 1] = pos / BN + 1;
  }
  TC_FENCE_BEFORE();
  __syncthreads();
  TC_FENCE_AFTER();
  const uint32_t tmem = sh->tmem_base;
  if (warp == 0) {
    int carry = 0;
    for (int first = 0; first < p.n_work; first += 32) {
      const int idx = first + lane;
      int v = idx < p.n_work ? sh->pre[idx + 1] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
      }
      if (idx < p.n_work) sh->pre[idx + 1] = v + carry;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
    if (lane == 0) sh->pre[0] = 0;
  }
  __syncthreads();
  const long long T = (long long)Hkv * sh->pre[p.n_work];
  const int nb = (int)min((long long)gridDim.x, T);            // with fewer tiles than blocks, one tile each
  if ((int)blockIdx.x >= nb) {
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    return;
  }
  const bool narrow = T * (nb + 1) < (1ll << 31);              // then 32-bit arithmetic holds every product below
  auto muldiv = [&](long long a, int b, long long c) -> int {  // floor(a b / c)
    return narrow ? (int)((unsigned)a * (unsigned)b / (unsigned)c) : (int)(a * b / c);
  };
  const int g0 = muldiv(T, blockIdx.x, nb), g1 = muldiv(T, blockIdx.x + 1, nb);
  const int ntb = g1 - g0;                                     // at least one
  auto block_of = [&](long long g) -> int {                    // the block whose range holds tile g
    return narrow ? (int)((((unsigned)g + 1u) * (unsigned)nb - 1u) / (unsigned)T) : (int)(((g + 1) * nb - 1) / T);
  };
  Cursor c0;
  {
    int lo = 0, hi = p.n_work - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if ((long long)sh->pre[mid] * Hkv <= g0) lo = mid; else hi = mid - 1;
    }
    c0.i = lo; c0.nt = sh->pre[lo + 1] - sh->pre[lo];
    const int rem = g0 - sh->pre[lo] * Hkv;
    c0.head = rem / c0.nt; c0.j = rem - c0.head * c0.nt; c0.seg = 0;
  }
  auto advance = [&](Cursor& c) {
    if (++c.j == c.nt) {
      c.j = 0; ++c.seg;
      if (++c.head == Hkv) {
        c.head = 0; ++c.i;
        c.nt = c.i < p.n_work ? sh->pre[c.i + 1] - sh->pre[c.i] : 1;
      }
    }
  };

  // The kernel before this one wrote the query and the new token's key and value.  Every other key and value
  // is from earlier steps, so the producers stream them at once, under the kernels before, and wait for those
  // only when they come to a pair's last tile (which holds the new token); the query producer waits first.
  if (warp == 0 || warp == 6) {
    // ------------------------------------------------------------------ producers: warp 0 keys, warp 6 values
    const int which = warp == 6;
    bool waited = false;
    const int P = p.page_size, pages_per_tile = BN / P;
    auto tile_pages = [&](const Cursor& c, bool wanted) -> int {   // lane l: the l-th page of the tile, -1 = none
      int page = -1;
      if (wanted && lane < pages_per_tile) {
        const int pi = c.j * pages_per_tile + lane;
        if (pi * P < sh->pos[c.i] + (FUSED ? 0 : 1) && pi < p.table_width) {
          page = p.block_table[(size_t)sh->entry[c.i] * p.table_width + pi];
          if (page < 0 || page >= p.num_pages) { atomicOr(p.status, JV_STATUS_BAD_PAGE); page = -1; }
        }
      }
      return page;
    };
    auto load_tile = [&](int t, int page, int kv_head) -> bool {
      const int s = t % STAGES, ph = (t / STAGES) & 1;
      uint64_t* full = which ? &sh->v_full[s] : &sh->k_full[s];
      uint64_t* empty = which ? &sh->v_empty[s] : &sh->k_empty[s];
      unsigned char* dst = (which ? v_s : k_s) + s * TILE_BYTES;
      const CUtensorMap* map = which ? &v_map : &k_map;
      const int n_pages = __popc(__ballot_sync(0xffffffffu, page >= 0));
      bool ok = true;
      if (lane == 0) {
        ok = mbar_wait(empty, ph ^ 1);
        if (ok) { sh->armed[which][s] = ph; mbar_expect_tx(full, n_pages * P * 128 * 2); }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);    // also orders the announcement before the copies
      if (ok && page >= 0) {                   // lane l starts the two boxes of page l
        tma_load_4d(dst + lane * P * 128, map, 0, kv_head, 0, page, full);
        tma_load_4d(dst + HALF_BYTES + lane * P * 128, map, 64, kv_head, 0, page, full);
      }
      return ok;
    };
    Cursor c = c0;
    bool ok = true;
    int pages = tile_pages(c, true);
    for (int t = 0; t < ntb && ok; ++t) {
      Cursor n = c;
      advance(n);
      const int pages_next = tile_pages(n, t + 1 < ntb);
      if (!FUSED && !waited && c.j == c.nt - 1) { pdl_wait(); waited = true; }
      if (ok) ok = load_tile(t, pages, c.head);
      pages = pages_next;
      c = n;
    }
    if (!ok && lane == 0) { atomicOr(p.status, JV_STATUS_WAIT_EXPIRED); sh->failed = 1; }
  } else if (warp == 7) {
    // ------------------------------------------------------------------ query producer: once per segment
    if constexpr (!FUSED) {
      if (lane == 0) {
        pdl_wait();
        Cursor c = c0;
        bool ok = true;
        for (int t = 0; t < ntb && ok; ++t) {
          if (t == 0 || c.j == 0) {               // a segment begins (the buffer was last read two segments ago)
            const int sp = c.seg & 1;
            if (c.seg >= 2) ok = mbar_wait(&sh->q_empty[sp], ((c.seg >> 1) - 1) & 1);
            if (ok) {
              sh->armed_q[sp] = (c.seg >> 1) & 1;
              mbar_expect_tx(&sh->q_full[sp], G * 128 * 2);
              tma_load_3d(q_s + sp * SMALL_BYTES, &q_map, 0, c.head * G, sh->token[c.i], &sh->q_full[sp]);
              tma_load_3d(q_s + sp * SMALL_BYTES + SMALL_HALF, &q_map, 64, c.head * G, sh->token[c.i], &sh->q_full[sp]);
            }
          }
          advance(c);
        }
        if (!ok) { atomicOr(p.status, JV_STATUS_WAIT_EXPIRED); sh->failed = 1; }
      }
    } else {
      // The whole warp prepares the segment's queries from q|k|v as the product left it: per-head norm and
      // rotation in 32-bit, rounded to bfloat16 into the swizzled operand tile.  Lane l has the elements
      // 2l, 2l+1 of a head and their rotation partners 64+2l, 64+2l+1.  The block that holds a pair's last tile
      // does the same for the new token's key, writes key and value to the cache (for later steps), and leaves
      // the new key's scores and the value in shared memory for the softmax warps.
      pdl_wait();
      auto weight = [&](const void* w, int i) -> float {
        return p.norm_w_f32 ? reinterpret_cast<const float*>(w)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(w)[i]);
      };
      // norm and rotation of one head whose four elements of this lane are (lo, hi); the result is rounded as the
      // operand will be
      auto prepare = [&](__nv_bfloat162 lo2, __nv_bfloat162 hi2, const void* w, const float (&cs)[2], const float (&sn)[2],
                         float (&out)[4]) {
        const float2 lo = __bfloat1622float2(lo2), hi = __bfloat1622float2(hi2);
        float a[2] = {lo.x, lo.y}, b[2] = {hi.x, hi.y};
        qk_prepare_head<2>(a, b, 2 * lane, D / 2, w != nullptr, p.eps, [&](int i) { return weight(w, i); }, cs, sn);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          out[i] = __bfloat162float(__float2bfloat16_rn(a[i]));
          out[2 + i] = __bfloat162float(__float2bfloat16_rn(b[i]));
        }
      };
      Cursor c = c0;
      bool ok = true;
      for (int t = 0; t < ntb && ok; ++t) {
        if (t == 0 || c.j == 0) {
          const int sp = c.seg & 1, pos = sh->pos[c.i];
          const bool has_last = t + (c.nt - 1 - c.j) < ntb;          // the pair's last tile is in this block's range
          // ---- all loads first, so that they are under way together
          const __nv_bfloat16* row = p.qkv + (size_t)sh->token[c.i] * p.qkv_stride;
          __nv_bfloat162 q_lo[GP], q_hi[GP], k_lo, k_hi, v_lo, v_hi;
#pragma unroll
          for (int h = 0; h < GP; ++h) {
            if (h < G) {
              const __nv_bfloat16* src = row + (size_t)(c.head * G + h) * D;
              q_lo[h] = *reinterpret_cast<const __nv_bfloat162*>(src + 2 * lane);
              q_hi[h] = *reinterpret_cast<const __nv_bfloat162*>(src + 64 + 2 * lane);
            }
          }
          int page = -1;
          if (has_last) {
            const __nv_bfloat16* k_src = row + (size_t)(p.n_q_heads + c.head) * D;
            const __nv_bfloat16* v_src = row + (size_t)(p.n_q_heads + Hkv + c.head) * D;
            k_lo = *reinterpret_cast<const __nv_bfloat162*>(k_src + 2 * lane);
            k_hi = *reinterpret_cast<const __nv_bfloat162*>(k_src + 64 + 2 * lane);
            v_lo = *reinterpret_cast<const __nv_bfloat162*>(v_src + 2 * lane);
            v_hi = *reinterpret_cast<const __nv_bfloat162*>(v_src + 64 + 2 * lane);
            const int pi = pos / p.page_size;
            if (pi < p.table_width) page = p.block_table[(size_t)sh->entry[c.i] * p.table_width + pi];
          }
          float cs[2] = {1.f, 1.f}, sn[2] = {0.f, 0.f};
          if (p.inv_freq != nullptr) {
#pragma unroll
            for (int i = 0; i < 2; ++i) qk_rotation(pos, p.inv_freq[2 * lane + i], &sn[i], &cs[i]);
          }
          if (lane == 0 && c.seg >= 2)                               // buffers of the segment before the last one:
            ok = mbar_wait(&sh->q_empty[sp], ((c.seg >> 1) - 1) & 1) &&      // its products have read the queries,
                 mbar_wait(&sh->o_free[sp], ((c.seg >> 1) - 1) & 1);         // its softmax the new key's scores and value
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (ok) {
            float kr[4] = {0.f, 0.f, 0.f, 0.f};
            if (has_last) {
              prepare(k_lo, k_hi, p.k_norm_w, cs, sn, kr);
              if (page >= 0 && page < p.num_pages) {
                const size_t slot = (((size_t)page * p.page_size + (pos % p.page_size)) * Hkv + c.head) * D;
                *reinterpret_cast<__nv_bfloat162*>(p.k_cache + slot + 2 * lane) = __floats2bfloat162_rn(kr[0], kr[1]);
                *reinterpret_cast<__nv_bfloat162*>(p.k_cache + slot + 64 + 2 * lane) = __floats2bfloat162_rn(kr[2], kr[3]);
                *reinterpret_cast<__nv_bfloat162*>(p.v_cache + slot + 2 * lane) = v_lo;
                *reinterpret_cast<__nv_bfloat162*>(p.v_cache + slot + 64 + 2 * lane) = v_hi;
              } else if (lane == 0) {
                atomicOr(p.status, JV_STATUS_BAD_PAGE);
              }
              const float2 vl = __bfloat1622float2(v_lo), vh = __bfloat1622float2(v_hi);
              sh->v_new[sp][2 * lane] = vl.x; sh->v_new[sp][2 * lane + 1] = vl.y;
              sh->v_new[sp][64 + 2 * lane] = vh.x; sh->v_new[sp][64 + 2 * lane + 1] = vh.y;
            }
            unsigned char* qt = q_s + sp * SMALL_BYTES;
#pragma unroll
            for (int h = 0; h < GP; ++h) {
              if (h < G) {
                float qr[4];
                prepare(q_lo[h], q_hi[h], p.q_norm_w, cs, sn, qr);
                // element d of head h: half d / 64, row h of 128 bytes, 16-byte chunk (d % 64) / 8 swizzled with the row
                const int off = h * 128 + ((((2 * lane) >> 3) ^ (h & 7)) << 4) + ((2 * lane) & 7) * 2;
                *reinterpret_cast<__nv_bfloat162*>(qt + off) = __floats2bfloat162_rn(qr[0], qr[1]);
                *reinterpret_cast<__nv_bfloat162*>(qt + SMALL_HALF + off) = __floats2bfloat162_rn(qr[2], qr[3]);
                if (has_last) {
                  float dot = qr[0] * kr[0] + qr[1] * kr[1] + qr[2] * kr[2] + qr[3] * kr[3];
#pragma unroll
                  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                  if (lane == 0) sh->s_new[sp][h] = dot;
                }
              }
            }
            PROXY_FENCE();                        // the queries are read by the tensor core
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->q_full[sp]);
          }
        }
        advance(c);
      }
      if (!ok && lane == 0) { atomicOr(p.status, JV_STATUS_WAIT_EXPIRED); sh->failed = 1; }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- mma issuer
    if (lane == 0) {
      auto issue_qk = [&](int t, const Cursor& c) -> bool {      // S^T[t % 2] = K_t Q^T
        const int s = t % STAGES, sp = c.seg & 1;
        if ((t == 0 || c.j == 0) && !mbar_wait(&sh->q_full[sp], (c.seg >> 1) & 1)) return false;
        if (!mbar_wait(&sh->k_full[s], (t / STAGES) & 1)) return false;
        TC_FENCE_AFTER();
        const uint32_t tmem_s = tmem + (t & 1) * NH;
        const uint64_t k_desc = desc_k_major(smem_u32(k_s + s * TILE_BYTES));
        const uint64_t q_desc = desc_k_major(smem_u32(q_s + sp * SMALL_BYTES));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma(tmem_s, k_desc + (kk >> 2) * (HALF_BYTES >> 4) + 2 * (kk & 3), q_desc + (kk >> 2) * (SMALL_HALF >> 4) + 2 * (kk & 3),
               IDESC_QK, kk != 0);
        umma_commit(&sh->k_empty[s]);
        if (t == ntb - 1 || c.j == c.nt - 1) umma_commit(&sh->q_empty[sp]);   // the segment's last use of its query
        umma_commit(&sh->s_full[t & 1]);
        return true;
      };
      Cursor cq = c0, cp = c0;
      bool ok = issue_qk(0, cq);
      for (int t = 0; t < ntb && ok; ++t) {
        if (t + 1 < ntb) {
          advance(cq);
          ok = issue_qk(t + 1, cq);
          if (!ok) break;
        }
        const int s = t % STAGES, sp = cp.seg & 1;
        const bool first = (t == 0 || cp.j == 0);
        if (!mbar_wait(&sh->p_full[t & 1], (t >> 1) & 1) || !mbar_wait(&sh->v_full[s], (t / STAGES) & 1)) { ok = false; break; }
        // this O^T buffer held the segment before the last one: it must have been read out
        if (first && cp.seg >= 2 && !mbar_wait(&sh->o_free[sp], ((cp.seg >> 1) - 1) & 1)) { ok = false; break; }
        TC_FENCE_AFTER();
        const uint64_t v_desc = desc_mn_major(smem_u32(v_s + s * TILE_BYTES));
        const uint64_t p_desc = desc_k_major(smem_u32(p_s + (t & 1) * SMALL_BYTES));
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)     // 16 keys further: 16 rows (2048 bytes) down V, 32 bytes along P^T's rows
          umma(tmem + 32 + sp * NH, v_desc + kk * (16 * 128 / 16), p_desc + (kk >> 2) * (SMALL_HALF >> 4) + 2 * (kk & 3), IDESC_PV,
               !(first && kk == 0));
        umma_commit(&sh->v_empty[s]);
        umma_commit(&sh->o_done[t & 1]);
        advance(cp);
      }
      if (!ok) { atomicOr(p.status, JV_STATUS_WAIT_EXPIRED); sh->failed = 1; }
    }
  } else {
    // ------------------------------------------------------------------ softmax: one key row per thread
    const int quad = warp & 3, sw = warp - 2;                    // TMEM lanes of this warp; index among the softmax warps
    const int row = quad * 32 + lane;                            // key row of the tile, and d for O^T
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    float l_part[GP];
    int seg_j0 = 0;                                              // first tile (of its pair) of the running segment
    Cursor c = c0;
    bool ok = true;
    for (int t = 0; t < ntb; ++t) {
      const bool first = (t == 0 || c.j == 0), last = (t == ntb - 1 || c.j == c.nt - 1);
      const int sp = c.seg & 1, pos = sh->pos[c.i];
      const uint32_t tmem_o = tmem + 32 + sp * NH + lane_addr;
      if (first) {
        seg_j0 = c.j;
#pragma unroll
        for (int h = 0; h < GP; ++h) l_part[h] = 0.f;
      }
      if (ok) ok = mbar_wait(&sh->s_full[t & 1], (t >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      float sc[GP];
      const int n_keys = FUSED ? pos : pos + 1;                  // keys of the pair that are in the cache
      const bool valid = c.j * BN + row < n_keys;                // only a pair's last tile has keys past the end
      bool exceeds = false;
      if (ok) {
        TC_FENCE_AFTER();
        tmem_ld<GP>(tmem + lane_addr + (t & 1) * NH, sc);
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          if (!valid || h >= G) sc[h] = -INFINITY;
          const float ref = first ? -INFINITY : sh->m_ref[h];
          exceeds |= sc[h] != -INFINITY && (ref == -INFINITY || (sc[h] - ref) * p.scale_log2 > LAZY);
        }
      }
      if (softmax_barrier_or(exceeds)) {      // the same answer in all 128 threads
        // ---- a segment's first tile, else rare: move the references to the tile's maxima, rescale O^T and the sums
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          float m = sc[h];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
          if (lane == 0) sh->red[sw][h] = m;
        }
        SOFTMAX_BARRIER();
        if (threadIdx.x - 64 < GP) {
          const int h = threadIdx.x - 64;
          const float m_tile = fmaxf(fmaxf(sh->red[0][h], sh->red[1][h]), fmaxf(sh->red[2][h], sh->red[3][h]));
          const float ref = first ? -INFINITY : sh->m_ref[h];
          const float m_new = fmaxf(ref, m_tile);
          sh->alpha[h] = (ref == -INFINITY || m_new == -INFINITY) ? 1.f : fast_exp2((ref - m_new) * p.scale_log2);
          sh->m_ref[h] = m_new;
        }
        SOFTMAX_BARRIER();
        if (!first) {
          if (ok) ok = mbar_wait(&sh->o_done[(t - 1) & 1], ((t - 1) >> 1) & 1);   // the last product must be complete
          ok = __all_sync(0xffffffffu, ok);
          if (ok) {
            TC_FENCE_AFTER();
            float o[GP];
            tmem_ld<GP>(tmem_o, o);
#pragma unroll
            for (int h = 0; h < GP; ++h) { o[h] *= sh->alpha[h]; l_part[h] *= sh->alpha[h]; }
            tmem_st<GP>(tmem_o, o);
          }
        }
      }
      // ---- this tile's P^T buffer was read by the product of tile t-2
      if (ok && t >= 2) ok = __all_sync(0xffffffffu, mbar_wait(&sh->o_done[t & 1], ((t - 2) >> 1) & 1));
      if (ok) {
        // ---- probabilities: P^T[head][key] as bfloat16 in the swizzled K-major tile (keys along the 128-byte rows)
        unsigned char* pt = p_s + (t & 1) * SMALL_BYTES + (row >> 6) * SMALL_HALF + (row & 7) * 2;
        const int chunk = (row & 63) >> 3;
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          if (h < G) {
            const float pr = (sc[h] == -INFINITY) ? 0.f : fast_exp2((sc[h] - sh->m_ref[h]) * p.scale_log2);
            l_part[h] += pr;
            *reinterpret_cast<__nv_bfloat16*>(pt + h * 128 + ((chunk ^ (h & 7)) << 4)) = __float2bfloat16_rn(pr);
          }
        }
        // ---- in a pair's last tile the value rows past the end become zero (they may hold anything)
        if (c.j == c.nt - 1 && n_keys < (c.j + 1) * BN) {
          const int s = t % STAGES;
          ok = __all_sync(0xffffffffu, mbar_wait(&sh->v_full[s], (t / STAGES) & 1));
          if (ok) {
            const int from = n_keys - c.j * BN;
            for (int i = (threadIdx.x - 64); i < (BN - from) * 16; i += 128) {
              const int key_row = from + i / 16, part = i % 16;
              *reinterpret_cast<uint4*>(v_s + s * TILE_BYTES + (part >> 3) * HALF_BYTES + key_row * 128 + (part & 7) * 16) =
                  make_uint4(0, 0, 0, 0);
            }
          }
        }
      }
      if (ok) {
        PROXY_FENCE();
        TC_FENCE_BEFORE();
        mbar_arrive(&sh->p_full[t & 1]);
      }
      if (last) {
        // ---- the segment ends: the sums of the key rows per head, then O^T (thread = d)
        float l_all[GP];
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          float v = l_part[h];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == 0) sh->red[sw][h] = v;
        }
        SOFTMAX_BARRIER();
#pragma unroll
        for (int h = 0; h < GP; ++h) l_all[h] = (sh->red[0][h] + sh->red[1][h]) + (sh->red[2][h] + sh->red[3][h]);
        const int pair = c.i * Hkv + c.head;
        const long long pair_g = (long long)sh->pre[c.i] * Hkv + (long long)c.head * c.nt;
        const int b_first = block_of(pair_g), b_last = block_of(pair_g + c.nt - 1);
        const int token = sh->token[c.i];
        if (ok) ok = mbar_wait(&sh->o_done[t & 1], (t >> 1) & 1);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
          TC_FENCE_AFTER();
          float o[GP], m_out[GP];
          tmem_ld<GP>(tmem_o, o);
#pragma unroll
          for (int h = 0; h < GP; ++h) m_out[h] = sh->m_ref[h];
          if constexpr (FUSED) {
            if (c.j == c.nt - 1) {
              // ---- the pair ends here: the new token, whose key and value are not in the cache yet, is one more
              // key, with its raw scores and its value left in shared memory by the query producer
              const bool had_keys = seg_j0 * BN < n_keys;            // else this segment is an empty last tile
              const float v = sh->v_new[sp][row];
#pragma unroll
              for (int h = 0; h < GP; ++h) {
                if (h < G) {
                  const float s_h = sh->s_new[sp][h];
                  const float ref = had_keys ? m_out[h] : -INFINITY;
                  const float m_fin = fmaxf(ref, s_h);
                  const float keep = (ref == -INFINITY) ? 0.f : fast_exp2((ref - m_fin) * p.scale_log2);
                  const float p_new = fast_exp2((s_h - m_fin) * p.scale_log2);
                  o[h] = o[h] * keep + p_new * v;
                  l_all[h] = l_all[h] * keep + p_new;
                  m_out[h] = m_fin;
                }
              }
            }
          }
          TC_FENCE_BEFORE();
          mbar_arrive(&sh->o_free[sp]);            // (after the reads above: the next but one segment may overwrite them)
          if (b_first == b_last) {              // the whole pair was this block's: normalise and write it
#pragma unroll
            for (int h = 0; h < GP; ++h)
              if (h < G)
                p.out[(size_t)token * p.out_stride + (size_t)(c.head * G + h) * D + row] = __float2bfloat16_rn(o[h] / l_all[h]);
          } else {                              // unnormalised, with (reference in exponent units, sum)
            const size_t slot = (size_t)(pair + (int)blockIdx.x) * G;
#pragma unroll
            for (int h = 0; h < GP; ++h) {
              if (h < G) {
                p.part_o[(slot + h) * D + row] = o[h];
                if (row == 0) {
                  p.part_ml[(slot + h) * 2] = m_out[h] * p.scale_log2;
                  p.part_ml[(slot + h) * 2 + 1] = l_all[h];
                }
              }
            }
          }
        } else if (lane == 0) {
          atomicOr(p.status, JV_STATUS_WAIT_EXPIRED);
          sh->failed = 1;
        }
        if (b_first != b_last) {                // the same in all 128 threads
          // ---- the block that finishes the pair last merges its segments in ascending order of the blocks
          __threadfence();
          SOFTMAX_BARRIER();
          if (threadIdx.x == 64) {
            const int done = atomicAdd(p.counters + pair, 1) + 1;
            sh->is_last = (done == b_last - b_first + 1);
            if (sh->is_last) p.counters[pair] = 0;          // ready for the next launch
          }
          SOFTMAX_BARRIER();
          if (sh->is_last) {
            __threadfence();
            // a thread takes four d of one head; the loads of eight segments are in flight together, and the
            // segments are added in ascending order of the blocks
            for (int w = threadIdx.x - 64; w < G * (D / 4); w += 128) {
              const int h = w / (D / 4), d4 = (w % (D / 4)) * 4;
              float m_run = -INFINITY, l_run = 0.f;
              float4 o_run = make_float4(0.f, 0.f, 0.f, 0.f);
              for (int b0 = b_first; b0 <= b_last; b0 += 8) {
                float2 ml[8];
                float4 oo[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                  ml[u] = make_float2(-INFINITY, 0.f);
                  oo[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                  if (b0 + u <= b_last) {
                    const size_t slot = (size_t)(pair + b0 + u) * G + h;
                    ml[u] = __ldcg(reinterpret_cast<const float2*>(p.part_ml + slot * 2));
                    oo[u] = __ldcg(reinterpret_cast<const float4*>(p.part_o + slot * D + d4));
                  }
                }
                float m_new = m_run;
#pragma unroll
                for (int u = 0; u < 8; ++u) m_new = fmaxf(m_new, ml[u].x);
                const float keep = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
                l_run *= keep; o_run.x *= keep; o_run.y *= keep; o_run.z *= keep; o_run.w *= keep;
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                  const float f = (ml[u].x == -INFINITY) ? 0.f : exp2f(ml[u].x - m_new);
                  l_run += f * ml[u].y;
                  o_run.x += f * oo[u].x; o_run.y += f * oo[u].y; o_run.z += f * oo[u].z; o_run.w += f * oo[u].w;
                }
                m_run = m_new;
              }
              const float inv = 1.f / l_run;
              __nv_bfloat162 lo = __floats2bfloat162_rn(o_run.x * inv, o_run.y * inv), hi = __floats2bfloat162_rn(o_run.z * inv, o_run.w * inv);
              uint2 packed;
              packed.x = *reinterpret_cast<uint32_t*>(&lo); packed.y = *reinterpret_cast<uint32_t*>(&hi);
              *reinterpret_cast<uint2*>(p.out + (size_t)token * p.out_stride + (size_t)(c.head * G + h) * D + d4) = packed;
            }
          }
        }
      }
      advance(c);
    }
  }

  // ---- tear-down
  TC_FENCE_BEFORE();
  __syncthreads();
  if (sh->failed) {
    // a wait ran out: products already issued may still write tensor memory and copies already asked for still land
    // in this block's shared memory; both get a bounded time to finish before tensor memory is freed and the block ends
    if (warp == 1 && lane == 0) drain_products_after_failure(&sh->drain);
    if ((warp == 0 || warp == 6) && lane == 0) {
      const int which = warp == 6;
      for (int s = 0; s < STAGES; ++s)
        if (sh->armed[which][s] >= 0) drain_copies_after_failure(which ? &sh->v_full[s] : &sh->k_full[s], sh->armed[which][s]);
    }
    if (warp == 7 && lane == 0)
      for (int b = 0; b < 2; ++b)
        if (sh->armed_q[b] >= 0) drain_copies_after_failure(&sh->q_full[b], sh->armed_q[b]);
    __syncthreads();
  }
  if (warp == 1) {
    TC_FENCE_AFTER();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
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

constexpr size_t SMEM_BYTES = 2 * STAGES * TILE_BYTES + 4 * SMALL_BYTES + sizeof(Shared) + 1024;

template <int GP, bool FUSED>
int launch(int n_blocks, cudaStream_t stream, const CUtensorMap& q_map, const CUtensorMap& k_map, const CUtensorMap& v_map,
           const Params& p) {
  static bool ready[JV_MAX_DEVICES];
  if (!jv_once_per_device(ready, [&] {
        return cudaFuncSetAttribute(attn_decode_tcgen05_kernel<GP, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)SMEM_BYTES) == cudaSuccess;
      }))
    return JV_ERR_UNSUPPORTED;
  return jv_launch(attn_decode_tcgen05_kernel<GP, FUSED>, dim3(n_blocks), dim3(THREADS), SMEM_BYTES, stream, q_map, k_map, v_map,
                   p);
}
}  // namespace

// 1 if this kernel takes the case (else the caller uses the mma.sync kernel).
JV_EXPORT int jv_attn_decode_tcgen05_supports(int head_dim, int n_q_heads, int n_kv_heads, int page_size, int window,
                                              int n_work) {
  if (head_dim != 128 || window > 0 || n_kv_heads < 1 || n_q_heads % n_kv_heads) return 0;
  if (n_q_heads / n_kv_heads > NH || n_work > MAX_WORK) return 0;
  return page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128;
}

// Floats of scratch that a launch of n_blocks blocks needs for n_work single tokens: [0] for part_o, [1] for part_ml.
JV_EXPORT void jv_attn_decode_tcgen05_scratch(int n_work, int n_q_heads, int n_kv_heads, int n_blocks, long long* floats) {
  const long long slots = (long long)n_work * n_kv_heads + n_blocks;
  floats[0] = slots * (n_q_heads / n_kv_heads) * D;
  floats[1] = slots * (n_q_heads / n_kv_heads) * 2;
}

// Single tokens only: work item i is the token cu_seqlens[work[2i]] of request work[2i], at position start_pos[.].
// q [n_tokens, q_stride]; part_o and part_ml: scratch of the sizes that jv_attn_decode_tcgen05_scratch gives;
// counters [n_work * n_kv_heads], zero before the first launch (a launch leaves them zero); n_blocks: the
// size of the grid, best the number of multiprocessors.
//
// fused != 0: `q` is the product q|k|v as it comes ([n_tokens, q_stride]: query heads, key heads, value heads);
// the kernel applies the per-head norm (weights q_norm_w, k_norm_w of head_dim elements, float if norm_w_f32
// else bfloat16; null: no norm) and the rotation (inv_freq [head_dim/2] float; null: none) at position
// start_pos[.], and writes the new token's key and value into the caches itself.
JV_EXPORT int jv_attn_decode_tcgen05(const void* q, int q_stride, int n_tokens, void* out, int out_stride, float* part_o,
                                     float* part_ml, int* counters, void* k_cache, void* v_cache,
                                     const int* block_table, int table_width, const int* cu_seqlens, const int* start_pos,
                                     const int* work, int n_work, int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                                     int num_pages, float scale, int n_blocks, int fused, const float* inv_freq,
                                     const void* q_norm_w, const void* k_norm_w, int norm_w_f32, float eps, int* status,
                                     cudaStream_t stream) {
  if (n_work == 0) return JV_OK;
  if (!jv_attn_decode_tcgen05_supports(head_dim, n_q_heads, n_kv_heads, page_size, 0, n_work) || n_blocks < 1)
    return JV_ERR_UNSUPPORTED;
  if ((q_stride % 8) || ((uintptr_t)q % 16) || ((uintptr_t)k_cache % 16) || ((uintptr_t)v_cache % 16)) return JV_ERR_UNSUPPORTED;
  if ((out_stride % 4) || ((uintptr_t)out % 8)) return JV_ERR_UNSUPPORTED;
  auto fn = encode_fn();
  if (fn == nullptr) return JV_ERR_UNSUPPORTED;
  const int G = n_q_heads / n_kv_heads;
  CUtensorMap q_map, k_map, v_map;
  {
    // query: (d, head, token); a box is 64 d x G heads x 1 token
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)n_q_heads, (cuuint64_t)n_tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)q_stride * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)G, 1};
    const cuuint32_t es[3] = {1, 1, 1};
    if (fn(&q_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, es,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return JV_ERR_UNSUPPORTED;
  }
  for (int which = 0; which < 2; ++which) {
    const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)n_kv_heads, (cuuint64_t)page_size, (cuuint64_t)num_pages};
    const cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)n_kv_heads * D * 2, (cuuint64_t)page_size * n_kv_heads * D * 2};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)page_size, 1};
    const cuuint32_t es[4] = {1, 1, 1, 1};
    if (fn(which ? &v_map : &k_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, (which ? v_cache : k_cache), dims,
           strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return JV_ERR_UNSUPPORTED;
  }
  Params p;
  p.out = (__nv_bfloat16*)out; p.out_stride = out_stride; p.part_o = part_o; p.part_ml = part_ml; p.counters = counters;
  p.block_table = block_table; p.table_width = table_width; p.cu_seqlens = cu_seqlens; p.start_pos = start_pos; p.work = work;
  p.n_work = n_work; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size; p.num_pages = num_pages;
  p.scale_log2 = scale * LOG2E; p.status = status;
  p.qkv = (const __nv_bfloat16*)q; p.qkv_stride = q_stride; p.inv_freq = inv_freq; p.q_norm_w = q_norm_w; p.k_norm_w = k_norm_w;
  p.norm_w_f32 = norm_w_f32; p.eps = eps; p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache;
  if (fused) {
    if (q_stride < (n_q_heads + 2 * n_kv_heads) * D) return JV_ERR_UNSUPPORTED;
    if (G <= 4) return launch<4, true>(n_blocks, stream, q_map, k_map, v_map, p);
    if (G <= 8) return launch<8, true>(n_blocks, stream, q_map, k_map, v_map, p);
    return launch<16, true>(n_blocks, stream, q_map, k_map, v_map, p);
  }
  if (G <= 4) return launch<4, false>(n_blocks, stream, q_map, k_map, v_map, p);
  if (G <= 8) return launch<8, false>(n_blocks, stream, q_map, k_map, v_map, p);
  return launch<16, false>(n_blocks, stream, q_map, k_map, v_map, p);
}
