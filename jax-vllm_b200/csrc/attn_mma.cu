// Paged causal attention for bfloat16 on the tensor cores (mma.sync m16n8k16, 32-bit
// accumulation), keys and values streamed from the pages by bulk copies (one per cache row, completion
// counted on mbarriers; every wait is bounded and reports to the status word).  Two kernels share
// the tile code:
//
//   attn_prefill_mma  prompt portions.  A tile is 64 rows = (token, query head) pairs of ONE
//       kv head (row r -> token r / HPT, head r % HPT), so a key/value tile is loaded once
//       for all query heads of the group; 4 warps own 16 rows each; 64-key tiles are double
//       buffered.
//   attn_decode_mma   single decoded tokens, split along the keys.  A block takes one split
//       (split_size key positions, by absolute position) of one request and kv head; its 16
//       rows are the query heads of the group; the 4 warps take 16 keys each of every 64-key
//       tile (3 tiles in flight) and are merged in shared memory; the block that finishes last
//       among the splits of a row merges them, in ascending order.
//
// Scores are scaled and masked in 32-bit (key j visible to position p iff j <= p and
// (window == 0 or j > p - window)); the running softmax keeps (max, sum) in 32-bit;
// probabilities are rounded to bfloat16 for the second product.  Head sizes 16..128 in the
// instantiated steps; other sizes are refused (the caller falls back to the CUDA-core kernel).
#include "common.cuh"
#include "mbarrier.cuh"
#include <math.h>

namespace {

constexpr int BN = 64;         // keys per tile
constexpr int NWARPS = 4;
constexpr int THREADS = NWARPS * 32;
constexpr int ROWS_PREFILL = 16 * NWARPS;
constexpr int DECODE_STAGES = 3;
constexpr float LOG2E = 1.4426950408889634f;

struct Params {
  const __nv_bfloat16* q; int q_stride;
  __nv_bfloat16* out; int out_stride;
  float* part_o; float* part_ml;
  const __nv_bfloat16* k_cache; const __nv_bfloat16* v_cache;
  const int* block_table; int table_width;
  const int* cu_seqlens; const int* start_pos;
  const int* work;
  int n_q_heads, n_kv_heads, page_size, num_pages, window;
  float scale_log2;            // softmax scale * log2(e)
  int tokens_per_tile, heads_per_tile, n_head_groups, split_size, n_splits;
  int* status;
  int* counters;               // decode: one per (work item, kv head, head group), zero between launches
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // 0 bytes read: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Rows of a shared-memory tile are D elements plus 8 of padding: the row stride in 4-byte words
// is then 4 modulo 8, so the eight 16-byte rows that one ldmatrix phase reads fall into distinct banks.
template <int D> struct Tile { static constexpr int STRIDE = D + 8; };

// Element offsets of the cache rows of keys [j0, j0 + BN) of one kv head (-1: beyond j_end, or no
// page), one per thread n < BN: the block table is read once per key, ahead of the copies.
template <int D>
__device__ __forceinline__ void tile_rows(long long* rows, const Params& p, int entry, int kv_head, int j0, int j_end,
                                          int tid) {
  if (tid < BN) {
    const int j = j0 + tid;
    long long off = -1;
    if (j < j_end) {
      const int pi = j / p.page_size;
      const int page = pi < p.table_width ? p.block_table[(size_t)entry * p.table_width + pi] : -1;
      if (page < 0 || page >= p.num_pages) atomicOr(p.status, JV_STATUS_BAD_PAGE);
      else off = (((long long)page * p.page_size + (j - pi * p.page_size)) * p.n_kv_heads + kv_head) * D;
    }
    rows[tid] = off;
  }
}

// ---- mbarrier + bulk-copy (TMA) helpers.  A cache row of one kv head is D contiguous elements, so a
// 64-key tile is 64 + 64 bulk copies, one per thread, instead of 16-byte copies by the thousand; their
// completion is counted in bytes on the stage's mbarrier.
__device__ __forceinline__ void bulk_copy(void* dst, const void* src, int bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Copies the rows listed by tile_rows into a K tile and a V tile: thread n < 64 the key row n, thread
// 64 + n the value row n (a row without a source is zeroed by the thread).  Every thread arrives once
// on `bar`, which completes when all bytes have landed.
template <int D>
__device__ __forceinline__ void issue_tile(__nv_bfloat16* ks, __nv_bfloat16* vs, const long long* rows, const Params& p,
                                           uint64_t* bar, int tid) {
  static_assert(THREADS == 2 * BN, "one thread per key row and per value row");
  constexpr int S = Tile<D>::STRIDE;
  const int n = tid & (BN - 1);
  const bool is_v = tid >= BN;
  const long long off = rows[n];
  __nv_bfloat16* dst = (is_v ? vs : ks) + n * S;
  if (off >= 0) {
    mbar_expect_tx(bar, D * 2);
    bulk_copy(dst, (is_v ? p.v_cache : p.k_cache) + off, D * 2, bar);
  } else {
#pragma unroll
    for (int c = 0; c < D / 8; ++c) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0, 0, 0, 0);
    mbar_arrive(bar);
  }
}

// Waits for a tile; on a timeout records it in the status word (the caller then leaves).
__device__ __forceinline__ bool wait_tile(uint64_t* bar, int parity, const Params& p) {
  if (mbar_wait(bar, parity)) return true;
  atomicOr(p.status, JV_STATUS_WAIT_EXPIRED);
  return false;
}

// S[16 rows, NB*8 keys] += Q[16, D] K[keys, D]^T for one warp.  `qs` points at the warp's first
// row, `ks` at the first key row.
template <int D, int NB>
__device__ __forceinline__ void qk_tile(float (&s)[NB][4], const __nv_bfloat16* qs, const __nv_bfloat16* ks, int lane) {
  constexpr int S = Tile<D>::STRIDE;
  const int mat = lane >> 3, r = lane & 7;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a[4];
    ldmatrix_x4(a, qs + ((mat & 1) * 8 + r) * S + kk * 16 + (mat >> 1) * 8);
#pragma unroll
    for (int nb2 = 0; nb2 < NB / 2; ++nb2) {
      uint32_t b[4];
      ldmatrix_x4(b, ks + (nb2 * 16 + (mat >> 1) * 8 + r) * S + kk * 16 + (mat & 1) * 8);
      mma_bf16(s[2 * nb2], a, b[0], b[1]);
      mma_bf16(s[2 * nb2 + 1], a, b[2], b[3]);
    }
  }
}

// O[16, D] += P[16, NB*8 keys] V[keys, D] for one warp; P comes from the score registers.
template <int D, int NB>
__device__ __forceinline__ void pv_tile(float (&o)[D / 8][4], const float (&pr)[NB][4], const __nv_bfloat16* vs, int lane) {
  constexpr int S = Tile<D>::STRIDE;
  const int mat = lane >> 3, r = lane & 7;
#pragma unroll
  for (int kk = 0; kk < NB / 2; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(pr[2 * kk][0], pr[2 * kk][1]);
    a[1] = pack_bf16(pr[2 * kk][2], pr[2 * kk][3]);
    a[2] = pack_bf16(pr[2 * kk + 1][0], pr[2 * kk + 1][1]);
    a[3] = pack_bf16(pr[2 * kk + 1][2], pr[2 * kk + 1][3]);
#pragma unroll
    for (int db2 = 0; db2 < D / 16; ++db2) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, vs + (kk * 16 + (mat & 1) * 8 + r) * S + db2 * 16 + (mat >> 1) * 8);
      mma_bf16(o[2 * db2], a, b[0], b[1]);
      mma_bf16(o[2 * db2 + 1], a, b[2], b[3]);
    }
  }
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// Exponentiates one warp's scores of a tile and updates the running (max, sum) of its two rows per
// thread; rescales the output accumulators.  The running maximum m is kept in units of the raw
// score; exp2(s*c - m*c) with c = scale * log2(e) is one multiply-add and one ex2.  With MASK the
// visibility test is applied first (key0 + nb*8 + (lane%4)*2 + (i&1) is the key of s[nb][i]; pos0/pos1
// are the positions of rows lane/4 and lane/4 + 8, -1 for an unused row); tiles that lie wholly
// inside every row's visible range are handled without it.
template <int D, int NB, bool MASK>
__device__ __forceinline__ void softmax_tile(float (&s)[NB][4], float (&o)[D / 8][4], float (&m)[2], float (&l)[2],
                                             int pos0, int pos1, int key0, int j_end, int window,
                                             float scale_log2, int lane) {
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (MASK) {
        const int key = key0 + nb * 8 + (lane & 3) * 2 + (i & 1);
        const int pos = (i < 2) ? pos0 : pos1;
        const bool vis = key < j_end && key <= pos && (window <= 0 || key > pos - window);
        if (!vis) s[nb][i] = -INFINITY;
      }
      mx[i >> 1] = fmaxf(mx[i >> 1], s[nb][i]);
    }
  float alpha[2], m_scaled[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    const float m_new = fmaxf(m[h], mx[h]);
    alpha[h] = (m[h] == -INFINITY) ? 0.f : fast_exp2((m[h] - m_new) * scale_log2);  // m_new == -inf only if m[h] is
    m_scaled[h] = (m_new == -INFINITY) ? 0.f : m_new * scale_log2;                   // then every score is -inf: p = 0
    m[h] = m_new;
  }
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float pr = fast_exp2(fmaf(s[nb][i], scale_log2, -m_scaled[i >> 1]));
      s[nb][i] = pr;
      sum[i >> 1] += pr;
    }
#pragma unroll
  for (int h = 0; h < 2; ++h) l[h] = l[h] * alpha[h] + sum[h];   // per-thread part; lanes are summed at the end
  if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
    for (int db = 0; db < D / 8; ++db) {
      o[db][0] *= alpha[0]; o[db][1] *= alpha[0];
      o[db][2] *= alpha[1]; o[db][3] *= alpha[1];
    }
  }
}

// ------------------------------------------------------------------------- prefill
template <int D>
__global__ void __launch_bounds__(THREADS) attn_prefill_mma_kernel(const Params p) {
  constexpr int S = Tile<D>::STRIDE;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);    // [64][S]
  __nv_bfloat16* ks = qs + ROWS_PREFILL * S;                          // [2][BN][S]
  __nv_bfloat16* vs = ks + 2 * BN * S;                                // [2][BN][S]
  __shared__ long long rows[2][BN];
  __shared__ __align__(8) uint64_t bars[2];
  pdl_trigger();
  if (threadIdx.x == 0) {
    mbar_init(&bars[0], THREADS);
    mbar_init(&bars[1], THREADS);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  pdl_wait();

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int entry = p.work[2 * blockIdx.x], q_off = p.work[2 * blockIdx.x + 1];
  const int kv_head = blockIdx.y / p.n_head_groups, hg = blockIdx.y % p.n_head_groups;
  const int G = p.n_q_heads / p.n_kv_heads;
  const int HPT = p.heads_per_tile;
  const int q_begin = p.cu_seqlens[entry];
  const int q_len = p.cu_seqlens[entry + 1] - q_begin;
  const int ctx = p.start_pos[entry];
  const int tokens_here = min(p.tokens_per_tile, q_len - q_off);
  if (tokens_here <= 0) return;
  const int pos_first = ctx + q_off;
  const int j_lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
  const int j_hi = pos_first + tokens_here;   // exclusive

  // ---- queries of the tile (unused rows zero)
  constexpr int CH = D / 8;
  for (int c = tid; c < ROWS_PREFILL * CH; c += THREADS) {
    const int r = c / CH, part = c - r * CH;
    const int t = r / HPT, hh = hg * HPT + r % HPT;
    const bool valid = t < tokens_here && hh < G;
    const size_t off = valid ? (size_t)(q_begin + q_off + t) * p.q_stride + (size_t)(kv_head * G + hh) * D + part * 8 : 0;
    cp_async16(qs + r * S + part * 8, p.q + off, valid);
  }
  const int n_tiles = (j_hi - j_lo + BN - 1) / BN;
  tile_rows<D>(rows[0], p, entry, kv_head, j_lo, j_hi, tid);
  tile_rows<D>(rows[1], p, entry, kv_head, j_lo + BN, j_hi, tid);
  cp_async_commit();                      // the queries
  __syncthreads();
  issue_tile<D>(ks, vs, rows[0], p, &bars[0], tid);
  __syncthreads();                        // rows[0] has been read by all before iteration 0 refills it

  // ---- this thread's two rows
  int pos[2];
  {
    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
    const int t0 = r0 / HPT, h0 = hg * HPT + r0 % HPT, t1 = r1 / HPT, h1 = hg * HPT + r1 % HPT;
    pos[0] = (t0 < tokens_here && h0 < G) ? pos_first + t0 : -1;
    pos[1] = (t1 < tokens_here && h1 < G) ? pos_first + t1 : -1;
  }
  // the last position any row of this warp has (its tiles beyond that are skipped)
  int warp_last = max(pos[0], pos[1]);
  int warp_first = min(pos[0] < 0 ? 0x7fffffff : pos[0], pos[1] < 0 ? 0x7fffffff : pos[1]);   // over rows in use
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    warp_last = max(warp_last, __shfl_xor_sync(0xffffffffu, warp_last, o));
    warp_first = min(warp_first, __shfl_xor_sync(0xffffffffu, warp_first, o));
  }

  float o_acc[D / 8][4];
#pragma unroll
  for (int db = 0; db < D / 8; ++db)
#pragma unroll
    for (int i = 0; i < 4; ++i) o_acc[db][i] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < n_tiles)
      issue_tile<D>(ks + (buf ^ 1) * BN * S, vs + (buf ^ 1) * BN * S, rows[buf ^ 1], p, &bars[buf ^ 1], tid);
    // rows of tile t+2 go where those of tile t were (read when tile t was issued, an iteration ago)
    if (t + 2 < n_tiles) tile_rows<D>(rows[buf], p, entry, kv_head, j_lo + (t + 2) * BN, j_hi, tid);
    if (t == 0) cp_async_wait<0>();
    // every thread takes the same way out: all saw the tile, or the block stops (status word set)
    if (!__syncthreads_and(wait_tile(&bars[buf], (t >> 1) & 1, p))) {
      wait_tile(&bars[buf], (t >> 1) & 1, p);   // once more, bounded, for copies that may still be landing
      return;
    }
    const int key0 = j_lo + t * BN;
    if (key0 <= warp_last) {
      float s[BN / 8][4];
#pragma unroll
      for (int nb = 0; nb < BN / 8; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[nb][i] = 0.f;
      qk_tile<D, BN / 8>(s, qs + warp * 16 * S, ks + buf * BN * S, lane);
      // the test is needed only where the tile reaches past the first row's position, past the end,
      // or a window cuts into it
      if (key0 + BN - 1 > warp_first || key0 + BN > j_hi || p.window > 0)
        softmax_tile<D, BN / 8, true>(s, o_acc, m, l, pos[0], pos[1], key0, j_hi, p.window, p.scale_log2, lane);
      else
        softmax_tile<D, BN / 8, false>(s, o_acc, m, l, pos[0], pos[1], key0, j_hi, p.window, p.scale_log2, lane);
      pv_tile<D, BN / 8>(o_acc, s, vs + buf * BN * S, lane);
    }
    __syncthreads();
  }

  // ---- normalise and write
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (pos[h] < 0) continue;
    const int r = warp * 16 + (lane >> 2) + h * 8;
    const int t = r / HPT, hh = hg * HPT + r % HPT;
    __nv_bfloat16* dst = p.out + (size_t)(q_begin + q_off + t) * p.out_stride + (size_t)(kv_head * G + hh) * D;
    const float inv = 1.f / l[h];
#pragma unroll
    for (int db = 0; db < D / 8; ++db) {
      const int d = db * 8 + (lane & 3) * 2;
      *reinterpret_cast<uint32_t*>(dst + d) = pack_bf16(o_acc[db][2 * h] * inv, o_acc[db][2 * h + 1] * inv);
    }
  }
}

// -------------------------------------------------------------------------- decode
template <int D>
__global__ void __launch_bounds__(THREADS) attn_decode_mma_kernel(const Params p) {
  constexpr int S = Tile<D>::STRIDE;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);    // [16][S]
  __nv_bfloat16* ks = qs + 16 * S;                                    // [STAGES][BN][S]
  __nv_bfloat16* vs = ks + DECODE_STAGES * BN * S;                    // [STAGES][BN][S]
  __shared__ long long rows[DECODE_STAGES][BN];
  __shared__ int is_last;
  __shared__ __align__(8) uint64_t bars[DECODE_STAGES];
  pdl_trigger();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int st = 0; st < DECODE_STAGES; ++st) mbar_init(&bars[st], THREADS);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  pdl_wait();

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int entry = p.work[2 * blockIdx.x];
  const int kv_head = blockIdx.y / p.n_head_groups, hg = blockIdx.y % p.n_head_groups;
  const int G = p.n_q_heads / p.n_kv_heads;
  const int HPT = p.heads_per_tile;
  const int pos_q = p.start_pos[entry];
  const int vis_lo = p.window > 0 ? max(0, pos_q - p.window + 1) : 0;   // visible keys: [vis_lo, pos_q]
  const int j_lo = max(vis_lo, (int)blockIdx.z * p.split_size);
  const int j_hi = min(pos_q + 1, ((int)blockIdx.z + 1) * p.split_size);
  if (j_lo >= j_hi) return;
  const int token = p.cu_seqlens[entry];

  constexpr int CH = D / 8;
  for (int c = tid; c < 16 * CH; c += THREADS) {
    const int r = c / CH, part = c - r * CH;
    const int hh = hg * HPT + r;
    const bool valid = r < HPT && hh < G;
    const size_t off = valid ? (size_t)token * p.q_stride + (size_t)(kv_head * G + hh) * D + part * 8 : 0;
    cp_async16(qs + r * S + part * 8, p.q + off, valid);
  }
  const int n_tiles = (j_hi - j_lo + BN - 1) / BN;
#pragma unroll
  for (int st = 0; st < DECODE_STAGES; ++st) tile_rows<D>(rows[st], p, entry, kv_head, j_lo + st * BN, j_hi, tid);
  cp_async_commit();                      // the queries
  __syncthreads();
#pragma unroll
  for (int st = 0; st < DECODE_STAGES - 1; ++st)
    if (st < n_tiles) issue_tile<D>(ks + st * BN * S, vs + st * BN * S, rows[st], p, &bars[st], tid);
  __syncthreads();                        // rows[0] has been read by all before iteration 0 refills it

  // every row is the same token: position pos_q for rows that hold a head, -1 otherwise
  int pos[2];
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
    pos[0] = (r0 < HPT && hg * HPT + r0 < G) ? pos_q : -1;
    pos[1] = (r1 < HPT && hg * HPT + r1 < G) ? pos_q : -1;
  }
  float o_acc[D / 8][4];
#pragma unroll
  for (int db = 0; db < D / 8; ++db)
#pragma unroll
    for (int i = 0; i < 4; ++i) o_acc[db][i] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  for (int t = 0; t < n_tiles; ++t) {
    const int nxt = t + DECODE_STAGES - 1;
    if (nxt < n_tiles) {
      const int nb = nxt % DECODE_STAGES;
      issue_tile<D>(ks + nb * BN * S, vs + nb * BN * S, rows[nb], p, &bars[nb], tid);
    }
    // rows of tile t+STAGES go where those of tile t were (read when tile t was issued)
    if (t + DECODE_STAGES < n_tiles)
      tile_rows<D>(rows[t % DECODE_STAGES], p, entry, kv_head, j_lo + (t + DECODE_STAGES) * BN, j_hi, tid);
    if (t == 0) cp_async_wait<0>();
    if (!__syncthreads_and(wait_tile(&bars[t % DECODE_STAGES], (t / DECODE_STAGES) & 1, p))) {
      wait_tile(&bars[t % DECODE_STAGES], (t / DECODE_STAGES) & 1, p);
      return;
    }
    const int buf = t % DECODE_STAGES;
    const int key0 = j_lo + t * BN + warp * 16;      // this warp's 16 keys of the tile
    if (key0 < j_hi) {
      float s[2][4];
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[nb][i] = 0.f;
      qk_tile<D, 2>(s, qs, ks + (buf * BN + warp * 16) * S, lane);
      // keys before j_lo are never loaded, so only the tile that reaches past j_hi needs the test
      if (key0 + 16 > j_hi)
        softmax_tile<D, 2, true>(s, o_acc, m, l, pos[0], pos[1], key0, j_hi, 0, p.scale_log2, lane);
      else
        softmax_tile<D, 2, false>(s, o_acc, m, l, pos[0], pos[1], key0, j_hi, 0, p.scale_log2, lane);
      pv_tile<D, 2>(o_acc, s, vs + (buf * BN + warp * 16) * S, lane);
    }
    __syncthreads();
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    m[h] *= p.scale_log2;   // from here on the maxima are exponents of two (warps and splits are merged with exp2)
  }

  // ---- merge the four warps (each saw a quarter of the keys) through shared memory
  float* mo = reinterpret_cast<float*>(ks);            // [NWARPS][16][D]  (the tiles are done with)
  float* mm = mo + NWARPS * 16 * D;                    // [NWARPS][16]
  float* ml = mm + NWARPS * 16;                        // [NWARPS][16]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = (lane >> 2) + h * 8;
    if (r >= HPT) continue;               // rows without a head are not merged
    if ((lane & 3) == 0) { mm[warp * 16 + r] = m[h]; ml[warp * 16 + r] = l[h]; }
#pragma unroll
    for (int db = 0; db < D / 8; ++db) {
      const int d = db * 8 + (lane & 3) * 2;
      mo[(warp * 16 + r) * D + d] = o_acc[db][2 * h];
      mo[(warp * 16 + r) * D + d + 1] = o_acc[db][2 * h + 1];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < HPT * D; idx += THREADS) {
    const int r = idx / D, d = idx - r * D;
    const int hh = hg * HPT + r;
    if (hh >= G) continue;
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) m_all = fmaxf(m_all, mm[w * 16 + r]);
    float o = 0.f, lsum = 0.f;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
      const float mw = mm[w * 16 + r];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - m_all);
      o += f * mo[(w * 16 + r) * D + d];
      lsum += f * ml[w * 16 + r];
    }
    const size_t slot = ((size_t)blockIdx.x * p.n_q_heads + (kv_head * G + hh)) * p.n_splits + blockIdx.z;
    p.part_o[slot * D + d] = o;
    if (d == 0) { p.part_ml[slot * 2] = m_all; p.part_ml[slot * 2 + 1] = lsum; }
  }

  // ---- the block that finishes last among the splits of this (token, kv head, head group) merges them,
  //      in ascending order of the splits whichever block that is.  Nobody waits: a block adds one to the
  //      counter when its partial result is written and leaves unless it brought the count to the total.
  const int s_first = vis_lo / p.split_size;
  int s_last = pos_q / p.split_size;
  if (s_last >= p.n_splits) {           // the launch has too few splits for this length
    if (tid == 0) atomicOr(p.status, JV_STATUS_BAD_ROW);
    s_last = p.n_splits - 1;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int* counter = p.counters + (size_t)blockIdx.x * gridDim.y + blockIdx.y;
    const int done = atomicAdd(counter, 1) + 1;
    is_last = (done == s_last - s_first + 1);
    if (is_last) *counter = 0;          // ready for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int idx = tid; idx < HPT * D; idx += THREADS) {
    const int r = idx / D, d = idx - r * D;
    const int hh = hg * HPT + r;
    if (hh >= G) continue;
    const int head = kv_head * G + hh;
    const size_t base = ((size_t)blockIdx.x * p.n_q_heads + head) * p.n_splits;
    float m_all = -INFINITY;
    for (int sp = s_first; sp <= s_last; ++sp) m_all = fmaxf(m_all, __ldcg(p.part_ml + (base + sp) * 2));
    float o = 0.f, l_all = 0.f;
    for (int sp = s_first; sp <= s_last; ++sp) {
      const float f = exp2f(__ldcg(p.part_ml + (base + sp) * 2) - m_all);
      l_all += f * __ldcg(p.part_ml + (base + sp) * 2 + 1);
      o += f * __ldcg(p.part_o + (base + sp) * D + d);
    }
    p.out[(size_t)token * p.out_stride + (size_t)head * D + d] = __float2bfloat16_rn(o / l_all);
  }
}

template <int D> size_t prefill_smem() { return sizeof(__nv_bfloat16) * (size_t)(ROWS_PREFILL + 4 * BN) * Tile<D>::STRIDE; }
template <int D> size_t decode_smem() {
  const size_t tiles = sizeof(__nv_bfloat16) * (size_t)(16 + 2 * DECODE_STAGES * BN) * Tile<D>::STRIDE;
  const size_t merge = sizeof(__nv_bfloat16) * 16 * Tile<D>::STRIDE + sizeof(float) * (NWARPS * 16 * D + 2 * NWARPS * 16);
  return tiles > merge ? tiles : merge;
}

template <int D>
int launch(const Params& p, int n_work, bool split, cudaStream_t stream) {
  if (!split) {
    static bool ready[JV_MAX_DEVICES];
    const size_t smem = prefill_smem<D>();
    if (!jv_once_per_device(ready, [&] {
          return cudaFuncSetAttribute(attn_prefill_mma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
        }))
      return JV_ERR_UNSUPPORTED;
    dim3 grid(n_work, p.n_kv_heads * p.n_head_groups);
    return jv_launch(attn_prefill_mma_kernel<D>, grid, dim3(THREADS), smem, stream, p);
  }
  static bool ready[JV_MAX_DEVICES];
  const size_t smem = decode_smem<D>();
  if (!jv_once_per_device(ready, [&] {
        return cudaFuncSetAttribute(attn_decode_mma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
      }))
    return JV_ERR_UNSUPPORTED;
  dim3 grid(n_work, p.n_kv_heads * p.n_head_groups, p.n_splits);
  return jv_launch(attn_decode_mma_kernel<D>, grid, dim3(THREADS), smem, stream, p);
}
}  // namespace

// 1 if the tensor-core kernels are instantiated for this head size.
JV_EXPORT int jv_attn_mma_supports(int head_dim) {
  return head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128;
}

// Tokens in a prefill tile: 64 rows / heads per tile, heads per tile = min(G, 16).
JV_EXPORT int jv_attn_mma_tokens_per_tile(int n_q_heads, int n_kv_heads) {
  const int G = n_q_heads / n_kv_heads;
  return ROWS_PREFILL / (G < 16 ? G : 16);
}

// Arguments as for jv_attn_simt (csrc/attn_simt.cu), bfloat16 only.  n_splits == 0: prompt portions,
// work = (entry, first token of the tile) with jv_attn_mma_tokens_per_tile tokens per tile.
// n_splits > 0: single tokens, part_o [n_work*Hq*n_splits*D] and part_ml [n_work*Hq*n_splits*2] floats of
// scratch, and `counters`, n_work * n_kv_heads * ceil(G/16) ints that are zero before the launch (the
// kernel leaves them zero).
JV_EXPORT int jv_attn_mma(const void* q, int q_stride, void* out, int out_stride, float* part_o, float* part_ml,
                          int* counters, const void* k_cache, const void* v_cache, const int* block_table, int table_width,
                          const int* cu_seqlens, const int* start_pos, const int* work, int n_work,
                          int n_q_heads, int n_kv_heads, int head_dim, int page_size, int num_pages, int window,
                          float scale, int split_size, int n_splits, int* status, cudaStream_t stream) {
  if (n_work == 0) return JV_OK;
  if (!jv_attn_mma_supports(head_dim) || n_kv_heads < 1 || n_q_heads % n_kv_heads != 0) return JV_ERR_UNSUPPORTED;
  if ((q_stride % 8) || (out_stride % 2) || ((uintptr_t)q % 16) || ((uintptr_t)k_cache % 16) || ((uintptr_t)v_cache % 16))
    return JV_ERR_UNSUPPORTED;   // 16-byte copies need aligned rows
  Params p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride; p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.part_o = part_o; p.part_ml = part_ml; p.counters = counters;
  p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache;
  p.block_table = block_table; p.table_width = table_width; p.cu_seqlens = cu_seqlens; p.start_pos = start_pos;
  p.work = work; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size;
  p.num_pages = num_pages; p.window = window; p.scale_log2 = scale * LOG2E; p.status = status;
  const int G = n_q_heads / n_kv_heads;
  p.heads_per_tile = G < 16 ? G : 16;
  p.n_head_groups = (G + p.heads_per_tile - 1) / p.heads_per_tile;
  p.tokens_per_tile = n_splits > 0 ? 1 : ROWS_PREFILL / p.heads_per_tile;
  p.split_size = split_size > 0 ? split_size : 1;
  p.n_splits = n_splits;
  const bool split = n_splits > 0;
  switch (head_dim) {
    case 16: return launch<16>(p, n_work, split, stream);
    case 32: return launch<32>(p, n_work, split, stream);
    case 64: return launch<64>(p, n_work, split, stream);
    case 128: return launch<128>(p, n_work, split, stream);
  }
  return JV_ERR_UNSUPPORTED;
}
