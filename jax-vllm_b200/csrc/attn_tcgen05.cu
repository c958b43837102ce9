// Paged causal attention of prompt portions on the 5th-generation tensor cores, for head size 128:
// scores and output accumulate in tensor memory (TMEM), queries, keys and values come in by TMA in the
// 128-byte-swizzle layout that tcgen05.mma reads.
//
// A work item is up to 128 rows = (token, query head) pairs of ONE kv head (row r -> token r / HPT, head
// r % HPT, HPT = query heads per kv head, any number up to 16: 128 / HPT tokens, the rows that are left over
// when HPT does not divide 128 are computed and thrown away), against 128-key tiles.  Blocks are persistent,
// one per multiprocessor: block b takes the items b, 2G-1-b, 2G+b, ... of the list ordered longest first (G
// blocks; back and forth, so that every block gets long and short ones), and the roles run through the tiles
// of all their items as one sequence, so that an item's first keys, its queries and its first scores are under
// way while the item before it is still in its softmax and its output leaves:
//   warp 0   key producer: reads the block table, issues the TMA loads of an item's query tile (two buffers)
//            and of the key tiles (one 4-D box per page and half of the head: [page slots, 64] elements);
//   warp 10  value producer: the same for the value tiles (a stage of values is free much later than a stage
//            of keys, and one warp that waits for both holds the keys back);
//   warp 1   one thread issues S = Q K^T (8 x tcgen05.mma 128x128x16 over the head) into one of two score
//            buffers in TMEM, and O += P V (8 x mma over the keys; P is read from TMEM, V is the MN-major
//            operand from shared memory), after the softmax warps have written P (bfloat16) to TMEM;
//   warps 2..9  softmax, two threads per row: read the scores from TMEM, mask, running (max, sum) in 32-bit,
//            exp2, write P; when a row's maximum has moved, rescale O in TMEM first.  At an item's end O / sum
//            leaves through the item's query buffer and a TMA store.
// The score buffer of the next tile (of this item or the next) is filled while the softmax of a tile runs.
// Shared memory moves 128 bytes a clock, which a 128x128x16 product with both operands there needs all by
// itself: P therefore never goes through shared memory.  Every mbarrier wait is bounded by a clock deadline and
// reports to the status word instead of spinning.
//
// Restrictions (the caller falls back to the mma.sync kernel otherwise): bfloat16, head size 128, no
// window, HPT up to 16, page size a power of two from 8 to 128.
#include "common.cuh"
#include "mbarrier.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>
#include <math.h>

namespace {

constexpr int D = 128, ROWS = 128, BN = 128;
constexpr int TILE_BYTES = 128 * 128 * 2;       // a 128 x 128 bfloat16 tile: two halves of [128 rows][128 bytes]
constexpr int HALF_BYTES = 128 * 128;            // one half: 128 rows of 128 bytes
constexpr int K_STAGES = 2, V_STAGES = 3, Q_BUFFERS = 2;   // 7 tiles of 32 KB
constexpr int THREADS = 352;                     // key producer warp, mma warp, 8 softmax warps, value producer warp
constexpr int SOFTMAX_THREADS = 256;
constexpr int TMEM_COLS = 512;                   // S0: [0,128)  S1: [128,256)  O: [256,384)  P0: [384,448)  P1: [448,512)
constexpr int TMEM_O = 256, TMEM_P = 384;        // a column of P holds two bfloat16: keys 2c and 2c+1
constexpr float LOG2E = 1.4426950408889634f;

struct Params {
  __nv_bfloat16* out; int out_stride;
  const int* block_table; int table_width;
  const int* cu_seqlens; const int* start_pos; const int* work;
  int n_work, n_q_heads, n_kv_heads, page_size, num_pages, hpt, tokens_per_tile;
  float scale_log2;
  int* status;
};

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
               ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, int x, int y, int z, int w, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n"
               ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];\n"
               ::"l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(src)) : "memory");
}

// Descriptor of a K-major operand tile (rows of 128 bytes along k, 8-row groups 1024 bytes apart, 128-byte swizzle).
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// Descriptor of an MN-major operand tile: rows of 128 bytes run along n (64 elements), consecutive rows are
// consecutive k, 8 rows = 1024 bytes (stride byte offset); the next 64 n are HALF_BYTES further (leading byte offset).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(HALF_BYTES >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// bfloat16 x bfloat16 -> float, M = 128, N = 128; B K-major (S = Q K^T) or MN-major (O = P V).
constexpr uint32_t IDESC_QK = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
constexpr uint32_t IDESC_PV = IDESC_QK | (1u << 16);

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the A operand in tensor memory (rows = lanes, two 16-bit elements of k per column).
__device__ __forceinline__ void umma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
               ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
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
// The same without waiting: several loads can be in flight; tmem_ld_wait() before the values are used.
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_st32_bits(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]),
        "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
        "r"(v[30]), "r"(v[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Two 32-bit floats in one 64-bit register pair, for the packed fma and add of sm_100.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
#define TC_FENCE_BEFORE() asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory")
#define TC_FENCE_AFTER() asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory")
#define PROXY_FENCE() asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory")

// Barrier of the two softmax warps that share 32 rows (64 threads; barriers 1..4, one for each pair) that also
// tells every one of them whether any had `flag` set.
__device__ __forceinline__ bool pair_barrier_or(int quad, bool flag) {
  uint32_t any;
  asm volatile("{\n.reg .pred p, q;\nsetp.ne.b32 q, %2, 0;\nbar.red.or.pred p, %1, 64, q;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(any) : "r"(quad + 1), "r"((uint32_t)flag) : "memory");
  return any != 0;
}
__device__ __forceinline__ void pair_barrier(int quad) { asm volatile("bar.sync %0, 64;\n" ::"r"(quad + 1) : "memory"); }

struct Shared {
  uint64_t q_full[Q_BUFFERS], q_free[Q_BUFFERS], k_full[K_STAGES], k_empty[K_STAGES], v_full[V_STAGES], v_empty[V_STAGES];
  uint64_t s_full[2], p_full[2], o_done[2];
  uint64_t o_free;              // the softmax threads have read an item's output: the next item's may be written
  uint64_t drain;               // used only after a wait ran out (see the tear-down)
  uint32_t tmem_base;
  int failed;                   // a role gave up on a wait
  int armed_q[Q_BUFFERS], armed_k[K_STAGES], armed_v[V_STAGES];   // parity of the phase a producer armed last; -1: never
  float xch[2][128];            // a row's two softmax threads exchange their maxima (and at the end their sums)
};

// One work item as every role sees it.
struct Item {
  int entry, kv_head, q_first;      // request of the batch, kv head, first row of the tile among all tokens
  int tokens_here, pos_first;       // tokens in the tile, position of the first
  int j_hi, n_tiles;                // keys [0, j_hi) are visible to the last row; key tiles
};

__global__ void __launch_bounds__(THREADS, 1) attn_tcgen05_kernel(const __grid_constant__ CUtensorMap q_map,
                                                                  const __grid_constant__ CUtensorMap k_map,
                                                                  const __grid_constant__ CUtensorMap v_map,
                                                                  const __grid_constant__ CUtensorMap out_map,
                                                                  const Params p) {
  pdl_trigger();      // a kernel launched behind this one (decode attention of the same step) may take the multiprocessors that the first blocks to end leave free
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = base;                                   // [buffers][2 halves of d][128 rows][128 B]
  unsigned char* k_s = q_s + Q_BUFFERS * TILE_BYTES;           // [stages][2 halves of d][128 keys][128 B]
  unsigned char* v_s = k_s + K_STAGES * TILE_BYTES;            // [stages][2 halves of d][128 keys][128 B]
  Shared* sh = reinterpret_cast<Shared*>(v_s + V_STAGES * TILE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.n_q_heads / p.n_kv_heads, HPT = p.hpt;
  const int n_items = p.n_work * p.n_kv_heads, n_blocks = gridDim.x;

  // The items of this block: in round r the blocks take the items r G .. r G + G - 1 of the list ordered longest
  // first (the work list is in ascending order of a tile's first token, so from its end), in the order of their
  // numbers in even rounds and against it in odd ones.  -1: this block has none in that round.
  auto item_of_round = [&](int r) -> int {
    const int L = r * n_blocks + ((r & 1) ? n_blocks - 1 - (int)blockIdx.x : (int)blockIdx.x);
    return L < n_items ? L : -1;
  };
  const int n_rounds = (n_items + n_blocks - 1) / n_blocks;
  auto load_item = [&](int L) -> Item {
    Item it;
    const int w = p.n_work - 1 - L / p.n_kv_heads;
    it.kv_head = L % p.n_kv_heads;
    it.entry = p.work[2 * w];
    const int q_off = p.work[2 * w + 1];
    const int q_begin = p.cu_seqlens[it.entry];
    const int q_len = p.cu_seqlens[it.entry + 1] - q_begin;
    it.q_first = q_begin + q_off;
    it.tokens_here = min(p.tokens_per_tile, q_len - q_off);
    it.pos_first = p.start_pos[it.entry] + q_off;
    it.j_hi = it.pos_first + it.tokens_here;
    it.n_tiles = it.tokens_here > 0 ? (it.j_hi + BN - 1) / BN : 0;
    return it;
  };

  if (threadIdx.x == 0) {
    for (int b = 0; b < Q_BUFFERS; ++b) { mbar_init(&sh->q_full[b], 1); mbar_init(&sh->q_free[b], 1); sh->armed_q[b] = -1; }
    for (int s = 0; s < K_STAGES; ++s) { mbar_init(&sh->k_full[s], 1); mbar_init(&sh->k_empty[s], 1); sh->armed_k[s] = -1; }
    for (int s = 0; s < V_STAGES; ++s) { mbar_init(&sh->v_full[s], 1); mbar_init(&sh->v_empty[s], 1); sh->armed_v[s] = -1; }
    mbar_init(&sh->s_full[0], 1); mbar_init(&sh->s_full[1], 1);
    mbar_init(&sh->p_full[0], SOFTMAX_THREADS); mbar_init(&sh->p_full[1], SOFTMAX_THREADS);
    mbar_init(&sh->o_done[0], 1); mbar_init(&sh->o_done[1], 1);
    mbar_init(&sh->o_free, SOFTMAX_THREADS);
    mbar_init(&sh->drain, 1);
    sh->failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  // The producers start at once; the others wait until the second warp has its tensor memory.  Shared memory is
  // not cleared: key rows that were never loaded give scores that are masked before they are looked at, and the
  // value rows past the end of the last tile are set to zero there.
  if (warp >= 1 && warp <= 9) {
    if (warp == 1) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh->tmem_base)), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    TC_FENCE_BEFORE();
    asm volatile("bar.sync 6, 288;\n" ::: "memory");
    TC_FENCE_AFTER();
  }
  const uint32_t tmem = (warp >= 1 && warp <= 9) ? sh->tmem_base : 0u;
  const uint32_t tmem_o = tmem + TMEM_O;

  if (warp == 0 || warp == 10) {
    // --------------------------------------------------------------- producers
    const int which = warp == 0 ? 0 : 1;                        // keys (and queries) or values
    const int stages = which ? V_STAGES : K_STAGES;
    pdl_wait();                         // queries, keys and values are the work of the kernels before this one
    const int P = p.page_size, pages_per_tile = BN / P;
    uint64_t* full_bars = which ? sh->v_full : sh->k_full;
    uint64_t* empty_bars = which ? sh->v_empty : sh->k_empty;
    int* armed = which ? sh->armed_v : sh->armed_k;
    unsigned char* tiles = which ? v_s : k_s;
    const CUtensorMap* map = which ? &v_map : &k_map;
    bool ok = true;
    int gt = 0, n = 0;                  // tiles and items of this block so far
    for (int r = 0; r < n_rounds && ok; ++r) {
      const int L = item_of_round(r);
      if (L < 0) continue;
      const Item it = load_item(L);
      if (it.n_tiles == 0) continue;
      if (which == 0 && lane == 0) {
        const int qb = n % Q_BUFFERS, ph = (n / Q_BUFFERS) & 1;
        ok = mbar_wait(&sh->q_free[qb], ph ^ 1);                 // the item two before this one has left through this buffer
        if (ok) {
          sh->armed_q[qb] = ph;
          mbar_expect_tx(&sh->q_full[qb], 2 * 128 * G * p.tokens_per_tile);      // two boxes of 64 d x G heads x tokens
          tma_load_3d(q_s + qb * TILE_BYTES, &q_map, 0, it.kv_head * G, it.q_first, &sh->q_full[qb]);
          tma_load_3d(q_s + qb * TILE_BYTES + HALF_BYTES, &q_map, 64, it.kv_head * G, it.q_first, &sh->q_full[qb]);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      // page ids of a tile: lane i reads the i-th (a tile has at most 16 pages); -1 = no page needed or none there
      auto tile_pages = [&](int j) -> int {
        const int pi = j * pages_per_tile + lane;
        int page = -1;
        if (j < it.n_tiles && lane < pages_per_tile && pi * P < it.j_hi && pi < p.table_width) {
          page = p.block_table[(size_t)it.entry * p.table_width + pi];
          if (page < 0 || page >= p.num_pages) { atomicOr(p.status, JV_STATUS_BAD_PAGE); page = -1; }
        }
        return page;
      };
      // the block-table entries of a tile are read while the tile before it is loaded
      int pages = tile_pages(0);
      for (int j = 0; j < it.n_tiles && ok; ++j, ++gt) {
        const int pages_next = tile_pages(j + 1);
        const int s = gt % stages, ph = (gt / stages) & 1;
        unsigned char* dst = tiles + s * TILE_BYTES;
        const int n_pages = __popc(__ballot_sync(0xffffffffu, pages >= 0));
        if (lane == 0) {
          ok = mbar_wait(&empty_bars[s], ph ^ 1);
          if (ok) { armed[s] = ph; mbar_expect_tx(&full_bars[s], n_pages * P * 128 * 2); }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);      // also orders the announcement before the copies
        // lane i issues the two boxes of page i
        if (ok && pages >= 0) {
          tma_load_4d(dst + lane * P * 128, map, 0, it.kv_head, 0, pages, &full_bars[s]);
          tma_load_4d(dst + HALF_BYTES + lane * P * 128, map, 64, it.kv_head, 0, pages, &full_bars[s]);
        }
        pages = pages_next;
      }
      ++n;
    }
    if (!ok && lane == 0) { atomicOr(p.status, JV_STATUS_WAIT_EXPIRED); sh->failed = 1; }
  } else if (warp == 1) {
    // -------------------------------------------------------------- mma issuer
    if (lane == 0) {
      uint64_t q_desc[Q_BUFFERS][2], k_desc[K_STAGES][2], v_desc[V_STAGES];
#pragma unroll
      for (int b = 0; b < Q_BUFFERS; ++b) {
        q_desc[b][0] = desc_k_major(smem_u32(q_s + b * TILE_BYTES));
        q_desc[b][1] = desc_k_major(smem_u32(q_s + b * TILE_BYTES + HALF_BYTES));
      }
#pragma unroll
      for (int st = 0; st < K_STAGES; ++st) {
        k_desc[st][0] = desc_k_major(smem_u32(k_s + st * TILE_BYTES));
        k_desc[st][1] = desc_k_major(smem_u32(k_s + st * TILE_BYTES + HALF_BYTES));
      }
#pragma unroll
      for (int st = 0; st < V_STAGES; ++st) v_desc[st] = desc_mn_major(smem_u32(v_s + st * TILE_BYTES));
      // Where this thread stands in the block's sequence of tiles: round, item number, tile of the item, its tiles.
      // The item after the current one is looked up when the current one begins, so that the loads for it have
      // long arrived when its first scores are due (while the current item's last softmax runs).
      struct At { int r, n, j, nt; };
      struct Ahead { int r, nt; };
      auto find_from = [&](int r) -> Ahead {                    // the first round from r on that holds an item with tiles
        for (; r < n_rounds; ++r) {
          const int L = item_of_round(r);
          if (L < 0) continue;
          const int nt = load_item(L).n_tiles;
          if (nt > 0) return Ahead{r, nt};
        }
        return Ahead{n_rounds, 0};
      };
      Ahead peek = find_from(0);
      At cur{peek.r, 0, 0, peek.nt};
      if (cur.r < n_rounds) peek = find_from(cur.r + 1);
      auto after = [&](const At& a) -> At {
        if (a.j + 1 < a.nt) return At{a.r, a.n, a.j + 1, a.nt};
        const At b{peek.r, a.n + 1, 0, peek.nt};
        if (b.r < n_rounds) peek = find_from(b.r + 1);
        return b;
      };
      auto issue_qk = [&](const At& a, int gt) -> bool {          // S[gt % 2] = Q K^T for tile gt of the sequence
        const int qb = a.n % Q_BUFFERS, s = gt % K_STAGES;
        if (a.j == 0 && !mbar_wait(&sh->q_full[qb], (a.n / Q_BUFFERS) & 1)) return false;
        if (!mbar_wait(&sh->k_full[s], (gt / K_STAGES) & 1)) return false;
        TC_FENCE_AFTER();
        const uint64_t q0 = q_desc[qb][0], q1 = q_desc[qb][1], k0 = k_desc[s][0], k1 = k_desc[s][1];
        const uint32_t tmem_s = tmem + (gt & 1) * 128;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) umma(tmem_s, q0 + 2 * kk, k0 + 2 * kk, IDESC_QK, kk != 0);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) umma(tmem_s, q1 + 2 * kk, k1 + 2 * kk, IDESC_QK, 1);
        umma_commit(&sh->k_empty[s]);
        umma_commit(&sh->s_full[gt & 1]);
        return true;
      };
      bool ok = true;
      if (cur.r < n_rounds) ok = issue_qk(cur, 0);
      for (int gt = 0; cur.r < n_rounds && ok; ++gt) {
        const At nxt = after(cur);
        if (nxt.r < n_rounds) ok = issue_qk(nxt, gt + 1);          // the next scores while this tile's softmax runs
        if (!ok) break;
        const int s = gt % V_STAGES;
        if (!mbar_wait(&sh->p_full[gt & 1], (gt >> 1) & 1) || !mbar_wait(&sh->v_full[s], (gt / V_STAGES) & 1)) { ok = false; break; }
        // an item's first product overwrites the output of the item before it, which its softmax threads must have read
        if (cur.j == 0 && cur.n > 0 && !mbar_wait(&sh->o_free, (cur.n - 1) & 1)) { ok = false; break; }
        TC_FENCE_AFTER();
        // O += P V_j : 8 steps of 16 keys; P from tensor memory (8 columns a step), V MN-major
        const uint32_t tmem_p = tmem + TMEM_P + (gt & 1) * 64;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)   // 16 keys further: 8 columns of P, 16 rows (2048 bytes) down V
          umma_a_tmem(tmem_o, tmem_p + kk * 8, v_desc[s] + kk * (16 * 128 / 16), IDESC_PV, (cur.j | kk) != 0);
        umma_commit(&sh->v_empty[s]);
        umma_commit(&sh->o_done[gt & 1]);
        cur = nxt;
      }
      if (!ok) { atomicOr(p.status, JV_STATUS_WAIT_EXPIRED); sh->failed = 1; }
    }
  } else {
    // ----------------------------------------------------------------- softmax
    // Two threads per row: warps 2..5 take the first 64 keys of a tile (and the first 64 columns of O),
    // warps 6..9 the other 64.  A warp reads the 32 TMEM lanes of its number modulo 4.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quad * 32 + lane;                           // this thread's row of the tile
    const int t = row / HPT, hh = row % HPT;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    constexpr float LAZY = 8.f;
    bool ok = true;
    int gt = 0, n = 0;
    int stored = -1;              // thread 64: the query buffer whose TMA store has been started but not yet waited for
    // the numbers of the next item are asked for while the current one runs (two dependent loads from global memory)
    auto next_item = [&](int& r, Item& out) -> bool {
      for (; r < n_rounds; ++r) {
        const int L = item_of_round(r);
        if (L < 0) continue;
        out = load_item(L);
        if (out.n_tiles > 0) return true;
      }
      return false;
    };
    int r_next = 0;
    Item upcoming;
    bool more = next_item(r_next, upcoming);
    while (more) {
      const Item it = upcoming;
      ++r_next;
      more = next_item(r_next, upcoming);
      const int n_tiles = it.n_tiles, j_hi = it.j_hi, pos_first = it.pos_first;
      const bool row_ok = t < it.tokens_here && hh < G;
      const int pos = row_ok ? pos_first + t : -1;
      // m_ref is the reference maximum that the exponentials are taken against.  It follows the true
      // maximum lazily: only when the maximum has grown by more than 2^8 (in the exponent) is O rescaled,
      // which is rare after the first tiles; until then probabilities may exceed 1 by at most that factor.
      float m_ref = -INFINITY, l_run = 0.f;
      // A wait that runs out makes `ok` false for the whole warp; the loops then only keep their appointments at
      // the named barriers (so that nobody is left waiting there) and do no further work.
      for (int j = 0; j < n_tiles; ++j, ++gt) {
        if (ok) ok = mbar_wait(&sh->s_full[gt & 1], (gt >> 1) & 1);
        ok = __all_sync(0xffffffffu, ok);
        const uint32_t s_addr = tmem + lane_addr + (gt & 1) * 128 + half * 64;
        const int key0 = j * BN + half * 64;                     // first key of this thread's 64
        const bool need_mask = j * BN + BN > j_hi || j * BN + BN - 1 > pos_first;   // block-uniform
        uint32_t sr[2][32];
        float my_max = -INFINITY;
        if (ok) {
          TC_FENCE_AFTER();
          tmem_ld32_issue(s_addr, sr[0]);
          tmem_ld32_issue(s_addr + 32, sr[1]);
          tmem_ld_wait();
          // masking is a loop of its own behind a branch that the whole block takes or not: only the last
          // tile of an item has keys to hide
          if (need_mask) {
            const int last = min(pos, j_hi - 1) - key0;          // the last of this thread's 64 keys that counts
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (c * 32 + i > last) sr[c][i] = __float_as_uint(-INFINITY);
          }
          float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 2)
              mx[(i >> 1) & 3] = max3(mx[(i >> 1) & 3], __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
          my_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        }
        // ---- the reference moves only if some score of the tile has outgrown it (always in a row's first tile
        // with keys, rarely later): one barrier tells all 256 threads whether any row is in that case, and only
        // then do the two threads of a row exchange their maxima
        const bool outgrown = ok && my_max != -INFINITY && (m_ref == -INFINITY || (my_max - m_ref) * p.scale_log2 > LAZY);
        float alpha = 1.f;
        if (pair_barrier_or(quad, outgrown)) {
          sh->xch[half][row] = my_max;
          pair_barrier(quad);
          const float m_tile = fmaxf(sh->xch[0][row], sh->xch[1][row]);
          pair_barrier(quad);                                        // both have read before a later tile writes
          if (ok && m_tile != -INFINITY && (m_ref == -INFINITY || (m_tile - m_ref) * p.scale_log2 > LAZY)) {
            alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2((m_ref - m_tile) * p.scale_log2);
            m_ref = m_tile;
          }
        }
        const float m_scaled = (m_ref == -INFINITY) ? 0.f : m_ref * p.scale_log2;
        // ---- O is rescaled only if some row of this warp moved its reference; the previous P V must be complete then
        if (ok && j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
          ok = __all_sync(0xffffffffu, mbar_wait(&sh->o_done[(gt - 1) & 1], ((gt - 1) >> 1) & 1));
          if (ok) {
            TC_FENCE_AFTER();
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
              float v[32];
              tmem_ld32(tmem_o + lane_addr + half * 64 + c * 32, v);
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] *= alpha;
              tmem_st32(tmem_o + lane_addr + half * 64 + c * 32, v);
            }
          }
        }
        // this tile's P buffer (in tensor memory) was read by the product of the tile two before it, which was issued
        // before the scores of this tile: their arrival has told that it is complete
        if (!ok) continue;
        // ---- probabilities: pairs of scores in packed 32-bit arithmetic, as bfloat16 pairs into this thread's 32
        // columns of the P buffer (column c of a row holds its keys 2c and 2c+1)
        float sum[4];
        {
          const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), neg_m2 = pack2(-m_scaled, -m_scaled);
          uint64_t sum2[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
          uint32_t pw[32];
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const uint64_t x2 = fma2(pack2(__uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1])), scale2, neg_m2);
              float x0, x1;
              unpack2(x2, x0, x1);
              const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
              sum2[(i >> 1) & 1] = add2(sum2[(i >> 1) & 1], pack2(p0, p1));
              const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
              pw[c * 16 + (i >> 1)] = *reinterpret_cast<const uint32_t*>(&h);
            }
          unpack2(sum2[0], sum[0], sum[1]);
          unpack2(sum2[1], sum[2], sum[3]);
          tmem_st32_bits(tmem + lane_addr + TMEM_P + (gt & 1) * 64 + half * 32, pw);
        }
        l_run = l_run * alpha + ((sum[0] + sum[1]) + (sum[2] + sum[3]));
        // ---- in an item's last tile the value rows past the end become zero (they may hold anything)
        if (j == n_tiles - 1 && j_hi < j * BN + BN) {
          const int s = gt % V_STAGES;
          ok = __all_sync(0xffffffffu, mbar_wait(&sh->v_full[s], (gt / V_STAGES) & 1));
          if (ok) {
            for (int i = (threadIdx.x - 64); i < (j * BN + BN - j_hi) * 16; i += SOFTMAX_THREADS) {
              const int key_row = (j_hi - j * BN) + i / 16, part = i % 16;     // 16 chunks of 16 bytes per row (both halves)
              *reinterpret_cast<uint4*>(v_s + s * TILE_BYTES + (part >> 3) * HALF_BYTES + key_row * 128 + (part & 7) * 16) =
                  make_uint4(0, 0, 0, 0);
            }
          }
        }
        if (!ok) continue;
        if (j == n_tiles - 1) PROXY_FENCE();                     // the zeroed rows visible to the tensor core
        TC_FENCE_BEFORE();                                       // P is in tensor memory before the arrival
        mbar_arrive(&sh->p_full[gt & 1]);
        if (stored >= 0) {
          // the output of the item before this one has long been read out of its query buffer by now: the buffer
          // may take the queries of the item after this one
          asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
          mbar_arrive(&sh->q_free[stored]);
          stored = -1;
        }
      }
      // ---- the item's output: O / sum, each thread its 64 columns; the row's sum is the two threads' together
      const int g_last = gt - 1, qb = n % Q_BUFFERS;
      sh->xch[half][row] = l_run;
      pair_barrier(quad);
      const float l_row = sh->xch[0][row] + sh->xch[1][row];
      pair_barrier(quad);                                        // both have read before the next item's first tile writes
      const bool got = ok && mbar_wait(&sh->o_done[g_last & 1], (g_last >> 1) & 1);
      const float inv = row_ok ? 1.f / l_row : 0.f;
      const bool whole = it.tokens_here == p.tokens_per_tile;
      // A whole tile leaves through shared memory (where the item's queries were: every product with them has
      // completed) and one TMA store per half of the head; threads that write their 128 bytes to rows 8 KB apart in
      // memory take five times as long.
      unsigned char* row_base = q_s + qb * TILE_BYTES + half * HALF_BYTES + row * 128;
      __nv_bfloat16* dst = p.out + (size_t)(it.q_first + t) * p.out_stride + (size_t)(it.kv_head * G + hh) * D + half * 64;
      if (got) {
        TC_FENCE_AFTER();
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          float v[32];
          tmem_ld32(tmem_o + lane_addr + half * 64 + c * 32, v);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 pk;
            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
            for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(v[q * 8 + 2 * e] * inv, v[q * 8 + 2 * e + 1] * inv);
            const int chunk = c * 4 + q;                       // 16-byte chunk within the 128-byte row
            if (whole) *reinterpret_cast<uint4*>(row_base + ((chunk ^ (row & 7)) << 4)) = pk;
            else if (row_ok) *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = pk;
          }
        }
        TC_FENCE_BEFORE();
        mbar_arrive(&sh->o_free);                                // this thread has read its part of the output
      }
      if (whole) {
        PROXY_FENCE();
        asm volatile("bar.sync 5, 256;\n" ::: "memory");
        if (threadIdx.x == 64) {
          if (got) {
            // started here, waited for after the next item's first tile (or at the end): this thread's warp is not held up
            tma_store_3d(&out_map, q_s + qb * TILE_BYTES, 0, it.kv_head * G, it.q_first);
            tma_store_3d(&out_map, q_s + qb * TILE_BYTES + HALF_BYTES, 64, it.kv_head * G, it.q_first);
            asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
            stored = qb;
          } else {
            mbar_arrive(&sh->q_free[qb]);
          }
        }
      } else if (threadIdx.x == 64) {
        mbar_arrive(&sh->q_free[qb]);                            // nothing left through the buffer
      }
      if (!got) ok = false;
      ++n;
    }
    if (stored >= 0) {                                           // shared memory must have been read before the block ends
      asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
      mbar_arrive(&sh->q_free[stored]);
    }
    if (!ok && lane == 0) { atomicOr(p.status, JV_STATUS_WAIT_EXPIRED); sh->failed = 1; }
  }

  TC_FENCE_BEFORE();
  __syncthreads();
  if (sh->failed) {
    // a wait ran out: products already issued may still write tensor memory and copies already asked for still land
    // in this block's shared memory; both get a bounded time to finish before tensor memory is freed and the block ends
    if (warp == 1 && lane == 0) drain_products_after_failure(&sh->drain);
    if (warp == 0 && lane == 0) {
      for (int b = 0; b < Q_BUFFERS; ++b)
        if (sh->armed_q[b] >= 0) drain_copies_after_failure(&sh->q_full[b], sh->armed_q[b]);
      for (int s = 0; s < K_STAGES; ++s)
        if (sh->armed_k[s] >= 0) drain_copies_after_failure(&sh->k_full[s], sh->armed_k[s]);
    }
    if (warp == 10 && lane == 0)
      for (int s = 0; s < V_STAGES; ++s)
        if (sh->armed_v[s] >= 0) drain_copies_after_failure(&sh->v_full[s], sh->armed_v[s]);
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
}  // namespace

// 1 if this kernel takes the case (else the caller uses the mma.sync kernel).
JV_EXPORT int jv_attn_tcgen05_supports(int head_dim, int n_q_heads, int n_kv_heads, int page_size, int window) {
  if (head_dim != 128 || window > 0 || n_kv_heads < 1 || n_q_heads % n_kv_heads) return 0;
  const int G = n_q_heads / n_kv_heads;
  if (G > 16) return 0;
  return page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 || page_size == 128;
}

// Tokens per 128-row tile.
JV_EXPORT int jv_attn_tcgen05_tokens_per_tile(int n_q_heads, int n_kv_heads) { return ROWS / (n_q_heads / n_kv_heads); }

// q: [n_tokens, q_stride] bfloat16 with head h of a token at column h*128; out: [n_tokens, out_stride];
// k_cache/v_cache: [num_pages, page_size, n_kv_heads, 128]; work: [n_work, 2] (entry, first token of the tile),
// tiles of jv_attn_tcgen05_tokens_per_tile tokens, in ascending order of work.
JV_EXPORT int jv_attn_tcgen05(const void* q, int q_stride, int n_tokens, void* out, int out_stride, const void* k_cache,
                              const void* v_cache, const int* block_table, int table_width, const int* cu_seqlens,
                              const int* start_pos, const int* work, int n_work, int n_q_heads, int n_kv_heads,
                              int head_dim, int page_size, int num_pages, float scale, int* status, cudaStream_t stream) {
  if (n_work == 0) return JV_OK;
  if (!jv_attn_tcgen05_supports(head_dim, n_q_heads, n_kv_heads, page_size, 0)) return JV_ERR_UNSUPPORTED;
  if ((q_stride % 8) || (out_stride % 8) || ((uintptr_t)q % 16) || ((uintptr_t)out % 16) || ((uintptr_t)k_cache % 16) ||
      ((uintptr_t)v_cache % 16))
    return JV_ERR_UNSUPPORTED;
  auto fn = encode_fn();
  if (fn == nullptr) return JV_ERR_UNSUPPORTED;
  const int G = n_q_heads / n_kv_heads;
  CUtensorMap q_map, k_map, v_map, out_map;
  for (int which = 0; which < 2; ++which) {
    // queries and output: (d, head, token); a box is 64 d x G heads x (128 / G) tokens = 128 rows, head fastest
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)n_q_heads, (cuuint64_t)n_tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)(which ? out_stride : q_stride) * 2};
    const cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(ROWS / G)};
    const cuuint32_t es[3] = {1, 1, 1};
    if (fn(which ? &out_map : &q_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, which ? out : const_cast<void*>(q), dims, strides, box, es,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return JV_ERR_UNSUPPORTED;
  }
  for (int which = 0; which < 2; ++which) {
    // cache: (d, kv head, slot, page); a box is 64 d x 1 head x page_size slots x 1 page
    const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)n_kv_heads, (cuuint64_t)page_size, (cuuint64_t)num_pages};
    const cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)n_kv_heads * D * 2, (cuuint64_t)page_size * n_kv_heads * D * 2};
    const cuuint32_t box[4] = {64, 1, (cuuint32_t)page_size, 1};
    const cuuint32_t es[4] = {1, 1, 1, 1};
    if (fn(which ? &v_map : &k_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(which ? v_cache : k_cache), dims,
           strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return JV_ERR_UNSUPPORTED;
  }
  Params p;
  p.out = (__nv_bfloat16*)out; p.out_stride = out_stride; p.block_table = block_table; p.table_width = table_width;
  p.cu_seqlens = cu_seqlens; p.start_pos = start_pos; p.work = work; p.n_work = n_work; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
  p.page_size = page_size; p.num_pages = num_pages; p.hpt = G; p.tokens_per_tile = ROWS / G;
  p.scale_log2 = scale * LOG2E; p.status = status;
  constexpr size_t smem = TILE_BYTES * (Q_BUFFERS + K_STAGES + V_STAGES) + sizeof(Shared) + 1024;
  static bool ready[JV_MAX_DEVICES];
  if (!jv_once_per_device(ready, [&] {
        return cudaFuncSetAttribute(attn_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
      }))
    return JV_ERR_UNSUPPORTED;
  // persistent blocks: one per multiprocessor (or per item, if there are fewer)
  static int sm_count[JV_MAX_DEVICES];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= JV_MAX_DEVICES) return JV_ERR_UNSUPPORTED;
  if (sm_count[dev] == 0 &&
      (cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count[dev] <= 0))
    sm_count[dev] = 148;
  const long long items = (long long)n_work * n_kv_heads;
  const int blocks = items < sm_count[dev] ? (int)items : sm_count[dev];
  return jv_launch(attn_tcgen05_kernel, dim3(blocks), dim3(THREADS), smem, stream, q_map, k_map, v_map, out_map, p);
}
