// Paged causal attention on CUDA cores with 32-bit arithmetic throughout: the kernel of
// the 32-bit path, and the fallback for head sizes that the tensor-core kernels do not
// take.  It serves prompt portions of any length (with earlier context in the cache),
// single decoded tokens, and decoded tokens split along the keys.
//
// Work item = (entry, first token of the tile); grid.y = kv head x head group;
// grid.z = key split (1 unless SPLIT).  The 16 rows of a tile are (token, query head)
// pairs of ONE kv head, so keys and values are read once for all query heads of the
// group: row m -> token q_off + m / heads_per_tile, head kv*G + hg*heads_per_tile +
// m % heads_per_tile.  Keys run over the entry's block table; key j is visible to a
// query at position p iff j <= p and (window == 0 or j > p - window).  Softmax is the
// running (max, sum) form; scores, probabilities and the output sum are float.
//
// SPLIT: split s covers key positions [s*split_size, (s+1)*split_size) of the visible
// range; it writes its unnormalised output sum and (max, sum) to `part_o`/`part_ml`;
// `attn_combine_kernel` merges the splits of a row in ascending order, so the result
// does not depend on what else is in the batch.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int BLOCK_M = 16;
constexpr int BLOCK_N = 32;
constexpr int THREADS = 128;

struct AttnParams {
  const void* q; int q_stride;
  void* out; int out_stride;
  float* part_o; float* part_ml;
  const void* k_cache; const void* v_cache;
  const int* block_table; int table_width;
  const int* cu_seqlens; const int* start_pos;
  const int* work;  // [n_work][2] = (entry, q_off)
  int n_q_heads, n_kv_heads, head_dim, page_size, num_pages, window;
  float scale;
  int tokens_per_tile, heads_per_tile, n_head_groups, split_size, n_splits;
  int* status;
};

template <typename T, bool SPLIT>
__global__ void __launch_bounds__(THREADS) attn_simt_kernel(const AttnParams p) {
  extern __shared__ float smem[];
  const int D = p.head_dim;
  float* Qs = smem;                                // [BLOCK_M][D]
  float* Ks = Qs + BLOCK_M * D;                    // [BLOCK_N][D+1]
  float* Vs = Ks + BLOCK_N * (D + 1);              // [BLOCK_N][D]
  float* Ss = Vs + BLOCK_N * D;                    // [BLOCK_M][BLOCK_N]
  float* row_m = Ss + BLOCK_M * BLOCK_N;           // [BLOCK_M]
  float* row_l = row_m + BLOCK_M;                  // [BLOCK_M]
  float* row_alpha = row_l + BLOCK_M;              // [BLOCK_M]
  int* row_pos = (int*)(row_alpha + BLOCK_M);      // [BLOCK_M] absolute position, -1 = unused row

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int entry = p.work[2 * blockIdx.x], q_off = p.work[2 * blockIdx.x + 1];
  const int kv_head = blockIdx.y / p.n_head_groups, hg = blockIdx.y % p.n_head_groups;
  const int G = p.n_q_heads / p.n_kv_heads;
  const int q_begin = p.cu_seqlens[entry];
  const int q_len = p.cu_seqlens[entry + 1] - q_begin;
  const int ctx = p.start_pos[entry];
  const int tokens_here = min(p.tokens_per_tile, q_len - q_off);
  if (tokens_here <= 0) return;

  // visible key range of the tile
  const int pos_first = ctx + q_off, pos_last = ctx + q_off + tokens_here - 1;
  int j_lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
  int j_hi = pos_last + 1;  // exclusive
  if (SPLIT) {
    j_lo = max(j_lo, blockIdx.z * p.split_size);
    j_hi = min(j_hi, (blockIdx.z + 1) * p.split_size);
    if (j_lo >= j_hi) return;
  }

  const T* q = (const T*)p.q;
  const T* kc = (const T*)p.k_cache;
  const T* vc = (const T*)p.v_cache;

  // rows: positions and query vectors
  if (tid < BLOCK_M) {
    const int t = tid / p.heads_per_tile, hh = hg * p.heads_per_tile + tid % p.heads_per_tile;
    row_pos[tid] = (t < tokens_here && hh < G) ? ctx + q_off + t : -1;
    row_m[tid] = -INFINITY;
    row_l[tid] = 0.f;
  }
  for (int idx = tid; idx < BLOCK_M * D; idx += THREADS) {
    const int m = idx / D, d = idx - m * D;
    const int t = m / p.heads_per_tile, hh = hg * p.heads_per_tile + m % p.heads_per_tile;
    float v = 0.f;
    if (t < tokens_here && hh < G)
      v = to_f32(q[(size_t)(q_begin + q_off + t) * p.q_stride + (size_t)(kv_head * G + hh) * D + d]);
    Qs[idx] = v;
  }

  constexpr int DC = 2;  // output columns per thread: d = tid, tid + THREADS  (head_dim <= 256)
  float acc[BLOCK_M][DC];
#pragma unroll
  for (int m = 0; m < BLOCK_M; ++m)
#pragma unroll
    for (int c = 0; c < DC; ++c) acc[m][c] = 0.f;
  __syncthreads();

  for (int j0 = j_lo; j0 < j_hi; j0 += BLOCK_N) {
    // ---- keys and values of this chunk into shared memory (one warp per key row)
    for (int n = warp; n < BLOCK_N; n += THREADS / 32) {
      const int j = j0 + n;
      const T* krow = nullptr;
      const T* vrow = nullptr;
      if (j < j_hi) {
        const int pi = j / p.page_size;
        const int page = pi < p.table_width ? p.block_table[(size_t)entry * p.table_width + pi] : -1;
        if (page < 0 || page >= p.num_pages) {
          if (lane == 0) atomicOr(p.status, JV_STATUS_BAD_PAGE);
        } else {
          const size_t off = (((size_t)page * p.page_size + (j % p.page_size)) * p.n_kv_heads + kv_head) * D;
          krow = kc + off;
          vrow = vc + off;
        }
      }
      for (int d = lane; d < D; d += 32) {
        Ks[n * (D + 1) + d] = krow ? to_f32(krow[d]) : 0.f;
        Vs[n * D + d] = vrow ? to_f32(vrow[d]) : 0.f;
      }
    }
    __syncthreads();

    // ---- scores: thread (n = lane, rows warp*4 .. warp*4+3)
    {
      float s[4] = {0.f, 0.f, 0.f, 0.f};
      const float* kr = Ks + lane * (D + 1);
      const float* q0 = Qs + (warp * 4) * D;
      for (int d = 0; d < D; ++d) {
        const float kv = kr[d];
#pragma unroll
        for (int r = 0; r < 4; ++r) s[r] = fmaf(q0[r * D + d], kv, s[r]);
      }
      const int j = j0 + lane;
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int m = warp * 4 + r;
        const int pos = row_pos[m];
        const bool vis = pos >= 0 && j < j_hi && j <= pos && (p.window <= 0 || j > pos - p.window);
        const float sc = vis ? s[r] * p.scale : -INFINITY;
        // ---- running softmax for row m (this warp owns the row)
        const float m_old = row_m[m];
        const float m_new = fmaxf(m_old, warp_max(sc));
        float pr = 0.f, alpha = 1.f;
        if (m_new != -INFINITY) {
          pr = vis ? expf(sc - m_new) : 0.f;
          alpha = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
        }
        const float psum = warp_sum(pr);
        Ss[m * BLOCK_N + lane] = pr;
        __syncwarp();
        if (lane == 0) {
          row_m[m] = m_new;
          row_l[m] = row_l[m] * alpha + psum;
          row_alpha[m] = alpha;
        }
      }
    }
    __syncthreads();

    // ---- output sum: thread owns columns d = tid + c*THREADS for all rows
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      const int d = tid + c * THREADS;
      if (d < D) {
#pragma unroll
        for (int m = 0; m < BLOCK_M; ++m) acc[m][c] *= row_alpha[m];
        for (int n = 0; n < BLOCK_N; ++n) {
          const float v = Vs[n * D + d];
#pragma unroll
          for (int m = 0; m < BLOCK_M; ++m) acc[m][c] = fmaf(Ss[m * BLOCK_N + n], v, acc[m][c]);
        }
      }
    }
    __syncthreads();
  }

  // ---- write
#pragma unroll
  for (int c = 0; c < DC; ++c) {
    const int d = tid + c * THREADS;
    if (d >= D) continue;
#pragma unroll
    for (int m = 0; m < BLOCK_M; ++m) {
      if (row_pos[m] < 0) continue;
      const int t = m / p.heads_per_tile, hh = hg * p.heads_per_tile + m % p.heads_per_tile;
      const int head = kv_head * G + hh;
      const size_t token = (size_t)(q_begin + q_off + t);
      if (SPLIT) {
        // rows of split launches are single tokens: index by work item
        const size_t slot = ((size_t)blockIdx.x * p.n_q_heads + head) * p.n_splits + blockIdx.z;
        p.part_o[slot * D + d] = acc[m][c];
        if (d == 0) {
          p.part_ml[slot * 2] = row_m[m];
          p.part_ml[slot * 2 + 1] = row_l[m];
        }
      } else {
        ((T*)p.out)[token * p.out_stride + (size_t)head * D + d] = from_f32<T>(acc[m][c] / row_l[m]);
      }
    }
  }
}

// Merges the key splits of single-token rows.  grid = (n_work, n_q_heads).
template <typename T>
__global__ void attn_combine_kernel(const AttnParams p) {
  const int x = blockIdx.x, head = blockIdx.y;
  const int entry = p.work[2 * x];
  const int D = p.head_dim;
  const int pos = p.start_pos[entry];
  const int j_lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int j_hi = pos + 1;
  const int s_first = j_lo / p.split_size;
  int s_last = (j_hi - 1) / p.split_size;  // inclusive
  if (s_last >= p.n_splits) {  // the launch has too few splits for this length
    if (threadIdx.x == 0) atomicOr(p.status, JV_STATUS_BAD_ROW);
    s_last = p.n_splits - 1;
  }
  const size_t base = ((size_t)x * p.n_q_heads + head) * p.n_splits;
  float m_all = -INFINITY;
  for (int s = s_first; s <= s_last; ++s) m_all = fmaxf(m_all, p.part_ml[(base + s) * 2]);
  float l_all = 0.f;
  for (int s = s_first; s <= s_last; ++s)
    l_all += expf(p.part_ml[(base + s) * 2] - m_all) * p.part_ml[(base + s) * 2 + 1];
  const size_t token = (size_t)p.cu_seqlens[entry];
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.f;
    for (int s = s_first; s <= s_last; ++s)
      o += expf(p.part_ml[(base + s) * 2] - m_all) * p.part_o[(base + s) * D + d];
    ((T*)p.out)[token * p.out_stride + (size_t)head * D + d] = from_f32<T>(o / l_all);
  }
}

size_t smem_bytes(int D) {
  return sizeof(float) * ((size_t)BLOCK_M * D + (size_t)BLOCK_N * (D + 1) + (size_t)BLOCK_N * D +
                          BLOCK_M * BLOCK_N + 3 * BLOCK_M) + sizeof(int) * BLOCK_M;
}
}  // namespace

// Rows of a tile that hold tokens: 16 / heads_per_tile, with heads_per_tile = min(G, 16).
JV_EXPORT int jv_attn_simt_tokens_per_tile(int n_q_heads, int n_kv_heads) {
  const int G = n_q_heads / n_kv_heads;
  const int hpt = G < BLOCK_M ? G : BLOCK_M;
  return BLOCK_M / hpt;
}

// q: rows of `q_stride` elements (head h of token n at q[n*q_stride + h*D]); out: [n, out_stride];
// k_cache/v_cache: [num_pages, page_size, n_kv_heads, head_dim]; block_table: [entries, table_width];
// cu_seqlens: [entries+1]; start_pos: [entries] (tokens cached before this step); work:
// [n_work, 2] int32 (entry, first token of the tile within the entry's new tokens).
// n_splits == 0: every work item attends to its whole visible range and writes `out`.
// n_splits > 0: work items are single tokens; part_o [n_work*Hq*n_splits*D] and part_ml
// [n_work*Hq*n_splits*2] floats are scratch; a second launch merges into `out`.
JV_EXPORT int jv_attn_simt(const void* q, int q_stride, void* out, int out_stride, int dtype,
                           float* part_o, float* part_ml, const void* k_cache, const void* v_cache,
                           const int* block_table, int table_width, const int* cu_seqlens,
                           const int* start_pos, const int* work, int n_work, int n_q_heads,
                           int n_kv_heads, int head_dim, int page_size, int num_pages, int window,
                           float scale, int split_size, int n_splits, int* status,
                           cudaStream_t stream) {
  if (n_work == 0) return JV_OK;
  if (head_dim < 1 || head_dim > 256 || n_kv_heads < 1 || n_q_heads % n_kv_heads != 0)
    return JV_ERR_UNSUPPORTED;
  AttnParams p;
  p.q = q; p.q_stride = q_stride; p.out = out; p.out_stride = out_stride;
  p.part_o = part_o; p.part_ml = part_ml; p.k_cache = k_cache; p.v_cache = v_cache;
  p.block_table = block_table; p.table_width = table_width; p.cu_seqlens = cu_seqlens;
  p.start_pos = start_pos; p.work = work; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads;
  p.head_dim = head_dim; p.page_size = page_size; p.num_pages = num_pages; p.window = window;
  p.scale = scale; p.status = status;
  const int G = n_q_heads / n_kv_heads;
  p.heads_per_tile = G < BLOCK_M ? G : BLOCK_M;
  p.tokens_per_tile = n_splits > 0 ? 1 : BLOCK_M / p.heads_per_tile;
  p.n_head_groups = (G + p.heads_per_tile - 1) / p.heads_per_tile;
  p.split_size = split_size > 0 ? split_size : 1;
  p.n_splits = n_splits;
  const size_t smem = smem_bytes(head_dim);
  dim3 grid(n_work, n_kv_heads * p.n_head_groups, n_splits > 0 ? n_splits : 1);
  int rc = JV_OK;
  JV_DISPATCH_DTYPE(dtype, T, {
    if (n_splits > 0) {
      auto kern = attn_simt_kernel<T, true>;
      static size_t allowed = 0;   // set once per size: the attribute call is kept out of stream captures
      if (smem > allowed) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
          return JV_ERR_UNSUPPORTED;
        allowed = smem;
      }
      kern<<<grid, THREADS, smem, stream>>>(p);
      rc = jv_check_launch();
      if (rc == JV_OK) {
        attn_combine_kernel<T><<<dim3(n_work, n_q_heads), 64, 0, stream>>>(p);
        rc = jv_check_launch();
      }
    } else {
      auto kern = attn_simt_kernel<T, false>;
      static size_t allowed = 0;
      if (smem > allowed) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
          return JV_ERR_UNSUPPORTED;
        allowed = smem;
      }
      kern<<<grid, THREADS, smem, stream>>>(p);
      rc = jv_check_launch();
    }
  });
  return rc;
}
