// Query/key preparation for an attention mixer, fused with the write of new keys and
// values into the paged cache.  One warp handles one head of one token of the packed
// projection output `qkv` ([n, (Hq + 2*Hkv) * D], query heads first, then key heads,
// then value heads):
//
//   query and key heads: optional RMSNorm over the head (weight [D], 32-bit math),
//       then the rotation  u'[j] = u[j]*cos(a_j) - u[j+half]*sin(a_j),
//                          u'[j+half] = u[j+half]*cos(a_j) + u[j]*sin(a_j),
//       a_j = float(position) * inv_freq[j], j < half = rot_dim/2 (the "half-split"
//       pairing); elements from rot_dim on pass through.  Angles, cos and sin are 32-bit.
//   query heads are written back in place; key heads (after norm and rotation) and value
//   heads (untouched) go to the cache slot of the token:
//       page = block_table[entry, position / page_size], slot = position % page_size,
//       cache[page, slot, kv_head, :].
#include "common.cuh"
#include "qk_prepare.cuh"

template <typename T, typename TW>
__global__ void rope_kv_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                               const int* __restrict__ token_entry, const int* __restrict__ block_table,
                               int table_width, const float* __restrict__ inv_freq, int rot_dim,
                               const TW* __restrict__ q_norm_w, const TW* __restrict__ k_norm_w, float eps,
                               T* __restrict__ k_cache, T* __restrict__ v_cache, int n_q_heads,
                               int n_kv_heads, int head_dim, int page_size, int num_pages,
                               int heads_to_do, int* __restrict__ status) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int n = blockIdx.x;
  const int head = blockIdx.y * warps + warp;
  if (head >= heads_to_do) return;
  float* buf = smem + warp * head_dim;

  // which kind of head
  const bool is_q = head < n_q_heads;
  const bool is_k = !is_q && head < n_q_heads + n_kv_heads;
  const int kv_head = is_q ? 0 : (is_k ? head - n_q_heads : head - n_q_heads - n_kv_heads);
  T* src = qkv + (size_t)n * row_stride + (size_t)head * head_dim;
  const int pos = positions[n];

  T* dst = src;
  if (!is_q) {
    const int entry = token_entry[n];
    const int page_idx = pos / page_size;
    const int page = (page_idx < table_width) ? block_table[(size_t)entry * table_width + page_idx] : -1;
    if (page < 0 || page >= num_pages) {
      if (lane == 0) atomicOr(status, JV_STATUS_BAD_PAGE);
      return;
    }
    T* cache = is_k ? k_cache : v_cache;
    dst = cache + (((size_t)page * page_size + (pos % page_size)) * n_kv_heads + kv_head) * head_dim;
  }

  if (!is_q && !is_k) {  // value head: plain copy
    for (int d = lane; d < head_dim; d += 32) dst[d] = src[d];
    return;
  }

  const TW* w = is_q ? q_norm_w : k_norm_w;
  float ss = 0.f;
  for (int d = lane; d < head_dim; d += 32) {
    const float v = to_f32(src[d]);
    buf[d] = v;
    ss += v * v;
  }
  if (w != nullptr) {
    ss = warp_sum(ss);
    const float inv = qk_norm_factor(ss, head_dim, eps);
    for (int d = lane; d < head_dim; d += 32) buf[d] = buf[d] * inv * to_f32(w[d]);
  }
  __syncwarp();
  const int half = rot_dim >> 1;
  for (int d = lane; d < head_dim; d += 32) {
    float v = buf[d];
    if (d < rot_dim) {
      const int j = d < half ? d : d - half;
      float sn, cs, first, second;
      qk_rotation(pos, inv_freq[j], &sn, &cs);
      qk_rotate_pair(buf[j], buf[j + half], cs, sn, &first, &second);
      v = d < half ? first : second;
    }
    dst[d] = from_f32<T>(v);
  }
}

// The common case without shared memory: the whole head rotates (rot_dim == head_dim) and half
// the head is a multiple of 32 (head sizes 64, 128, 256).  A lane holds E = head_dim/64 consecutive
// elements of the first half and their partners of the second half, so norm and rotation stay in
// registers and accesses are E elements wide.
template <typename T, int E> struct alignas(sizeof(T) * E) VecE { T v[E]; };

template <typename T, typename TW, int E>
__global__ void rope_kv_fast_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                                    const int* __restrict__ token_entry, const int* __restrict__ block_table,
                                    int table_width, const float* __restrict__ inv_freq,
                                    const TW* __restrict__ q_norm_w, const TW* __restrict__ k_norm_w, float eps,
                                    T* __restrict__ k_cache, T* __restrict__ v_cache, int n_q_heads,
                                    int n_kv_heads, int page_size, int num_pages, int heads_to_do,
                                    int* __restrict__ status) {
  constexpr int HALF = 32 * E, D = 2 * HALF;
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x;
  const int head = blockIdx.y * (blockDim.x >> 5) + warp;
  if (head >= heads_to_do) return;
  const bool is_q = head < n_q_heads;
  const bool is_k = !is_q && head < n_q_heads + n_kv_heads;
  const int kv_head = is_q ? 0 : (is_k ? head - n_q_heads : head - n_q_heads - n_kv_heads);
  T* src = qkv + (size_t)n * row_stride + (size_t)head * D;
  const int pos = positions[n];
  T* dst = src;
  if (!is_q) {
    const int entry = token_entry[n];
    const int page_idx = pos / page_size;
    const int page = (page_idx < table_width) ? block_table[(size_t)entry * table_width + page_idx] : -1;
    if (page < 0 || page >= num_pages) {
      if (lane == 0) atomicOr(status, JV_STATUS_BAD_PAGE);
      return;
    }
    T* cache = is_k ? k_cache : v_cache;
    dst = cache + (((size_t)page * page_size + (pos - page_idx * page_size)) * n_kv_heads + kv_head) * D;
  }
  using V = VecE<T, E>;
  const int d0 = lane * E;
  V lo = *reinterpret_cast<const V*>(src + d0), hi = *reinterpret_cast<const V*>(src + HALF + d0);
  if (!is_q && !is_k) {
    *reinterpret_cast<V*>(dst + d0) = lo;
    *reinterpret_cast<V*>(dst + HALF + d0) = hi;
    return;
  }
  float a[E], b[E], cs[E], sn[E];
#pragma unroll
  for (int i = 0; i < E; ++i) {
    a[i] = to_f32(lo.v[i]); b[i] = to_f32(hi.v[i]);
    sn[i] = 0.f; cs[i] = 1.f;
    if (inv_freq != nullptr) qk_rotation(pos, inv_freq[d0 + i], &sn[i], &cs[i]);
  }
  const TW* w = is_q ? q_norm_w : k_norm_w;
  qk_prepare_head<E>(a, b, d0, HALF, w != nullptr, eps, [&](int i) { return to_f32(w[i]); }, cs, sn);
#pragma unroll
  for (int i = 0; i < E; ++i) { lo.v[i] = from_f32<T>(a[i]); hi.v[i] = from_f32<T>(b[i]); }
  *reinterpret_cast<V*>(dst + d0) = lo;
  *reinterpret_cast<V*>(dst + HALF + d0) = hi;
}

// The same for many tokens (prompt portions): one block per token takes all its heads, so the token's
// cosines and sines are computed once (not once per head) and its page is looked up once.
template <typename T, typename TW, int E>
__global__ void __launch_bounds__(256) rope_kv_token_kernel(
    T* __restrict__ qkv, int row_stride, const int* __restrict__ positions, const int* __restrict__ token_entry,
    const int* __restrict__ block_table, int table_width, const float* __restrict__ inv_freq,
    const TW* __restrict__ q_norm_w, const TW* __restrict__ k_norm_w, float eps, T* __restrict__ k_cache,
    T* __restrict__ v_cache, int n_q_heads, int n_kv_heads, int page_size, int num_pages, int heads_to_do,
    int* __restrict__ status) {
  constexpr int HALF = 32 * E, D = 2 * HALF;
  __shared__ float cs_s[HALF], sn_s[HALF];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  const int n = blockIdx.x;
  const int pos = positions[n];
  for (int i = threadIdx.x; i < HALF; i += blockDim.x) {
    float sn = 0.f, cs = 1.f;
    if (inv_freq != nullptr) qk_rotation(pos, inv_freq[i], &sn, &cs);
    cs_s[i] = cs; sn_s[i] = sn;
  }
  size_t slot = 0;                       // the token's row in the cache, in units of heads
  bool have_slot = false;
  if (heads_to_do > n_q_heads) {
    const int entry = token_entry[n];
    const int page_idx = pos / page_size;
    const int page = (page_idx < table_width) ? block_table[(size_t)entry * table_width + page_idx] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, JV_STATUS_BAD_PAGE);
    } else {
      slot = ((size_t)page * page_size + (pos - page_idx * page_size)) * n_kv_heads;
      have_slot = true;
    }
  }
  __syncthreads();
  using V = VecE<T, E>;
  const int d0 = lane * E;
  for (int head = warp; head < heads_to_do; head += n_warps) {
    const bool is_q = head < n_q_heads;
    const bool is_k = !is_q && head < n_q_heads + n_kv_heads;
    if (!is_q && !have_slot) continue;
    const int kv_head = is_q ? 0 : (is_k ? head - n_q_heads : head - n_q_heads - n_kv_heads);
    T* src = qkv + (size_t)n * row_stride + (size_t)head * D;
    T* dst = is_q ? src : (is_k ? k_cache : v_cache) + (slot + kv_head) * D;
    V lo = *reinterpret_cast<const V*>(src + d0), hi = *reinterpret_cast<const V*>(src + HALF + d0);
    if (!is_q && !is_k) {
      *reinterpret_cast<V*>(dst + d0) = lo;
      *reinterpret_cast<V*>(dst + HALF + d0) = hi;
      continue;
    }
    float a[E], b[E], cs[E], sn[E];
#pragma unroll
    for (int i = 0; i < E; ++i) {
      a[i] = to_f32(lo.v[i]); b[i] = to_f32(hi.v[i]);
      cs[i] = cs_s[d0 + i]; sn[i] = sn_s[d0 + i];
    }
    const TW* w = is_q ? q_norm_w : k_norm_w;
    qk_prepare_head<E>(a, b, d0, HALF, w != nullptr, eps, [&](int i) { return to_f32(w[i]); }, cs, sn);
#pragma unroll
    for (int i = 0; i < E; ++i) { lo.v[i] = from_f32<T>(a[i]); hi.v[i] = from_f32<T>(b[i]); }
    *reinterpret_cast<V*>(dst + d0) = lo;
    *reinterpret_cast<V*>(dst + HALF + d0) = hi;
  }
}

// qkv: [n, row_stride] of `dtype`; positions, token_entry: [n] int32; block_table:
// [entries, table_width] int32; inv_freq: [rot_dim/2] float; q_norm_w/k_norm_w: [head_dim]
// of `w_dtype` or null; k_cache/v_cache: [num_pages, page_size, n_kv_heads, head_dim] of
// `dtype`, or null when this layer writes no cache (then only query heads are handled).
JV_EXPORT int jv_rope_kv(void* qkv, int dtype, int row_stride, const int* positions,
                         const int* token_entry, const int* block_table, int table_width,
                         const float* inv_freq, int rot_dim, const void* q_norm_w,
                         const void* k_norm_w, int w_dtype, float eps, void* k_cache, void* v_cache,
                         int n, int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                         int num_pages, int* status, cudaStream_t stream) {
  if (n == 0) return JV_OK;
  if (head_dim < 1 || rot_dim > head_dim || (rot_dim & 1) || page_size < 1) return JV_ERR_UNSUPPORTED;
  const int heads_to_do = k_cache ? n_q_heads + 2 * n_kv_heads : n_q_heads;
  const int warps = 4;
  dim3 grid(n, (heads_to_do + warps - 1) / warps);
  const int E = head_dim / 64;
  const bool whole = (rot_dim == head_dim || rot_dim == 0) && (head_dim == 64 || head_dim == 128 || head_dim == 256);
  const int esz = dtype == 0 ? 4 : 2;
  if (whole && (row_stride * esz) % (E * esz) == 0 && ((uintptr_t)qkv % 16) == 0 &&
      (k_cache == nullptr || (((uintptr_t)k_cache % 16) == 0 && ((uintptr_t)v_cache % 16) == 0))) {
    const float* freq = rot_dim ? inv_freq : nullptr;
#define JV_ROPE_FAST(EE)                                                                                   \
    JV_DISPATCH_DTYPE(dtype, T, JV_DISPATCH_DTYPE(w_dtype, TW,                                              \
        return jv_launch(rope_kv_fast_kernel<T, TW, EE>, grid, dim3(warps * 32), 0, stream,                \
            (T*)qkv, row_stride, positions, token_entry, block_table, table_width, freq, (const TW*)q_norm_w, \
            (const TW*)k_norm_w, eps, (T*)k_cache, (T*)v_cache, n_q_heads, n_kv_heads, page_size, num_pages, \
            heads_to_do, status)))
    if (n >= 64) {                       // many tokens: a block per token, the angles once per token
#define JV_ROPE_TOKEN(EE)                                                                                  \
      JV_DISPATCH_DTYPE(dtype, T, JV_DISPATCH_DTYPE(w_dtype, TW,                                            \
          return jv_launch(rope_kv_token_kernel<T, TW, EE>, dim3(n), dim3(256), 0, stream,                 \
              (T*)qkv, row_stride, positions, token_entry, block_table, table_width, freq, (const TW*)q_norm_w, \
              (const TW*)k_norm_w, eps, (T*)k_cache, (T*)v_cache, n_q_heads, n_kv_heads, page_size, num_pages, \
              heads_to_do, status)))
      if (E == 1) JV_ROPE_TOKEN(1); else if (E == 2) JV_ROPE_TOKEN(2); else JV_ROPE_TOKEN(4);
#undef JV_ROPE_TOKEN
      return JV_ERR_UNSUPPORTED;
    }
    if (E == 1) JV_ROPE_FAST(1); else if (E == 2) JV_ROPE_FAST(2); else JV_ROPE_FAST(4);
#undef JV_ROPE_FAST
    return JV_ERR_UNSUPPORTED;
  }
  const size_t smem = (size_t)warps * head_dim * sizeof(float);
  if (smem > 48 * 1024) return JV_ERR_UNSUPPORTED;
  JV_DISPATCH_DTYPE(dtype, T, JV_DISPATCH_DTYPE(w_dtype, TW,
      return jv_launch(rope_kv_kernel<T, TW>, grid, dim3(warps * 32), smem, stream,
          (T*)qkv, row_stride, positions, token_entry, block_table, table_width, inv_freq, rot_dim,
          (const TW*)q_norm_w, (const TW*)k_norm_w, eps, (T*)k_cache, (T*)v_cache, n_q_heads,
          n_kv_heads, head_dim, page_size, num_pages, heads_to_do, status)));
  return JV_ERR_UNSUPPORTED;
}
