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

template <typename T, typename TW>
__global__ void rope_kv_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                               const int* __restrict__ token_entry, const int* __restrict__ block_table,
                               int table_width, const float* __restrict__ inv_freq, int rot_dim,
                               const TW* __restrict__ q_norm_w, const TW* __restrict__ k_norm_w, float eps,
                               T* __restrict__ k_cache, T* __restrict__ v_cache, int n_q_heads,
                               int n_kv_heads, int head_dim, int page_size, int num_pages,
                               int heads_to_do, int* __restrict__ status) {
  extern __shared__ float smem[];
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
    const float inv = rsqrtf(ss / (float)head_dim + eps);
    for (int d = lane; d < head_dim; d += 32) buf[d] = buf[d] * inv * to_f32(w[d]);
  }
  __syncwarp();
  const int half = rot_dim >> 1;
  for (int d = lane; d < head_dim; d += 32) {
    float v = buf[d];
    if (d < rot_dim) {
      const int j = d < half ? d : d - half;
      const float ang = (float)pos * inv_freq[j];
      float sn, cs;
      sincosf(ang, &sn, &cs);
      const float other = d < half ? -buf[d + half] : buf[d - half];
      v = v * cs + other * sn;
    }
    dst[d] = from_f32<T>(v);
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
  const size_t smem = (size_t)warps * head_dim * sizeof(float);
  if (smem > 48 * 1024) return JV_ERR_UNSUPPORTED;
  JV_DISPATCH_DTYPE(dtype, T, JV_DISPATCH_DTYPE(w_dtype, TW,
      (rope_kv_kernel<T, TW><<<grid, warps * 32, smem, stream>>>(
          (T*)qkv, row_stride, positions, token_entry, block_table, table_width, inv_freq, rot_dim,
          (const TW*)q_norm_w, (const TW*)k_norm_w, eps, (T*)k_cache, (T*)v_cache, n_q_heads,
          n_kv_heads, head_dim, page_size, num_pages, heads_to_do, status))));
  return jv_check_launch();
}
