// jv_attn_decode_static: the split decode attention of attn_mma.cu with its scratch memory in
// a fixed device array of this library instead of buffers from the caller.  See
// attn_decode_static.h for who needs this and for the rules of use.  The kernels are the ones
// of attn_mma.cu, compiled into this library a second time; nothing of the existing entry
// points changes.
#include "attn_decode_static.h"

#include "attn_mma.cu"

namespace {

constexpr size_t SCRATCH_WORDS = JV_ATTN_STATIC_SCRATCH_BYTES / sizeof(float);
constexpr size_t COUNTER_WORDS = JV_ATTN_STATIC_COUNTERS;            // first part: arrival counters (ints)
constexpr size_t SCRATCH_FLOATS = SCRATCH_WORDS - COUNTER_WORDS;     // rest: partial outputs and (max, sum) pairs

// Arrival counters, then partial outputs and (max, sum) pairs of the key splits.  In host code this
// name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_static_scratch[SCRATCH_WORDS];

constexpr int MAX_DEVICES = JV_MAX_DEVICES;
float* g_scratch_ptr[MAX_DEVICES] = {};   // per device, filled by its first call (two threads racing there store the same value)

// The device address of the scratch array on the current device; null if it cannot be had.
float* scratch_on_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
  if (g_scratch_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    if (cudaGetSymbolAddress((void**)&ptr, g_static_scratch) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    g_scratch_ptr[dev] = ptr;
  }
  return g_scratch_ptr[dev];
}

}  // namespace

extern "C" __attribute__((visibility("default"))) long long jv_attn_decode_static_scratch_floats(
    int n_work, int n_q_heads, int n_splits, int head_dim) {
  return (long long)n_work * n_q_heads * n_splits * (head_dim + 2);
}

extern "C" __attribute__((visibility("default"))) int jv_attn_decode_static(
    const void* q, int q_stride, void* out, int out_stride, const void* k_cache, const void* v_cache,
    const int* block_table, int table_width, const int* cu_seqlens, const int* start_pos, const int* work,
    int n_work, int n_q_heads, int n_kv_heads, int head_dim, int page_size, int num_pages, int window, float scale,
    int split_size, int n_splits, int* status, cudaStream_t stream) {
  if (n_work == 0) return JV_OK;
  if (n_work < 0 || n_splits < 1 || split_size < 1 || n_q_heads < 1) return JV_ERR_UNSUPPORTED;
  if (n_kv_heads < 1 || n_q_heads % n_kv_heads != 0) return JV_ERR_UNSUPPORTED;
  // what jv_attn_mma would refuse is refused here, before anything is enqueued on the stream
  if (!jv_attn_mma_supports(head_dim) || (q_stride % 8) || (out_stride % 2) || ((uintptr_t)q % 16) ||
      ((uintptr_t)k_cache % 16) || ((uintptr_t)v_cache % 16))
    return JV_ERR_UNSUPPORTED;
  const long long need = jv_attn_decode_static_scratch_floats(n_work, n_q_heads, n_splits, head_dim);
  const int G = n_q_heads / n_kv_heads;
  const long long n_counters = (long long)n_work * n_kv_heads * ((G + 15) / 16);
  if (need > (long long)SCRATCH_FLOATS || n_counters > (long long)COUNTER_WORDS)
    return JV_ERR_UNSUPPORTED;   // beyond the fixed array: refused
  float* scratch = scratch_on_current_device();
  if (scratch == nullptr) return 3;
  int* counters = reinterpret_cast<int*>(scratch);
  // the counters must be zero when the kernel starts; it leaves them zero, but a call that failed half
  // way would not, so they are cleared every time (a memset node, not an allocation)
  if (cudaMemsetAsync(counters, 0, (size_t)n_counters * sizeof(int), stream) != cudaSuccess) return JV_ERR_LAUNCH;
  float* part_o = scratch + COUNTER_WORDS;                                     // [n_work*Hq*n_splits][D]
  float* part_ml = part_o + (size_t)n_work * n_q_heads * n_splits * head_dim;  // [n_work*Hq*n_splits][2]
  return jv_attn_mma(q, q_stride, out, out_stride, part_o, part_ml, counters, k_cache, v_cache, block_table, table_width,
                     cu_seqlens, start_pos, work, n_work, n_q_heads, n_kv_heads, head_dim, page_size, num_pages,
                     window, scale, split_size, n_splits, status, stream);
}
